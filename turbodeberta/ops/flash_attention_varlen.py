"""``turbodeberta.ops.flash_attention_varlen`` of the reference
(``src/turbodeberta/ops/flash_attention_varlen.py:348-374``)."""
from turbodeberta_b200.ops.flash_attention_varlen import flash_attention_with_disentangled_varlen  # noqa: F401
