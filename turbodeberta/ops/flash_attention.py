"""``turbodeberta.ops.flash_attention`` of the reference (``src/turbodeberta/ops/flash_attention.py:345-369``)."""
from turbodeberta_b200.ops.flash_attention import check_pending_status, flash_attention_with_disentangled  # noqa: F401
