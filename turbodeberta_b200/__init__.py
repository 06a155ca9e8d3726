"""turbodeberta_b200: B200 (sm_100a) fused disentangled self-attention for DeBERTa-v2/v3.

Module paths mirror the reference package (``turbodeberta``): ``.ops.flash_attention``,
``.ops.flash_attention_varlen``, ``.padding`` and ``.model``.  Importing the ops loads the
C-ABI library ``libtdb_b200.so`` and fails loudly when it has not been built.
"""
__version__ = "0.1.0"
