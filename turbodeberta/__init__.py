"""Import-path alias: the module layout of the reference package (``turbodeberta.model``,
``turbodeberta.ops.flash_attention``, ``turbodeberta.ops.flash_attention_varlen``, ``turbodeberta.padding``) backed by
the sm_100a implementation in ``turbodeberta_b200``.  Code written against the reference imports unchanged."""
