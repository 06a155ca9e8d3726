"""``turbodeberta.padding`` of the reference (``src/turbodeberta/padding.py``), served by ``turbodeberta_b200.padding``."""
from turbodeberta_b200.padding import (  # noqa: F401
    _get_unpad_data, _upad_input, index_first_axis, index_put_first_axis, pad_input, unpad_input)
