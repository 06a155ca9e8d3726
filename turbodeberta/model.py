"""``turbodeberta.model`` of the reference (``src/turbodeberta/model.py``): the same class names, served by
``turbodeberta_b200.model``."""
from turbodeberta_b200.model import (  # noqa: F401
    FlashDebertaV2Attention, FlashDebertaV2Encoder, FlashDebertaV2ForMaskedLM, FlashDebertaV2ForMultipleChoice,
    FlashDebertaV2ForQuestionAnswering, FlashDebertaV2ForSequenceClassification, FlashDebertaV2ForTokenClassification,
    FlashDebertaV2Layer, FlashDebertaV2Model, FlashDisentangledSelfAttention, patch_model)
