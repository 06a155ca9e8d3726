"""HF DeBERTa-v2/v3 model patch: same class names as the reference's ``model.py``.

``FlashDisentangledSelfAttention`` keeps the eager module's parameters and signature
(``model.py:34-39`` of the reference, HF ``modeling_deberta_v2.py:191-199``) and replaces its arithmetic by
one fused kernel call.  Differences from the reference module, all on the host side:

* the ``Q.Kr^T`` / ``K.Qr^T`` tensors of ``model.py:122-125,143-148`` are never built; the projected
  relative tables are computed by the library once and cached until a weight changes;
* Q, K, V stay in the ``[B, L, H*D]`` layout the Linear layers produce (no ``transform`` copies,
  ``model.py:70-73,118-120``) and the output is produced directly in ``[B, L, H*D]``;
* the attention mask HF's encoder passes (``[B,1,L,L] = m (x) m^T``) is reduced to per-row key validity
  once per forward (cached on the mask tensor), instead of the per-layer ``sum == numel`` test of
  ``model.py:55-63``; right-padded batches use the padded kernel with lengths, any other token-validity
  pattern goes through pack -> packed kernel -> re-pad (``model.py:138-183``);
* the stray ``print`` of ``model.py:145`` is gone.
"""
from __future__ import annotations

import math
import weakref

import torch
from torch import nn
from transformers.models.deberta_v2.modeling_deberta_v2 import (
    DebertaV2Attention, DebertaV2Encoder, DebertaV2ForMaskedLM, DebertaV2ForMultipleChoice,
    DebertaV2ForQuestionAnswering, DebertaV2ForSequenceClassification, DebertaV2ForTokenClassification,
    DebertaV2Layer, DebertaV2Model, DisentangledSelfAttention)

from . import relpos as _relpos
from .ops.flash_attention import check_pending_status, flash_attention_with_disentangled
from .ops.flash_attention_varlen import flash_attention_with_disentangled_varlen
from .padding import _upad_input, pad_input


class MaskInfo:
    """Key validity derived from an attention mask: lengths, and the packing indices when needed."""
    __slots__ = ("all_ones", "right_padded", "seqlens", "key_mask")

    def __init__(self, all_ones, right_padded, seqlens, key_mask):
        self.all_ones, self.right_padded, self.seqlens, self.key_mask = all_ones, right_padded, seqlens, key_mask


_MASK_CACHE: dict = {}


def analyse_mask(attention_mask: torch.Tensor | None, batch: int, length: int) -> MaskInfo:
    """Reduce a ``[B,L]``, ``[B,L,L]`` or ``[B,1,L,L]`` mask to per-row key validity.

    Costs one device synchronisation (two booleans are read back); the result is cached on the mask
    tensor object (weak reference) and its version, so the 24 layers of one forward share it.  A mask that is not the
    outer product of a token-validity vector (i.e. whose valid queries disagree about the keys) is rejected."""
    if attention_mask is None:
        return MaskInfo(True, True, None, None)
    key = id(attention_mask)
    hit = _MASK_CACHE.get(key)
    if hit is not None:
        ref, version, cached = hit
        if ref() is attention_mask and version == attention_mask._version:     # same live tensor object, unmodified
            return cached
    m = attention_mask
    if m.dim() == 4:
        if m.shape[1] != 1:
            raise ValueError("per-head attention masks are not supported")
        m = m[:, 0]
    if m.dim() == 3:
        full = m != 0
        key_mask = full.any(dim=1)                                  # a key is valid if any query may see it
        query_mask = full.any(dim=2)
        outer = key_mask[:, None, :] & query_mask[:, :, None]
        consistent = torch.equal(outer, full) and torch.equal(key_mask, query_mask)
        if not consistent:
            raise ValueError("attention_mask is not of the form m (x) m^T for a token-validity vector m; "
                             "the fused kernels support token padding masks only")
    elif m.dim() == 2:
        key_mask = m != 0
    else:
        raise ValueError(f"unsupported attention_mask rank {attention_mask.dim()}")
    if key_mask.shape != (batch, length):
        raise ValueError("attention_mask does not match the hidden states")
    seqlens = key_mask.sum(-1, dtype=torch.int32)
    prefix = torch.arange(length, device=key_mask.device)[None, :] < seqlens[:, None]
    flags = torch.stack([key_mask.all(), (prefix == key_mask).all()]).tolist()      # the one sync
    info = MaskInfo(bool(flags[0]), bool(flags[1]), seqlens, key_mask)
    if len(_MASK_CACHE) > 8:
        _MASK_CACHE.clear()
    _MASK_CACHE[key] = (weakref.ref(attention_mask), attention_mask._version, info)
    return info


class FlashDisentangledSelfAttention(DisentangledSelfAttention):
    """Drop-in for HF's ``DisentangledSelfAttention`` running the fused sm_100a kernels."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._tables = None
        self._tables_key = None

    # -- relative tables ---------------------------------------------------------------------------
    def _relative_tables(self, rel_embeddings: torch.Tensor, dtype: torch.dtype):
        c2p, p2c = "c2p" in self.pos_att_type, "p2c" in self.pos_att_type
        if not self.relative_attention or not (c2p or p2c) or rel_embeddings is None:
            return None
        if self.share_att_key:
            kp, qp = self.key_proj, self.query_proj
        else:
            kp = self.pos_key_proj if c2p else None
            qp = self.pos_query_proj if p2c else None
        stamp = getattr(rel_embeddings, "_tdb_stamp", None)
        params = [t for lin in (kp, qp) if lin is not None for t in (lin.weight, lin.bias) if t is not None]
        key = (stamp, dtype, rel_embeddings.device, tuple((t.data_ptr(), t._version) for t in params))
        if stamp is not None and self._tables is not None and self._tables_key == key:
            return self._tables
        rel = rel_embeddings.detach().to(dtype)
        tables = _relpos.build_tables(
            rel, num_heads=self.num_attention_heads, position_buckets=self.position_buckets,
            max_relative_positions=self.max_relative_positions,
            key_weight=None if kp is None else kp.weight.detach(), key_bias=None if kp is None else kp.bias,
            query_weight=None if qp is None else qp.weight.detach(), query_bias=None if qp is None else qp.bias,
            c2p=c2p, p2c=p2c)
        if stamp is not None:
            self._tables, self._tables_key = tables, key
        return tables

    # -- forward ------------------------------------------------------------------------------------
    def forward(self, hidden_states, attention_mask, output_attentions=False, query_states=None,
                relative_pos=None, rel_embeddings=None):
        """Same contract as the reference (``model.py:34-186``): returns ``(context [B, L, H*D], None)``.
        ``relative_pos`` is accepted and ignored (positions are implied by the token order), and attention
        probabilities are never materialised, so the second element is always None."""
        if query_states is None:
            query_states = hidden_states
        B, L, _ = hidden_states.shape
        if query_states.shape[1] != L:
            raise NotImplementedError("query and key lengths must match (encoder self-attention)")
        H, D = self.num_attention_heads, self.attention_head_size
        q = self.query_proj(query_states).view(B, L, H, D)
        k = self.key_proj(hidden_states).view(B, L, H, D)
        v = self.value_proj(hidden_states).view(B, L, H, D)
        scale_factor = 1 + int("c2p" in self.pos_att_type) + int("p2c" in self.pos_att_type)
        sm_scale = 1.0 / math.sqrt(D * scale_factor)
        tables = None
        if self.relative_attention:
            rel_embeddings = self.pos_dropout(rel_embeddings)
            tables = self._relative_tables(rel_embeddings, q.dtype)
        info = analyse_mask(attention_mask, B, L)
        buckets = self.position_buckets if self.relative_attention else 0
        max_rel = self.max_relative_positions if self.relative_attention else 0
        if info.all_ones or info.right_padded:
            out = flash_attention_with_disentangled(
                q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), None, None, False, sm_scale,
                buckets, max_rel, seqlens=None if info.all_ones else info.seqlens, tables=tables,
                check_status=False)
            out = out.transpose(1, 2).reshape(B, L, H * D)
        else:
            (qu, ku, vu, _, _, indices, (cu_q, cu_k), (max_q, max_k)) = _upad_input(
                q, k, v, None, None, info.key_mask, L, H)
            out_unpad = flash_attention_with_disentangled_varlen(
                qu, ku, vu, None, None, cu_q, cu_k, max_q, max_k, False, sm_scale, buckets, max_rel, tables=tables,
                check_status=False)
            out = pad_input(out_unpad, indices, B, L).reshape(B, L, H * D)
        return (out, None)


class FlashDebertaV2Attention(DebertaV2Attention):
    def __init__(self, config):
        super().__init__(config)
        self.self = FlashDisentangledSelfAttention(config)


class FlashDebertaV2Layer(DebertaV2Layer):
    def __init__(self, config):
        super().__init__(config)
        self.attention = FlashDebertaV2Attention(config)


class FlashDebertaV2Encoder(DebertaV2Encoder):
    """HF encoder whose layers use the fused attention.  Two host-side savings: the ``[L, L]`` relative
    position matrix is not built (the kernels do not read it), and in eval mode the LayerNorm'd relative
    embeddings are computed once and stamped so that every layer can keep its derived tables."""

    def __init__(self, config):
        super().__init__(config)
        self.layer = nn.ModuleList([FlashDebertaV2Layer(config) for _ in range(config.num_hidden_layers)])
        self._rel_cache = None
        self._rel_cache_key = None
        self._rel_stamp = 0

    def get_rel_pos(self, hidden_states, query_states=None, relative_pos=None):
        return relative_pos

    def forward(self, *args, **kwargs):
        out = super().forward(*args, **kwargs)
        check_pending_status()          # one synchronisation per encoder forward instead of one per layer
        return out

    def get_rel_embedding(self):
        if not self.relative_attention:
            return None
        params = [self.rel_embeddings.weight]
        if "layer_norm" in self.norm_rel_ebd:
            params += [self.LayerNorm.weight, self.LayerNorm.bias]
        if self.training or torch.is_grad_enabled():
            return super().get_rel_embedding()
        key = tuple((t.data_ptr(), t._version, t.dtype, t.device) for t in params)
        if self._rel_cache is None or key != self._rel_cache_key:
            rel = super().get_rel_embedding().detach()
            self._rel_stamp += 1
            rel._tdb_stamp = (id(self), self._rel_stamp)
            self._rel_cache, self._rel_cache_key = rel, key
        return self._rel_cache


class FlashDebertaV2Model(DebertaV2Model):
    def __init__(self, config):
        super().__init__(config)
        self.encoder = FlashDebertaV2Encoder(config)
        self.post_init()


def patch_model(model: nn.Module) -> nn.Module:
    """Swap, in place, every eager ``DisentangledSelfAttention`` of an already built HF DeBERTa-v2 model for
    the fused module (parameters are shared, not copied) and give its encoder the cached relative embeddings."""
    for name, mod in list(model.named_modules()):
        if isinstance(mod, DebertaV2Attention) and not isinstance(mod.self, FlashDisentangledSelfAttention):
            old = mod.self
            new = FlashDisentangledSelfAttention.__new__(FlashDisentangledSelfAttention)
            new.__dict__.update(old.__dict__)
            new._tables, new._tables_key = None, None
            mod.self = new
        if type(mod) is DebertaV2Encoder:
            mod.__class__ = FlashDebertaV2Encoder
            mod._rel_cache, mod._rel_cache_key, mod._rel_stamp = None, None, 0
    return model


class FlashDebertaV2ForMaskedLM(DebertaV2ForMaskedLM):
    def __init__(self, config):
        super().__init__(config)
        self.deberta = FlashDebertaV2Model(config)
        self.post_init()


class FlashDebertaV2ForSequenceClassification(DebertaV2ForSequenceClassification):
    def __init__(self, config):
        super().__init__(config)
        self.deberta = FlashDebertaV2Model(config)
        self.post_init()


class FlashDebertaV2ForTokenClassification(DebertaV2ForTokenClassification):
    def __init__(self, config):
        super().__init__(config)
        self.deberta = FlashDebertaV2Model(config)
        self.post_init()


class FlashDebertaV2ForQuestionAnswering(DebertaV2ForQuestionAnswering):
    def __init__(self, config):
        super().__init__(config)
        self.deberta = FlashDebertaV2Model(config)
        self.post_init()


class FlashDebertaV2ForMultipleChoice(DebertaV2ForMultipleChoice):
    def __init__(self, config):
        super().__init__(config)
        self.deberta = FlashDebertaV2Model(config)
        self.post_init()
