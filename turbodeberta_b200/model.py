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
import warnings
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
from .padding import _get_unpad_data, _upad_input, index_first_axis, pad_input


class PackedSequences:
    """Stands in for the attention mask when the encoder runs on the packed token stream: hidden states are
    ``[1, T, hidden]`` with the sequences back to back, ``cu_seqlens`` (int32 ``[n_seqs + 1]``) marks them."""
    __slots__ = ("cu_seqlens", "max_seqlen")

    def __init__(self, cu_seqlens: torch.Tensor, max_seqlen: int):
        self.cu_seqlens, self.max_seqlen = cu_seqlens, int(max_seqlen)


class MaskInfo:
    """Key validity derived from an attention mask: lengths, and the packing indices when needed."""
    __slots__ = ("all_ones", "right_padded", "seqlens", "key_mask")

    def __init__(self, all_ones, right_padded, seqlens, key_mask):
        self.all_ones, self.right_padded, self.seqlens, self.key_mask = all_ones, right_padded, seqlens, key_mask


_MASK_CACHE: dict = {}


def _mask_cache_put(tensor: torch.Tensor, info) -> None:
    """Remember the analysis of a live mask tensor.  Entries of tensors that have been freed are dropped first; only
    if more than 64 live masks are tracked does the oldest entry go (so a mask that is passed again and again, e.g.
    the static input of a captured graph, is never re-analysed because other masks came and went)."""
    dead = [k for k, (ref, _, _) in _MASK_CACHE.items() if ref() is None]
    for k in dead:
        del _MASK_CACHE[k]
    while len(_MASK_CACHE) >= 64:
        del _MASK_CACHE[next(iter(_MASK_CACHE))]
    _MASK_CACHE[id(tensor)] = (weakref.ref(tensor), tensor._version, info)


def analyse_mask(attention_mask: torch.Tensor | None, batch: int, length: int, refresh: bool = False) -> MaskInfo:
    """Reduce a ``[B,L]``, ``[B,L,L]`` or ``[B,1,L,L]`` mask to per-row key validity.

    The first analysis of a mask costs one device synchronisation (two booleans are read back: all ones? right
    padded?); the result is cached on the mask tensor object (weak reference) and its version, so the 24 layers of
    one forward share it.  A mask that is not the outer product of a token-validity vector (i.e. whose valid queries
    disagree about the keys) is rejected.

    ``refresh=True`` (what the encoder passes once per forward) keeps the cached pair of booleans but recomputes the
    length and validity tensors from the mask with synchronisation-free operations.  Inside a CUDA-graph capture that
    puts the recomputation into the graph: replays then follow the lengths currently in the (static) mask buffer,
    while the choice between the all-ones, right-padded and packed routes stays the one made at capture."""
    if attention_mask is None:
        return MaskInfo(True, True, None, None)
    key = id(attention_mask)
    hit = _MASK_CACHE.get(key)
    flags = None
    if hit is not None:
        ref, version, cached = hit
        if ref() is attention_mask and version == attention_mask._version:     # same live tensor object, unmodified
            if not refresh:
                return cached
            flags = (cached.all_ones, cached.right_padded)
    m = attention_mask
    if m.dim() == 4:
        if m.shape[1] != 1:
            raise ValueError("per-head attention masks are not supported")
        m = m[:, 0]
    if m.dim() == 3:
        full = m != 0
        key_mask = full.any(dim=1)                                  # a key is valid if any query may see it
        if flags is None:
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
    if flags is None:
        prefix = torch.arange(length, device=key_mask.device)[None, :] < seqlens[:, None]
        flags = torch.stack([key_mask.all(), (prefix == key_mask).all()]).tolist()      # the one sync
    info = MaskInfo(bool(flags[0]), bool(flags[1]), seqlens, key_mask)
    _mask_cache_put(attention_mask, info)
    return info


_WARNED: set = set()


def _warn_once(key: str, message: str) -> None:
    if key not in _WARNED:
        _WARNED.add(key)
        warnings.warn(message, stacklevel=3)


class FlashDisentangledSelfAttention(DisentangledSelfAttention):
    """Drop-in for HF's ``DisentangledSelfAttention`` running the fused sm_100a kernels."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._tables = None
        self._tables_key = None
        self._qkv = None
        self._qkv_key = None

    # -- fused Q/K/V projection ------------------------------------------------------------------
    def _project_qkv(self, hidden_states: torch.Tensor, query_states: torch.Tensor):
        """Q, K, V as ``[..., H, D]`` views.  For inference self-attention the three Linear layers run as one GEMM
        over a cached concatenation of their weights (rebuilt when a weight changes); the result is consumed through
        strided views, so no copy follows.  With gradients enabled, or a separate query input, the layers run as is."""
        H, D = self.num_attention_heads, self.attention_head_size
        lead = hidden_states.shape[:-1]
        if query_states is hidden_states and not torch.is_grad_enabled():
            params = (self.query_proj.weight, self.query_proj.bias, self.key_proj.weight, self.key_proj.bias,
                      self.value_proj.weight, self.value_proj.bias)
            key = tuple((t.data_ptr(), t._version, t.dtype, t.device) for t in params)
            if self._qkv is None or self._qkv_key != key:
                w = torch.cat([params[0], params[2], params[4]], 0).detach()
                b = torch.cat([params[1], params[3], params[5]], 0).detach()
                self._qkv, self._qkv_key = (w, b), key
            qkv = torch.nn.functional.linear(hidden_states, *self._qkv).view(*lead, 3, H, D)
            return qkv.select(-3, 0), qkv.select(-3, 1), qkv.select(-3, 2)
        q = self.query_proj(query_states).view(*query_states.shape[:-1], H, D)
        k = self.key_proj(hidden_states).view(*lead, H, D)
        v = self.value_proj(hidden_states).view(*lead, H, D)
        return q, k, v

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
        if self.training and float(getattr(self.dropout, "p", 0.0)) > 0.0:
            _warn_once("dropout", "the fused attention has no dropout on the attention probabilities (neither has the "
                       "reference's kernel) and no backward pass: attention_probs_dropout_prob is ignored")
        q, k, v = self._project_qkv(hidden_states, query_states)
        if q.dtype == torch.float32 and B * L >= 4096:
            _warn_once("fp32", "float32 inputs run on the exact CUDA-core attention kernel (one warp per query row), "
                       "which is a correctness mode and far slower than the bf16 tensor-core kernel; "
                       "convert the model with .bfloat16() for throughput")
        scale_factor = 1 + int("c2p" in self.pos_att_type) + int("p2c" in self.pos_att_type)
        sm_scale = 1.0 / math.sqrt(D * scale_factor)
        tables = None
        if self.relative_attention:
            rel_embeddings = self.pos_dropout(rel_embeddings)
            tables = self._relative_tables(rel_embeddings, q.dtype)
        buckets = self.position_buckets if self.relative_attention else 0
        max_rel = self.max_relative_positions if self.relative_attention else 0
        if isinstance(attention_mask, PackedSequences):                  # packed stream from the encoder: [1, T, hidden]
            cu = attention_mask.cu_seqlens
            out = flash_attention_with_disentangled_varlen(
                q[0], k[0], v[0], None, None, cu, cu, attention_mask.max_seqlen, attention_mask.max_seqlen, False,
                sm_scale, buckets, max_rel, tables=tables, check_status=False)
            return (out.reshape(1, L, H * D), None)
        info = analyse_mask(attention_mask, B, L)
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

    #: run padded batches on the packed token stream (unpad once after the embeddings, re-pad once at the end)
    pack_padded_batches = True
    #: with packing, re-pad only the last layer's output; earlier entries of ``hidden_states`` stay ``[1, T, hidden]``
    skip_intermediate_padding = False

    def forward(self, hidden_states, attention_mask, output_hidden_states=True, output_attentions=False,
                query_states=None, relative_pos=None, return_dict=True):
        self._mask_info = None
        if (query_states is None and self.conv is None and not output_attentions
                and hidden_states.is_cuda and hidden_states.dim() == 3):
            # One analysis of the user's mask per forward (cached per mask tensor, so a repeated call with the same
            # tensor - e.g. while the forward is being captured into a CUDA graph - costs no synchronisation); the
            # expanded mask that the HF encoder builds from it inherits the result in get_attention_mask().
            info = analyse_mask(attention_mask, hidden_states.shape[0], hidden_states.shape[1], refresh=True)
            if self.pack_padded_batches and not info.all_ones:
                out = self._forward_packed(hidden_states, info, output_hidden_states, return_dict)
                self._check_status_unless_capturing()
                return out
            self._mask_info = info
        out = super().forward(hidden_states, attention_mask, output_hidden_states=output_hidden_states,
                              output_attentions=output_attentions, query_states=query_states,
                              relative_pos=relative_pos, return_dict=return_dict)
        self._check_status_unless_capturing()   # one synchronisation per encoder forward instead of one per layer
        return out

    def get_attention_mask(self, attention_mask):
        out = super().get_attention_mask(attention_mask)
        info = getattr(self, "_mask_info", None)
        if info is not None and isinstance(out, torch.Tensor) and out is not attention_mask:
            _mask_cache_put(out, info)
        return out

    @staticmethod
    def _check_status_unless_capturing():
        """Reading the device status words synchronises, which a stream capture does not allow: while the forward is
        being captured into a CUDA graph the words stay pending (the graph's replays rewrite them) and the next
        ``check_pending_status()`` outside a capture reads them."""
        if not torch.cuda.is_current_stream_capturing():
            check_pending_status()

    def _forward_packed(self, hidden_states, info: MaskInfo, output_hidden_states: bool, return_dict: bool):
        """The layer loop of the HF encoder (``modeling_deberta_v2.py:630-682``) on valid tokens only.  The reference
        packs and re-pads inside every attention call (``model.py:157-183``); here the whole stack (attention, both
        projections, FFN, LayerNorms) sees ``[1, T, hidden]`` and padding costs nothing.  Padded positions of the
        returned tensors are zero."""
        from transformers.modeling_outputs import BaseModelOutput
        B, L, hid = hidden_states.shape
        indices, cu_seqlens, max_seqlen = _get_unpad_data(info.key_mask)
        x = index_first_axis(hidden_states.reshape(B * L, hid), indices)[None]
        seqs = PackedSequences(cu_seqlens, max_seqlen)
        rel_embeddings = self.get_rel_embedding()
        all_hidden = (hidden_states,) if output_hidden_states else None
        n = len(self.layer)
        for i, layer in enumerate(self.layer):
            x, _ = layer(x, seqs, query_states=None, relative_pos=None, rel_embeddings=rel_embeddings,
                         output_attentions=False)
            if output_hidden_states:
                last = i == n - 1
                all_hidden = all_hidden + ((pad_input(x[0], indices, B, L) if (last or not self.skip_intermediate_padding)
                                            else x),)
        output_states = all_hidden[-1] if output_hidden_states else pad_input(x[0], indices, B, L)
        if not return_dict:
            return tuple(v for v in [output_states, all_hidden, None] if v is not None)
        return BaseModelOutput(last_hidden_state=output_states, hidden_states=all_hidden, attentions=None)

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
            new._tables, new._tables_key, new._qkv, new._qkv_key = None, None, None, None
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
