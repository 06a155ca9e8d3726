"""Pack / unpack glue between padded ``[B, L, ...]`` batches and the packed ``[T, ...]`` token stream.

Same function names, argument order and return conventions as the reference's ``padding.py``
(``index_first_axis`` :76, ``pad_input`` :30-44, ``_get_unpad_data`` :79-88, ``unpad_input`` :90-111,
``_upad_input`` :113-166).  Two differences: plain tensor indexing replaces the hand-written autograd
functions (the path is forward-only), and the relative-position arguments of ``_upad_input`` are the
projected tables, which are per layer rather than per token and therefore pass through untouched.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def index_first_axis(x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """Rows ``indices`` of ``x`` along the first axis (``padding.py:76``)."""
    if x.dim() < 2:
        raise ValueError("index_first_axis expects at least 2 dimensions")
    return x.index_select(0, indices)


def index_put_first_axis(values: torch.Tensor, indices: torch.Tensor, first_axis_dim: int) -> torch.Tensor:
    """Zero tensor with ``first_axis_dim`` rows whose rows ``indices`` are ``values`` (``padding.py:28``)."""
    if indices.dim() != 1 or values.dim() < 2:
        raise ValueError("index_put_first_axis expects 1-D indices and values with at least 2 dimensions")
    out = torch.zeros(first_axis_dim, *values.shape[1:], device=values.device, dtype=values.dtype)
    out.index_copy_(0, indices, values)
    return out


def pad_input(hidden_states: torch.Tensor, indices: torch.Tensor, batch: int, seqlen: int) -> torch.Tensor:
    """``(total_nnz, ...)`` -> ``(batch, seqlen, ...)`` with zeros at the padded positions (``padding.py:30-44``)."""
    out = index_put_first_axis(hidden_states, indices, batch * seqlen)
    return out.view(batch, seqlen, *hidden_states.shape[1:])


def _get_unpad_data(attention_mask: torch.Tensor):
    """``(indices, cu_seqlens, max_seqlen_in_batch)`` of a 2-D validity mask (``padding.py:79-88``).
    ``max_seqlen_in_batch`` is a Python int, which costs one device synchronisation, as in the reference."""
    if attention_mask.dim() != 2:
        raise ValueError("expected a [batch, seqlen] validity mask")
    seqlens = attention_mask.sum(dim=-1, dtype=torch.int32)
    indices = torch.nonzero(attention_mask.flatten(), as_tuple=False).flatten()
    max_seqlen = int(seqlens.max().item()) if seqlens.numel() else 0
    cu_seqlens = F.pad(torch.cumsum(seqlens, dim=0, dtype=torch.int32), (1, 0))
    return indices, cu_seqlens, max_seqlen


def unpad_input(hidden_states: torch.Tensor, attention_mask: torch.Tensor):
    """``(batch, seqlen, ...)`` -> ``(tokens, indices, cu_seqlens, max_seqlen_in_batch)`` (``padding.py:90-111``)."""
    indices, cu_seqlens, max_seqlen = _get_unpad_data(attention_mask)
    flat = hidden_states.reshape(-1, *hidden_states.shape[2:])
    return index_first_axis(flat, indices), indices, cu_seqlens, max_seqlen


def _upad_input(query_layer, key_layer, value_layer, pos_key, pos_query, attention_mask, query_length, NH):
    """Unpad Q, K, V ``[B, L, H, D]`` for self-attention (``padding.py:113-166``).

    Returns ``(q, k, v, pos_key, pos_query, indices_q, (cu_q, cu_k), (max_q, max_k))``.  Only the
    equal-length branch (``padding.py:130-142``) exists here: the fused kernels are self-attention only.
    ``pos_key`` / ``pos_query`` are returned unchanged (they are tables, not per-token tensors)."""
    batch, kv_len, n_heads, head_dim = key_layer.shape
    if query_length != kv_len or query_layer.shape[1] != kv_len:
        raise NotImplementedError("query and key lengths must match (encoder self-attention)")
    if n_heads != NH:
        raise ValueError("head count mismatch")
    indices, cu_seqlens, max_seqlen = _get_unpad_data(attention_mask)
    q = index_first_axis(query_layer.reshape(batch * kv_len, NH, head_dim), indices)
    k = index_first_axis(key_layer.reshape(batch * kv_len, n_heads, head_dim), indices)
    v = index_first_axis(value_layer.reshape(batch * kv_len, n_heads, head_dim), indices)
    return q, k, v, pos_key, pos_query, indices, (cu_seqlens, cu_seqlens), (max_seqlen, max_seqlen)
