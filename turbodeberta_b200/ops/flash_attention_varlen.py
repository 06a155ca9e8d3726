"""Packed (varlen) fused disentangled attention.

Same entry point as the reference's ``ops/flash_attention_varlen.py:348-374``::

    flash_attention_with_disentangled_varlen(q, k, v, q_pos, k_pos, cu_seqlens_q, cu_seqlens_k,
                                             max_seqlen_q, max_seqlen_k, causal=False, sm_scale=None,
                                             position_buckets=0, max_relative_distance=0)

q, k, v are ``(T, H, D)`` with the sequences back to back; ``cu_seqlens`` is int32 ``(n_seqs + 1)``.  As in the
fixed-length op, ``q_pos``/``k_pos`` are the projected tables ``(H, 2*span, D)`` rather than the per-token score
tensors ``(T, H, 2*span)`` of the reference.  Relative positions restart at every sequence.  The tile list is
built on the device from ``cu_seqlens``; nothing is read back except the status words at the end of the call.
Score tensors of shape ``(T, H, 2*span)`` are still accepted and gathered by a CUDA-core compatibility kernel
(``p2c_mirrored=True`` reproduces the reference kernel's index, ``ops/flash_attention_varlen.py:144-152``).
"""
from __future__ import annotations

import math

import torch

from .. import _cabi as cabi
from .flash_attention import (_PENDING_STATUS, _check_status, _index_table_for_scores, _is_materialised,
                              _tables_from_args, refuse_gradients)


class _VarlenFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, tables, cu_seqlens, max_seqlen, sm_scale, kernel, return_lse, check, cu_seqlens_k=None):
        dev = cabi.require_cuda(q, k, v, cu_seqlens)
        if q.dim() != 3 or k.shape != q.shape or v.shape != q.shape:
            raise ValueError("q, k, v must share the shape (T, H, D)")
        T, H, D = q.shape
        if not (q.dtype == k.dtype == v.dtype):
            raise ValueError("q, k, v must share a dtype")
        code = cabi.dtype_code(q.dtype)
        for t in (q, k, v):
            if t.stride(-1) != 1:
                raise ValueError("the head dimension must be contiguous")
        if cu_seqlens.dtype != torch.int32 or cu_seqlens.dim() != 1 or cu_seqlens.numel() < 1:
            raise ValueError("cu_seqlens must be a 1-D int32 tensor of n_seqs + 1 offsets")
        cu_seqlens = cu_seqlens.contiguous()
        n_seqs = cu_seqlens.numel() - 1
        o = torch.empty((T, H, D), dtype=q.dtype, device=dev)
        if T == 0 or n_seqs == 0:                    # nothing to compute
            st = torch.zeros(4, dtype=torch.int32, device=dev)
            return (o, torch.empty((H, T), dtype=torch.float32, device=dev) if return_lse else None, st)
        lse = torch.empty((H, T), dtype=torch.float32, device=dev) if return_lse else None
        status = torch.zeros(4, dtype=torch.int32, device=dev)
        ws_bytes = int(cabi.lib.tdb_attn_workspace_bytes(n_seqs, T))
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
        flags = 0
        kr = qr = idx = kr_exp = qr_exp = None
        two_span = idm = edm = erows = 0
        if tables is not None:
            kr, qr, idx, kr_exp, qr_exp = tables.kr, tables.qr, tables.idx, tables.kr_exp, tables.qr_exp
            two_span, idm, edm, erows = tables.two_span, tables.idx_delta_max, tables.exp_delta_max, tables.exp_rows
            flags = (cabi.TDB_FLAG_C2P if kr is not None else 0) | (cabi.TDB_FLAG_P2C if qr is not None else 0)
            for t in (kr, qr):
                if t is not None and t.dtype != q.dtype:
                    raise ValueError("relative tables must have the dtype of q")
        with torch.cuda.device(dev):
            rc = cabi.lib.tdb_attn_fwd_varlen(
                cabi.ptr(q), cabi.ptr(k), cabi.ptr(v), cabi.ptr(o),
                q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1), o.stride(0), o.stride(1),
                cabi.ptr(kr), cabi.ptr(qr), two_span, cabi.ptr(idx), idm, cabi.ptr(kr_exp), cabi.ptr(qr_exp), edm, erows,
                cabi.ptr(cu_seqlens), n_seqs, T, int(max_seqlen), H, D, float(sm_scale), flags, code, kernel,
                cabi.ptr(ws), ws_bytes, cabi.ptr(lse), cabi.ptr(status), cabi.stream_ptr(dev))
        cabi.check(rc)
        _flag_offset_mismatch(status, cu_seqlens, cu_seqlens_k)
        if check:
            _check_status(status)
        else:
            _PENDING_STATUS.append(status)
        ctx.mark_non_differentiable(status)
        if lse is not None:
            ctx.mark_non_differentiable(lse)
        return (o, lse, status)

    @staticmethod
    def backward(ctx, *grads):
        raise RuntimeError("turbodeberta_b200 attention is forward-only (as in the reference: no backward kernel)")


def _flag_offset_mismatch(status, cu_q, cu_k) -> None:
    """Self-attention only: key offsets must equal the query offsets.  When the caller passes two different tensors
    the comparison runs on the device and lands in status word 1 (the malformed-offsets word), so the call itself
    never waits for the GPU."""
    if cu_k is None or cu_k is cu_q or (cu_k.data_ptr() == cu_q.data_ptr() and cu_k.shape == cu_q.shape):
        return
    status[1:2].add_((cu_k.to(cu_q.device) != cu_q).any().to(torch.int32))


def _scores_varlen(q, k, v, c2p_scores, p2c_scores, cu_seqlens, max_seqlen, sm_scale, position_buckets,
                   max_relative_distance, p2c_mirrored, return_lse, check_status, cu_seqlens_k=None):
    """Legacy form of the packed op: gather from materialised ``(T, H, 2*span)`` score tensors."""
    dev = cabi.require_cuda(q, k, v, cu_seqlens)
    refuse_gradients(q, k, v, c2p_scores, p2c_scores)
    if q.dim() != 3 or k.shape != q.shape or v.shape != q.shape:
        raise ValueError("q, k, v must share the shape (T, H, D)")
    T, H, D = q.shape
    code = cabi.dtype_code(q.dtype)
    some = c2p_scores if c2p_scores is not None else p2c_scores
    two_span = some.shape[-1]
    for t, name in ((c2p_scores, "q_pos"), (p2c_scores, "k_pos")):
        if t is not None and (tuple(t.shape) != (T, H, two_span) or t.dtype != q.dtype or t.stride(-1) != 1):
            raise ValueError(f"{name} must be (T, H, 2*span) of q's dtype with a contiguous last dimension")
    for t in (q, k, v):
        if t.stride(-1) != 1:
            raise ValueError("the head dimension must be contiguous")
    if cu_seqlens.dtype != torch.int32 or cu_seqlens.dim() != 1 or cu_seqlens.numel() < 1:
        raise ValueError("cu_seqlens must be a 1-D int32 tensor of n_seqs + 1 offsets")
    cu_seqlens = cu_seqlens.contiguous()
    n_seqs = cu_seqlens.numel() - 1
    idx, idm = _index_table_for_scores(two_span, position_buckets, max_relative_distance, dev)
    o = torch.empty((T, H, D), dtype=q.dtype, device=dev)
    lse = torch.empty((H, T), dtype=torch.float32, device=dev) if return_lse else None
    if T == 0 or n_seqs == 0:
        return o, lse
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    flags = ((cabi.TDB_FLAG_C2P if c2p_scores is not None else 0) | (cabi.TDB_FLAG_P2C if p2c_scores is not None else 0)
             | (cabi.TDB_FLAG_P2C_MIRRORED if p2c_mirrored else 0))

    def s(t):
        return (t.stride(0), t.stride(1)) if t is not None else (0, 0)

    with torch.cuda.device(dev):
        rc = cabi.lib.tdb_attn_fwd_varlen_scores(
            cabi.ptr(q), cabi.ptr(k), cabi.ptr(v), cabi.ptr(o), *s(q), *s(k), *s(v), *s(o),
            cabi.ptr(c2p_scores), *s(c2p_scores), cabi.ptr(p2c_scores), *s(p2c_scores), two_span, cabi.ptr(idx), idm,
            cabi.ptr(cu_seqlens), n_seqs, T, max_seqlen, H, D, float(sm_scale), flags, code, cabi.ptr(lse),
            cabi.ptr(status), cabi.stream_ptr(dev))
    cabi.check(rc)
    _flag_offset_mismatch(status, cu_seqlens, cu_seqlens_k)
    if check_status:
        _check_status(status)
    else:
        _PENDING_STATUS.append(status)
    return o, lse


def flash_attention_with_disentangled_varlen(q, k, v, q_pos, k_pos, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                                             max_seqlen_k, causal=False, sm_scale=None, position_buckets=0,
                                             max_relative_distance=0, *, tables=None, kernel=cabi.TDB_KERNEL_AUTO,
                                             return_lse=False, check_status=True, p2c_mirrored=False):
    """Fused disentangled attention on packed ``(T, H, D)`` inputs; returns ``o`` of the same shape."""
    if causal:
        raise NotImplementedError("causal masking is not part of the DeBERTa encoder path")
    if cu_seqlens_k is not None and cu_seqlens_k is not cu_seqlens_q:
        if cu_seqlens_k.shape != cu_seqlens_q.shape or cu_seqlens_k.dtype != cu_seqlens_q.dtype:
            raise ValueError("query and key offsets must be equal: only self-attention is supported")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    T = q.shape[0]
    max_seqlen = max(int(max_seqlen_q), int(max_seqlen_k if max_seqlen_k is not None else max_seqlen_q))
    max_seqlen = max(1, min(max_seqlen, T)) if T > 0 else 1
    mat = lambda t: _is_materialised(t, q, position_buckets, max_relative_distance)
    if tables is None and (mat(q_pos) or mat(k_pos)):
        if (q_pos is not None and not mat(q_pos)) or (k_pos is not None and not mat(k_pos)):
            raise ValueError("q_pos and k_pos must both be tables (H, 2*span, D) or both be score tensors (T, H, 2*span)")
        o, lse = _scores_varlen(q, k, v, q_pos, k_pos, cu_seqlens_q, max_seqlen, sm_scale, position_buckets,
                                max_relative_distance, p2c_mirrored, return_lse, check_status, cu_seqlens_k)
        return (o, lse) if return_lse else o
    if p2c_mirrored:
        raise ValueError("p2c_mirrored applies to materialised score tensors only")
    tables = _tables_from_args(q_pos, k_pos, q, position_buckets, max_relative_distance, tables)
    o, lse, status = _VarlenFn.apply(q, k, v, tables, cu_seqlens_q, max_seqlen, sm_scale, kernel, return_lse,
                                     check_status, cu_seqlens_k)
    if return_lse:
        return o, lse
    return o
