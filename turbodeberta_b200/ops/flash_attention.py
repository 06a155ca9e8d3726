"""Fixed-length (padded) fused disentangled attention.

Same entry point as the reference's ``ops/flash_attention.py:345-369``::

    flash_attention_with_disentangled(q, k, v, q_pos, k_pos, causal=False, sm_scale=None,
                                      position_buckets=0, max_relative_distance=0)

with q, k, v of logical shape ``(B, H, L, D)`` and arbitrary strides (a permuted view of the
``[B, L, H*D]`` projection output works without a copy).  One semantic change: the reference expects
``q_pos``/``k_pos`` to be the materialised score tensors ``Q.Kr^T`` / ``K.Qr^T`` of shape ``(B, H, L, 2*span)``
(``model.py:122-125``); here they are the projected tables ``Kr`` / ``Qr`` themselves, ``(H, 2*span, D)`` or
``(1, H, 2*span, D)`` (what ``model.py:95-100`` calls ``pos_key_layer`` / ``pos_query_layer``), or a prebuilt
``RelPosTables``; the products are formed on chip.  The keyword-only ``seqlens`` adds right-padding masking,
which the reference kernel does not have.  Forward only, like the reference (``ops/flash_attention.py:341-343``).

The reference's own calling convention still works: when ``q_pos`` / ``k_pos`` have the shape ``(B, H, L, 2*span)``
they are taken as the materialised scores and only gathered (a CUDA-core compatibility path, far slower than the
fused one).  The gather follows the eager module (same index for both terms) unless ``p2c_mirrored=True``, which
reproduces the reference kernel's mirrored position->content index (``ops/flash_attention.py:126-132``).
"""
from __future__ import annotations

import math

import torch

from .. import _cabi as cabi
from .. import relpos as _relpos
from .. import status as _status


def _tables_from_args(q_pos, k_pos, q, position_buckets, max_relative_distance, tables):
    """Normalise the position arguments into a RelPosTables (or None when no term is requested)."""
    if tables is not None:
        return tables
    if q_pos is None and k_pos is None:
        return None
    H, D = q.shape[-3] if q.dim() == 4 else q.shape[-2], q.shape[-1]

    def norm(t, name):
        if t is None:
            return None
        if t.dim() == 4 and t.shape[0] == 1:
            t = t[0]
        if t.dim() != 3 or t.shape[0] != H or t.shape[-1] != D:
            raise ValueError(
                f"{name} must be the projected relative table of shape (H, 2*span, D) = ({H}, 2*span, {D}) or the "
                f"materialised score tensor of q's leading shape with 2*span columns; got {tuple(t.shape)}.")
        return t.to(q.dtype).contiguous()

    kr, qr = norm(q_pos, "q_pos"), norm(k_pos, "k_pos")
    two_span = (kr if kr is not None else qr).shape[1]
    if position_buckets > 0:
        if two_span != 2 * position_buckets:
            raise ValueError(f"table has {two_span} rows but position_buckets={position_buckets}")
        if max_relative_distance <= 0:
            raise ValueError("max_relative_distance must be given with position_buckets")
    else:
        if max_relative_distance <= 0:
            max_relative_distance = two_span // 2
        if two_span != 2 * max_relative_distance:
            raise ValueError(f"table has {two_span} rows but max_relative_distance={max_relative_distance}")
    dev = q.device
    sat = _relpos.saturation_distance(position_buckets, max_relative_distance)
    idx = _relpos.bucket_index_table(position_buckets, max_relative_distance, sat + 1, dev)
    exp_dm = sat + cabi.TDB_EXPAND_MARGIN
    want_exp = q.dtype == torch.bfloat16
    kr_exp = _relpos.expand(kr, idx, exp_dm) if (want_exp and kr is not None) else None
    qr_exp = _relpos.expand(qr, idx, exp_dm) if (want_exp and qr is not None) else None
    return _relpos.RelPosTables(position_buckets, max_relative_distance, two_span, idx, sat + 1, kr, qr, kr_exp,
                                qr_exp, exp_dm, (2 * exp_dm + 1 + 7) // 8 * 8)


def _is_materialised(t, q, position_buckets=0, max_relative_distance=0) -> bool:
    """True when ``t`` is a per-token score tensor (``q.shape[:-1] + (2*span,)``) rather than a projected table
    (``(H, 2*span, D)``, optionally with a leading 1).  Where both readings fit the shape, the geometry arguments
    decide (a table has 2*span rows, a score tensor 2*span columns); if they do not, it is taken as a table."""
    if t is None or t.dim() != q.dim() or tuple(t.shape[:-1]) != tuple(q.shape[:-1]):
        return False
    H, D = q.shape[-3] if q.dim() == 4 else q.shape[-2], q.shape[-1]
    table = t.shape[0] == 1 and t.shape[1] == H and t.shape[3] == D if t.dim() == 4 else (t.shape[0] == H and t.shape[2] == D)
    if not table:
        return True
    want = 2 * position_buckets if position_buckets > 0 else 2 * max_relative_distance
    return want > 0 and t.shape[-1] == want and t.shape[-2] != want


def _index_table_for_scores(two_span, position_buckets, max_relative_distance, dev):
    if position_buckets > 0:
        if two_span != 2 * position_buckets:
            raise ValueError(f"score tensors have {two_span} columns but position_buckets={position_buckets}")
        if max_relative_distance <= 0:
            raise ValueError("max_relative_distance must be given with position_buckets")
    else:
        if max_relative_distance <= 0:
            max_relative_distance = two_span // 2
        if two_span != 2 * max_relative_distance:
            raise ValueError(f"score tensors have {two_span} columns but max_relative_distance={max_relative_distance}")
    sat = _relpos.saturation_distance(position_buckets, max_relative_distance)
    return _relpos.bucket_index_table(position_buckets, max_relative_distance, sat + 1, dev), sat + 1


def refuse_gradients(*tensors) -> None:
    """The score-tensor form runs outside any autograd function, so nothing would stop a training loop from getting
    an output without a gradient path; refuse it up front (the fused form raises in ``backward`` instead, like the
    reference, ``ops/flash_attention.py:341-343``)."""
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors):
        raise RuntimeError("turbodeberta_b200 attention is forward-only (as in the reference: no backward kernel); "
                           "call it under torch.no_grad() or with detached inputs")


def _scores_fixed(q, k, v, c2p_scores, p2c_scores, seqlens, sm_scale, position_buckets, max_relative_distance,
                  p2c_mirrored, return_lse, check_status):
    """Legacy form of the fixed-length op: gather from materialised ``(B, H, L, 2*span)`` score tensors."""
    dev = cabi.require_cuda(q, k, v, seqlens)
    refuse_gradients(q, k, v, c2p_scores, p2c_scores)
    if q.dim() != 4 or k.shape != q.shape or v.shape != q.shape:
        raise ValueError("q, k, v must share the shape (B, H, L, D)")
    B, H, L, D = q.shape
    code = cabi.dtype_code(q.dtype)
    some = c2p_scores if c2p_scores is not None else p2c_scores
    two_span = some.shape[-1]
    for t, name in ((c2p_scores, "q_pos"), (p2c_scores, "k_pos")):
        if t is None:
            continue
        if tuple(t.shape) != (B, H, L, two_span) or t.dtype != q.dtype or t.stride(-1) != 1:
            raise ValueError(f"{name} must be (B, H, L, 2*span) of q's dtype with a contiguous last dimension")
    for t in (q, k, v):
        if t.stride(-1) != 1:
            raise ValueError("the head dimension must be contiguous")
    idx, idm = _index_table_for_scores(two_span, position_buckets, max_relative_distance, dev)
    o = torch.empty((B, L, H, D), dtype=q.dtype, device=dev).permute(0, 2, 1, 3)
    lse = torch.empty((B, H, L), dtype=torch.float32, device=dev) if return_lse else None
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    if B == 0 or L == 0:
        return o, lse
    if seqlens is not None:
        seqlens = seqlens.to(device=dev, dtype=torch.int32).contiguous()
    flags = ((cabi.TDB_FLAG_C2P if c2p_scores is not None else 0) | (cabi.TDB_FLAG_P2C if p2c_scores is not None else 0)
             | (cabi.TDB_FLAG_P2C_MIRRORED if p2c_mirrored else 0))

    def s(t):
        return (t.stride(0), t.stride(2), t.stride(1)) if t is not None else (0, 0, 0)      # batch, token, head

    with torch.cuda.device(dev):
        rc = cabi.lib.tdb_attn_fwd_fixed_scores(
            cabi.ptr(q), cabi.ptr(k), cabi.ptr(v), cabi.ptr(o), *s(q), *s(k), *s(v), *s(o),
            cabi.ptr(c2p_scores), *s(c2p_scores), cabi.ptr(p2c_scores), *s(p2c_scores), two_span, cabi.ptr(idx), idm,
            cabi.ptr(seqlens), B, L, H, D, float(sm_scale), flags, code, cabi.ptr(lse), cabi.ptr(status),
            cabi.stream_ptr(dev))
    cabi.check(rc)
    if check_status:
        _check_status(status)
    else:
        _PENDING_STATUS.append(status)
    return o, lse


# Status words of calls made with check_status=False; read by check_pending_status().
_PENDING_STATUS = _status.PENDING


def check_pending_status() -> None:
    """Read (one synchronisation) the device status words of every call since the last check that was made
    with ``check_status=False`` and raise if any bounded device wait gave up or any ``cu_seqlens`` was malformed."""
    pending = _PENDING_STATUS.drain()
    if not pending:
        return
    by_dev = {}
    for st in pending:
        by_dev.setdefault(st.device, []).append(st)
    for dev, sts in by_dev.items():
        _check_status(torch.stack(sts).amax(dim=0))


def _check_status(status: torch.Tensor):
    """Read the device status words (synchronises); raise if a wait gave up or cu_seqlens was invalid."""
    st = status.tolist()
    if st[0]:
        raise cabi.TdbError(cabi.ERR_TIMEOUT, f"a device-side wait gave up (barrier code {st[0]})")
    if st[1]:
        raise ValueError("cu_seqlens is not a non-decreasing sequence ending at the token count (or the key offsets "
                         "differ from the query offsets, or max_seqlen is smaller than the longest sequence)")


class _FixedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, tables, seqlens, sm_scale, kernel, return_lse, check):
        dev = cabi.require_cuda(q, k, v, seqlens)
        if q.dim() != 4 or k.shape != q.shape or v.shape != q.shape:
            raise ValueError("q, k, v must share the shape (B, H, L, D); cross-attention lengths are not supported")
        B, H, L, D = q.shape
        if not (q.dtype == k.dtype == v.dtype):
            raise ValueError("q, k, v must share a dtype")
        code = cabi.dtype_code(q.dtype)
        for t in (q, k, v):
            if t.stride(-1) != 1:
                raise ValueError("the head dimension must be contiguous")
        o = torch.empty((B, L, H, D), dtype=q.dtype, device=dev).permute(0, 2, 1, 3)     # (B,H,L,D) view of [B,L,H,D]
        lse = torch.empty((B, H, L), dtype=torch.float32, device=dev) if return_lse else None
        status = torch.zeros(4, dtype=torch.int32, device=dev)
        if B == 0 or L == 0:                         # nothing to compute
            return (o, lse, status)
        if seqlens is not None:
            seqlens = seqlens.to(device=dev, dtype=torch.int32).contiguous()
            if seqlens.numel() != B:
                raise ValueError("seqlens must have one entry per batch row")
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

        def s(t):
            return (t.stride(0), t.stride(2), t.stride(1))      # batch, token, head

        with torch.cuda.device(dev):
            rc = cabi.lib.tdb_attn_fwd_fixed(
                cabi.ptr(q), cabi.ptr(k), cabi.ptr(v), cabi.ptr(o), *s(q), *s(k), *s(v), *s(o),
                cabi.ptr(kr), cabi.ptr(qr), two_span, cabi.ptr(idx), idm, cabi.ptr(kr_exp), cabi.ptr(qr_exp), edm, erows,
                cabi.ptr(seqlens), B, L, H, D, float(sm_scale), flags, code, kernel, cabi.ptr(lse), cabi.ptr(status),
                cabi.stream_ptr(dev))
        cabi.check(rc)
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


def flash_attention_with_disentangled(q, k, v, q_pos, k_pos, causal=False, sm_scale=None, position_buckets=0,
                                      max_relative_distance=0, *, seqlens=None, tables=None,
                                      kernel=cabi.TDB_KERNEL_AUTO, return_lse=False, check_status=True,
                                      p2c_mirrored=False):
    """Fused disentangled attention on padded ``(B, H, L, D)`` inputs; returns ``o`` with the shape of ``q``
    (memory layout ``[B, L, H, D]``, so ``o.transpose(1, 2).reshape(B, L, H*D)`` is a free view).

    ``q_pos`` feeds the content->position term (table ``Kr``), ``k_pos`` the position->content term (``Qr``);
    either may be None.  ``seqlens`` (int ``[B]``) masks keys beyond each row's length and zeroes its padded
    query rows.  ``check_status=False`` skips the end-of-call read of the device status words (no host sync);
    the caller then owns checking ``status``.
    """
    if causal:
        raise NotImplementedError("causal masking is not part of the DeBERTa encoder path")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    mat = lambda t: _is_materialised(t, q, position_buckets, max_relative_distance)
    if tables is None and (mat(q_pos) or mat(k_pos)):
        if (q_pos is not None and not mat(q_pos)) or (k_pos is not None and not mat(k_pos)):
            raise ValueError("q_pos and k_pos must both be tables (H, 2*span, D) or both be score tensors (B, H, L, 2*span)")
        o, lse = _scores_fixed(q, k, v, q_pos, k_pos, seqlens, sm_scale, position_buckets, max_relative_distance,
                               p2c_mirrored, return_lse, check_status)
        return (o, lse) if return_lse else o
    if p2c_mirrored:
        raise ValueError("p2c_mirrored applies to materialised score tensors only")
    tables = _tables_from_args(q_pos, k_pos, q, position_buckets, max_relative_distance, tables)
    o, lse, status = _FixedFn.apply(q, k, v, tables, seqlens, sm_scale, kernel, return_lse, check_status)
    if return_lse:
        return o, lse
    return o
