"""Host side of the once-per-layer relative-position tables.

``RelPosTables`` owns, for one attention layer on one device and dtype:
  * ``idx``     int16 ``[2*delta_max+1]``: distance -> table row (``tdb_bucket_table``), shared by all layers
                with the same (position_buckets, max_relative_positions);
  * ``kr, qr``  ``[H, 2*span, D]``: projected relative embeddings (``tdb_relpos_project``), what the reference
                recomputes in every forward at ``model.py:92-110``;
  * ``kr_exp, qr_exp`` bf16 ``[H, exp_rows, D]``: distance-expanded copies (``tdb_relpos_expand``) for the
                tensor-core kernel.
All of it is derived data: ``build_tables`` recomputes it from the module's weights; the patched module caches
the result keyed on the weights' versions.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _cabi as cabi
from .status import PENDING as PENDING_STATUS

_IDX_CACHE: dict = {}


def att_span(position_buckets: int, max_relative_positions: int) -> int:
    return position_buckets if position_buckets > 0 else max_relative_positions


def saturation_distance(position_buckets: int, max_relative_positions: int) -> int:
    """A distance |q-k| from which the table row no longer changes (both signs).

    Log buckets: the row index clamps once bucket >= span, i.e. once
    ``|delta| > mid * ((P-1)/mid) ** ((span-mid-1)/(mid-1))``; for an even bucket count that is ``|delta| >= P``.
    Without buckets the index is ``clamp(delta + span)`` and clamps at ``|delta| >= span``."""
    span = att_span(position_buckets, max_relative_positions)
    if position_buckets <= 0:
        return span
    mid = position_buckets // 2
    if mid <= 1:
        return max_relative_positions + 2
    bound = mid * ((max_relative_positions - 1) / mid) ** ((span - mid - 1) / (mid - 1))
    return max(max_relative_positions, int(math.ceil(bound)) + 2)


def bucket_index_table(position_buckets: int, max_relative_positions: int, delta_max: int, device) -> torch.Tensor:
    """int16 tensor ``idx[delta + delta_max]`` on ``device`` (cached per device and geometry)."""
    device = torch.device(device)
    key = (device, position_buckets, max_relative_positions, delta_max)
    t = _IDX_CACHE.get(key)
    if t is None:
        t = torch.empty(2 * delta_max + 1, dtype=torch.int16, device=device)
        with torch.cuda.device(device):
            cabi.check(cabi.lib.tdb_bucket_table(position_buckets, max_relative_positions, delta_max,
                                                 cabi.ptr(t), cabi.stream_ptr(device)))
        _IDX_CACHE[key] = t
    return t


def project(rel: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, num_heads: int) -> torch.Tensor:
    """``[2*span, hidden] x [H*D, hidden]^T (+bias)`` -> ``[H, 2*span, D]`` in the dtype of ``rel``."""
    dev = cabi.require_cuda(rel, weight, bias)
    rel = rel.contiguous()
    weight = weight.to(rel.dtype).contiguous()
    bias = None if bias is None else bias.to(rel.dtype).contiguous()
    two_span, hidden = rel.shape
    hd = weight.shape[0]
    if weight.shape[1] != hidden or hd % num_heads:
        raise ValueError("projection weight does not match the relative embeddings / head count")
    D = hd // num_heads
    out = torch.empty(num_heads, two_span, D, dtype=rel.dtype, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        cabi.check(cabi.lib.tdb_relpos_project(cabi.ptr(rel), cabi.ptr(weight), cabi.ptr(bias), two_span, hidden,
                                               num_heads, D, cabi.dtype_code(rel.dtype), cabi.ptr(out),
                                               cabi.ptr(status), cabi.stream_ptr(dev)))
    PENDING_STATUS.append(status)          # read by ops.flash_attention.check_pending_status (no sync here)
    return out


def expand(table: torch.Tensor, idx: torch.Tensor, exp_delta_max: int) -> torch.Tensor:
    """Distance-expanded bf16 copy ``[H, exp_rows, D]`` of a projected table ``[H, 2*span, D]``."""
    dev = cabi.require_cuda(table, idx)
    H, two_span, D = table.shape
    exp_rows = (2 * exp_delta_max + 1 + 7) // 8 * 8
    out = torch.empty(H, exp_rows, D, dtype=torch.bfloat16, device=dev)
    idx_delta_max = (idx.numel() - 1) // 2
    with torch.cuda.device(dev):
        cabi.check(cabi.lib.tdb_relpos_expand(cabi.ptr(table.contiguous()), cabi.ptr(idx), idx_delta_max, H, two_span,
                                              D, cabi.dtype_code(table.dtype), exp_delta_max, exp_rows,
                                              cabi.ptr(out), cabi.stream_ptr(dev)))
    return out


@dataclass
class RelPosTables:
    position_buckets: int
    max_relative_positions: int
    two_span: int
    idx: torch.Tensor
    idx_delta_max: int
    kr: torch.Tensor | None
    qr: torch.Tensor | None
    kr_exp: torch.Tensor | None
    qr_exp: torch.Tensor | None
    exp_delta_max: int
    exp_rows: int


def build_tables(rel_embeddings: torch.Tensor, *, num_heads: int, position_buckets: int,
                 max_relative_positions: int, key_weight=None, key_bias=None, query_weight=None, query_bias=None,
                 c2p: bool = True, p2c: bool = True, expanded: bool | None = None) -> RelPosTables:
    """Project ``rel_embeddings[:2*span]`` with the given Linear parameters (``key_*`` feeds the
    content->position term, ``query_*`` the position->content term) and derive the expanded copies."""
    dev = cabi.require_cuda(rel_embeddings)
    span = att_span(position_buckets, max_relative_positions)
    sat = saturation_distance(position_buckets, max_relative_positions)
    idx_delta_max = sat + 1
    idx = bucket_index_table(position_buckets, max_relative_positions, idx_delta_max, dev)
    rel = rel_embeddings[: 2 * span]
    if rel.shape[0] != 2 * span:
        raise ValueError(f"rel_embeddings has {rel_embeddings.shape[0]} rows, the module needs {2 * span}")
    kr = project(rel, key_weight, key_bias, num_heads) if c2p else None
    qr = project(rel, query_weight, query_bias, num_heads) if p2c else None
    if expanded is None:
        expanded = rel.dtype == torch.bfloat16
    exp_delta_max = sat + cabi.TDB_EXPAND_MARGIN
    exp_rows = (2 * exp_delta_max + 1 + 7) // 8 * 8
    kr_exp = expand(kr, idx, exp_delta_max) if (expanded and kr is not None) else None
    qr_exp = expand(qr, idx, exp_delta_max) if (expanded and qr is not None) else None
    return RelPosTables(position_buckets, max_relative_positions, 2 * span, idx, idx_delta_max, kr, qr,
                        kr_exp, qr_exp, exp_delta_max, exp_rows)
