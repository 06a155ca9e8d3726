"""The five benchmark configurations at (or near) full size on the GPU.

The numpy oracle is too slow for whole configurations, so each one is checked two ways: the tensor-core kernel
against the exact CUDA-core kernel on identical bf16 inputs (a size-independent property: both must produce the
same attention), and the tensor-core kernel against the oracle on a few whole sequences picked from the batch.
"""
import numpy as np
import pytest
import torch

from oracle import disentangled_oracle as orc
from tests import util
from turbodeberta_b200 import workloads

pytestmark = pytest.mark.gpu
UMMA, SIMT = 2, 1
DT = torch.bfloat16


def _setup(w):
    q, k, v, rel, P = util.device_inputs(w, DT)
    tables = util.make_tables(w, rel, P)
    return q, k, v, tables


def _oracle_rows(q, k, v, tables, w, lo, hi):
    """Oracle attention for one sequence given as token range [lo, hi) of packed (or one padded row's) q, k, v."""
    return orc.attention_single(util.f64(q[lo:hi]), util.f64(k[lo:hi]), util.f64(v[lo:hi]), util.f64(tables.kr),
                                util.f64(tables.qr), position_buckets=w.position_buckets,
                                max_relative_positions=w.max_relative_positions, sm_scale=1.0 / (3 * 64) ** 0.5)


def _fixed(w, kernel, q, k, v, tables):
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    lens = torch.as_tensor(np.asarray(w.lengths), dtype=torch.int32, device="cuda")
    o = flash_attention_with_disentangled(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), None, None,
                                          False, 1.0 / (3 * 64) ** 0.5, w.position_buckets, w.max_relative_positions,
                                          seqlens=lens, tables=tables, kernel=kernel)
    return o.permute(0, 2, 1, 3)


def _varlen(w, kernel, q, k, v, tables):
    from turbodeberta_b200.ops.flash_attention_varlen import flash_attention_with_disentangled_varlen
    cu = torch.as_tensor(w.cu_seqlens, device="cuda")
    mx = int(w.lengths.max())
    return flash_attention_with_disentangled_varlen(q, k, v, None, None, cu, cu, mx, mx, False, 1.0 / (3 * 64) ** 0.5,
                                                    w.position_buckets, w.max_relative_positions, tables=tables,
                                                    kernel=kernel)


def test_config2_padded_batch():
    w = workloads.config2()
    q, k, v, tables = _setup(w)
    o = _fixed(w, UMMA, q, k, v, tables)
    o_ref = _fixed(w, SIMT, q, k, v, tables)
    assert torch.isfinite(o.float()).all()
    assert (o.float() - o_ref.float()).abs().max().item() < 1e-2
    for b in (int(np.argmin(w.lengths)), int(np.argmax(w.lengths))):
        n = int(w.lengths[b])
        ref = _oracle_rows(q[b], k[b], v[b], tables, w, 0, n)
        util.assert_close(o[b, :n], ref, DT, f"config 2 row {b}")
        assert torch.count_nonzero(o[b, n:]).item() == 0


def test_config3_packed_stream():
    w = workloads.config3()
    q, k, v, tables = _setup(w)
    o = _varlen(w, UMMA, q, k, v, tables)
    o_ref = _varlen(w, SIMT, q, k, v, tables)
    assert torch.isfinite(o.float()).all()
    assert (o.float() - o_ref.float()).abs().max().item() < 1e-2
    cu = w.cu_seqlens
    order = np.argsort(w.lengths)
    for s in (int(order[0]), int(order[len(order) // 2]), int(order[-1])):
        ref = _oracle_rows(q, k, v, tables, w, int(cu[s]), int(cu[s + 1]))
        util.assert_close(o[cu[s]:cu[s + 1]], ref, DT, f"config 3 sequence {s} (length {w.lengths[s]})")


def test_config5_fixed_long_sequences():
    w = workloads.config5_fixed()
    q, k, v, tables = _setup(w)
    o = _fixed(w, UMMA, q, k, v, tables)
    o_ref = _fixed(w, SIMT, q, k, v, tables)
    assert torch.isfinite(o.float()).all()
    assert (o.float() - o_ref.float()).abs().max().item() < 1e-2
    # oracle on one head of one sequence (4096 x 4096 scores)
    w1 = workloads.config5_fixed(batch=1)
    ref = orc.attention_single(util.f64(q[0, :, :1]), util.f64(k[0, :, :1]), util.f64(v[0, :, :1]),
                               util.f64(tables.kr[:1]), util.f64(tables.qr[:1]), position_buckets=256,
                               max_relative_positions=512, sm_scale=1.0 / (3 * 64) ** 0.5)
    util.assert_close(o[0, :, :1], ref, DT, "config 5 fixed, sequence 0, head 0")


def test_config5_packed_long_sequences():
    """Eight of the 64 sequences of the packed long-sequence case (lengths 2048..8192, every far tile saturated)."""
    w = workloads.config5_varlen(n_seqs=8)
    q, k, v, tables = _setup(w)
    o = _varlen(w, UMMA, q, k, v, tables)
    o_ref = _varlen(w, SIMT, q, k, v, tables)
    assert torch.isfinite(o.float()).all()
    assert (o.float() - o_ref.float()).abs().max().item() < 1e-2
    # the oracle itself on one head of the shortest sequence (>= 2048 tokens: band tiles and saturated tiles)
    s = int(np.argmin(w.lengths))
    lo, hi = int(w.cu_seqlens[s]), int(w.cu_seqlens[s + 1])
    ref = orc.attention_single(util.f64(q[lo:hi, :1]), util.f64(k[lo:hi, :1]), util.f64(v[lo:hi, :1]),
                               util.f64(tables.kr[:1]), util.f64(tables.qr[:1]), position_buckets=256,
                               max_relative_positions=512, sm_scale=1.0 / (3 * 64) ** 0.5)
    util.assert_close(o[lo:hi, :1], ref, DT, f"config 5 packed, sequence {s} (length {hi - lo}), head 0")
