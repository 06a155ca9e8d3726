"""The workspace-free packed attention entry point, called straight through the C ABI.

`tdb_attn_fwd_varlen_static` is for hosts that cannot hand the library scratch memory: for example a serving
runtime whose execute callback receives nothing but its bound input and output buffers, or a C program that
has given every byte of device memory to a framework's pool and cannot reach that pool's allocator.  It keeps
the tile list in a fixed array inside the library image, so it must give exactly the result of the regular
entry point (which takes a caller-allocated workspace), call after call, even though the array still holds
the previous call's list.  This file is collected last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from tests import util
from turbodeberta_b200 import workloads

pytestmark = pytest.mark.gpu
DT = torch.bfloat16
UMMA = 2


def _problem(lengths, seed):
    w = workloads.make_attention_workload("noalloc", seed=seed, hidden_size=128, num_heads=2, lengths=lengths,
                                          padded_len=None, dtype=DT)
    q, k, v, rel, P = util.device_inputs(w, DT)
    tables = util.make_tables(w, rel, P)
    cu = torch.as_tensor(w.cu_seqlens, device="cuda")
    return w, q, k, v, tables, cu


def _call(static, q, k, v, t, cu, max_len):
    """One attention call through ctypes; `static` picks the workspace-free entry point."""
    from turbodeberta_b200 import _cabi as cabi
    T, H, D = q.shape
    n = cu.numel() - 1
    o = torch.full((T, H, D), float("nan"), dtype=DT, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    head = [cabi.ptr(q), cabi.ptr(k), cabi.ptr(v), cabi.ptr(o),
            q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1), o.stride(0), o.stride(1),
            cabi.ptr(t.kr), cabi.ptr(t.qr), t.two_span, cabi.ptr(t.idx), t.idx_delta_max,
            cabi.ptr(t.kr_exp), cabi.ptr(t.qr_exp), t.exp_delta_max, t.exp_rows,
            cabi.ptr(cu), n, T, max_len, H, D, 1.0 / (3 * 64) ** 0.5, 3, cabi.TDB_DTYPE_BF16, UMMA]
    tail = [None, cabi.ptr(status), cabi.stream_ptr(q.device)]
    if static:
        rc = cabi.lib.tdb_attn_fwd_varlen_static(*head, *tail)
        ws = None
    else:
        nbytes = int(cabi.lib.tdb_attn_workspace_bytes(n, T))
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        rc = cabi.lib.tdb_attn_fwd_varlen(*head, cabi.ptr(ws), nbytes, *tail)
    cabi.check(rc)
    torch.cuda.synchronize()
    assert status.tolist()[:2] == [0, 0]
    return o


def _assert_static_call_takes_no_device_memory(q, k, v, t, cu, max_len):
    """The point of the entry point: a repeated call (the array's address is known by now) leaves the device's free
    memory exactly as it found it.  The output and status tensors are made first, so that the only thing between the
    two readings is the library call itself; the readings come from the driver, not from torch's caching allocator."""
    from turbodeberta_b200 import _cabi as cabi
    T, H, D = q.shape
    o = torch.empty((T, H, D), dtype=DT, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    args = [cabi.ptr(q), cabi.ptr(k), cabi.ptr(v), cabi.ptr(o),
            q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1), o.stride(0), o.stride(1),
            cabi.ptr(t.kr), cabi.ptr(t.qr), t.two_span, cabi.ptr(t.idx), t.idx_delta_max,
            cabi.ptr(t.kr_exp), cabi.ptr(t.qr_exp), t.exp_delta_max, t.exp_rows,
            cabi.ptr(cu), cu.numel() - 1, T, max_len, H, D, 1.0 / (3 * 64) ** 0.5, 3, cabi.TDB_DTYPE_BF16, UMMA,
            None, cabi.ptr(status), cabi.stream_ptr(q.device)]
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    cabi.check(cabi.lib.tdb_attn_fwd_varlen_static(*args))
    free_during, _ = torch.cuda.mem_get_info()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_before == free_during == free_after, (free_before, free_during, free_after)


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row():
    # first call: many tiles; second call: fewer and different ones, so stale entries of the first call sit
    # behind the part of the list that the second call rewrites
    for lengths, seed in (([300, 17, 129, 640, 1, 128], 71), ([90, 257], 72)):
        w, q, k, v, tables, cu = _problem(lengths, seed)
        mx = max(lengths)
        ref = _call(False, q, k, v, tables, cu, mx)
        got = _call(True, q, k, v, tables, cu, mx)
        _assert_static_call_takes_no_device_memory(q, k, v, tables, cu, mx)
        assert torch.isfinite(got.float()).all()
        err = (got.float() - ref.float()).abs().max().item()
        assert err <= util.BF16_ABS_TOL, err
        assert torch.equal(got, ref)          # same kernel, same inputs: bit-identical
        oracle = util.oracle_varlen(q, k, v, tables, w.cu_seqlens, w, sm_scale=1.0 / (3 * 64) ** 0.5)
        util.assert_close(got, oracle, DT, f"static scratch {lengths}")


def test_static_scratch_rejects_oversized_problems_before_launch():
    from turbodeberta_b200 import _cabi as cabi
    w, q, k, v, tables, cu = _problem([64, 64], 73)
    T, H, D = q.shape
    o = torch.zeros_like(q)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    too_many = cabi.TDB_STATIC_MAX_TILES          # n_seqs alone already exceeds the limit
    rc = cabi.lib.tdb_attn_fwd_varlen_static(
        cabi.ptr(q), cabi.ptr(k), cabi.ptr(v), cabi.ptr(o), q.stride(0), q.stride(1), k.stride(0), k.stride(1),
        v.stride(0), v.stride(1), o.stride(0), o.stride(1), cabi.ptr(tables.kr), cabi.ptr(tables.qr), tables.two_span,
        cabi.ptr(tables.idx), tables.idx_delta_max, cabi.ptr(tables.kr_exp), cabi.ptr(tables.qr_exp),
        tables.exp_delta_max, tables.exp_rows, cabi.ptr(cu), too_many, T, 64, H, D, 0.07, 3, cabi.TDB_DTYPE_BF16, UMMA,
        None, cabi.ptr(status), cabi.stream_ptr(q.device))
    assert rc == cabi.ERR_WORKSPACE
    assert b"built-in scratch" in cabi.lib.tdb_last_error()
    torch.cuda.synchronize()
    assert torch.count_nonzero(o).item() == 0      # nothing was launched
