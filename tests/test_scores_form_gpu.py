"""GPU parity of the legacy operator form (materialised position scores, reference model.py:122-137 and 143-182)
against the oracle: fixed and packed, fp32 and bf16, eager and mirrored position->content index."""
import numpy as np
import pytest
import torch

from oracle import disentangled_oracle as orc
from tests import util
from turbodeberta_b200 import workloads

pytestmark = pytest.mark.gpu


def _inputs(dtype, lengths, padded, seed=41, heads=2, buckets=32, maxpos=64):
    w = workloads.make_attention_workload("t", seed=seed, hidden_size=64 * heads, num_heads=heads, lengths=lengths,
                                          padded_len=padded, position_buckets=buckets, max_relative_positions=maxpos,
                                          dtype=dtype)
    q, k, v, rel, P = util.device_inputs(w, dtype)
    tables = util.make_tables(w, rel, P)
    return w, q, k, v, tables


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mirrored", [False, True])
def test_fixed_scores_form(dtype, mirrored):
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    w, q, k, v, tables = _inputs(dtype, [150, 97], 150)
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))                    # (B, H, L, D) views
    pos_key = torch.matmul(qh, tables.kr.transpose(-1, -2))                      # (B, H, L, 2span), reference model.py:123
    pos_query = torch.matmul(kh, tables.qr.transpose(-1, -2))
    scale = 1.0 / (3 * 64) ** 0.5
    lens = torch.as_tensor(np.asarray(w.lengths), dtype=torch.int32, device="cuda")
    o = flash_attention_with_disentangled(qh, kh, vh, pos_key, pos_query, False, scale, 32, 64, seqlens=lens,
                                          p2c_mirrored=mirrored)
    assert o.shape == qh.shape
    ref = np.zeros((2, 150, 2, 64))
    for b, n in enumerate(w.lengths):
        ref[b, :n] = orc.attention_single_scores(
            util.f64(q[b, :n]), util.f64(k[b, :n]), util.f64(v[b, :n]), util.f64(pos_key[b, :, :n].permute(1, 0, 2)),
            util.f64(pos_query[b, :, :n].permute(1, 0, 2)), position_buckets=32, max_relative_positions=64,
            sm_scale=scale, p2c_mirrored=mirrored)
    util.assert_close(o.permute(0, 2, 1, 3), ref, dtype, f"scores form fixed mirrored={mirrored}")
    if not mirrored and dtype == torch.float32:      # same numbers as the fused table form
        o2 = flash_attention_with_disentangled(qh, kh, vh, None, None, False, scale, 32, 64, seqlens=lens, tables=tables)
        assert (o - o2).abs().max().item() < 1e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_varlen_scores_form(dtype):
    from turbodeberta_b200.ops.flash_attention_varlen import flash_attention_with_disentangled_varlen
    w = workloads.make_attention_workload("t", seed=43, hidden_size=128, num_heads=2, lengths=[70, 1, 130, 33],
                                          padded_len=None, position_buckets=32, max_relative_positions=64, dtype=dtype)
    q, k, v, rel, P = util.device_inputs(w, dtype)
    tables = util.make_tables(w, rel, P)
    pos_key = torch.einsum("thd,hmd->thm", q, tables.kr)                          # (T, H, 2span), reference model.py:146
    pos_query = torch.einsum("thd,hmd->thm", k, tables.qr)
    cu = torch.as_tensor(np.asarray(w.cu_seqlens), dtype=torch.int32, device="cuda")
    scale = 1.0 / (3 * 64) ** 0.5
    o, lse = flash_attention_with_disentangled_varlen(q, k, v, pos_key, pos_query, cu, cu, 130, 130, False, scale, 32, 64,
                                                      return_lse=True)
    ref = np.zeros(tuple(q.shape))
    cuh = np.asarray(w.cu_seqlens)
    for b in range(len(cuh) - 1):
        s, e = int(cuh[b]), int(cuh[b + 1])
        ref[s:e] = orc.attention_single_scores(util.f64(q[s:e]), util.f64(k[s:e]), util.f64(v[s:e]),
                                               util.f64(pos_key[s:e]), util.f64(pos_query[s:e]), position_buckets=32,
                                               max_relative_positions=64, sm_scale=scale)
    util.assert_close(o, ref, dtype, "scores form packed")
    assert torch.isfinite(lse).all()
    only = flash_attention_with_disentangled_varlen(q, k, v, pos_key, None, cu, cu, 130, 130, False, scale, 32, 64)
    ref1 = orc.attention_varlen(util.f64(q), util.f64(k), util.f64(v), util.f64(tables.kr), None, cuh,
                                position_buckets=32, max_relative_positions=64, p2c=False, sm_scale=scale)
    util.assert_close(only, ref1, dtype, "scores form packed, c2p only")


def test_scores_form_argument_errors():
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    w, q, k, v, tables = _inputs(torch.float32, [96], 96)     # (L = 2*span = D would read as a table: documented corner)
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    pos_key = torch.matmul(qh, tables.kr.transpose(-1, -2))
    with pytest.raises(ValueError):                   # one table, one score tensor
        flash_attention_with_disentangled(qh, kh, vh, pos_key, tables.qr, False, None, 32, 64)
    with pytest.raises(ValueError):                   # geometry does not match the score columns
        flash_attention_with_disentangled(qh, kh, vh, pos_key, None, False, None, 16, 64)
    with pytest.raises(ValueError):                   # the mirrored index exists for score tensors only
        flash_attention_with_disentangled(qh, kh, vh, tables.kr, tables.qr, False, None, 32, 64, p2c_mirrored=True)
