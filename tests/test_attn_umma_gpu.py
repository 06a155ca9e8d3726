"""GPU parity of the tensor-core (tcgen05) attention kernel against the oracle, bf16."""
import numpy as np
import pytest
import torch

from tests import util
from turbodeberta_b200 import workloads

pytestmark = pytest.mark.gpu
UMMA, SIMT = 2, 1
DT = torch.bfloat16


def _fixed(w, c2p=True, p2c=True, with_lens=True, kernel=UMMA):
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    q, k, v, rel, P = util.device_inputs(w, DT)
    tables = util.make_tables(w, rel, P, c2p, p2c) if (c2p or p2c) else None
    scale = 1.0 / (w.head_dim * (1 + int(c2p) + int(p2c))) ** 0.5
    lens = torch.as_tensor(np.asarray(w.lengths), dtype=torch.int32, device="cuda") if with_lens else None
    o = flash_attention_with_disentangled(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3),
                                          None, None, False, scale, w.position_buckets, w.max_relative_positions,
                                          seqlens=lens, tables=tables, kernel=kernel)
    ref = util.oracle_fixed(q, k, v, tables, w.lengths if with_lens else None, w, c2p, p2c, scale)
    return o.permute(0, 2, 1, 3), ref


def _wl(lengths, padded, hidden=128, heads=2, seed=31, buckets=256, maxpos=512):
    return workloads.make_attention_workload("t", seed=seed, hidden_size=hidden, num_heads=heads, lengths=lengths,
                                             padded_len=padded, position_buckets=buckets,
                                             max_relative_positions=maxpos, dtype=DT)


def test_umma_content_only_one_tile():
    o, ref = _fixed(_wl([128], 128, hidden=64, heads=1), c2p=False, p2c=False, with_lens=False)
    util.assert_close(o, ref, DT, "QK^T/softmax/PV only, one tile")


def test_umma_content_only_multi_tile():
    o, ref = _fixed(_wl([384, 300], 384), c2p=False, p2c=False)
    util.assert_close(o, ref, DT, "content only, 3 key tiles, padded")


def test_umma_c2p_only():
    o, ref = _fixed(_wl([256, 200], 256), c2p=True, p2c=False)
    util.assert_close(o, ref, DT, "c2p only")


def test_umma_p2c_only():
    o, ref = _fixed(_wl([256, 200], 256), c2p=False, p2c=True)
    util.assert_close(o, ref, DT, "p2c only")


@pytest.mark.parametrize("lengths,padded", [([128], 128), ([512, 64, 333, 129], 512), ([700, 1], 700), ([40, 23], 40)])
def test_umma_both_terms_fixed(lengths, padded):
    o, ref = _fixed(_wl(lengths, padded))
    util.assert_close(o, ref, DT, f"fixed {lengths}")


def test_umma_all_ones_no_lengths():
    o, ref = _fixed(_wl([256, 256, 256], 256, hidden=192, heads=3), with_lens=False)
    util.assert_close(o, ref, DT, "all ones")


@pytest.mark.parametrize("pair", [(32, 64), (0, 64), (64, 128)])
def test_umma_other_bucket_geometries(pair):
    o, ref = _fixed(_wl([300, 257], 300, buckets=pair[0], maxpos=pair[1]))
    util.assert_close(o, ref, DT, f"buckets {pair}")


def test_umma_matches_simt_closely():
    """Both kernels see identical bf16 inputs; they must agree much more tightly than the oracle tolerance."""
    w = _wl([512, 384], 512, hidden=256, heads=4)
    o1, _ = _fixed(w, kernel=UMMA)
    o2, _ = _fixed(w, kernel=SIMT)
    assert (o1.float() - o2.float()).abs().max().item() < 1e-2


def test_umma_varlen():
    from turbodeberta_b200.ops.flash_attention_varlen import flash_attention_with_disentangled_varlen
    lengths = [5, 1, 33, 17, 128, 129, 127, 600, 16, 15, 1100]
    w = _wl(lengths, None)
    q, k, v, rel, P = util.device_inputs(w, DT)
    tables = util.make_tables(w, rel, P)
    cu = torch.as_tensor(w.cu_seqlens, device="cuda")
    scale = 1.0 / (3 * 64) ** 0.5
    o, lse = flash_attention_with_disentangled_varlen(q, k, v, None, None, cu, cu, 1100, 1100, False, scale, 256, 512,
                                                      tables=tables, kernel=UMMA, return_lse=True)
    ref = util.oracle_varlen(q, k, v, tables, w.cu_seqlens, w, sm_scale=scale)
    util.assert_close(o, ref, DT, "varlen")
    o2, lse2 = flash_attention_with_disentangled_varlen(q, k, v, None, None, cu, cu, 1100, 1100, False, scale, 256, 512,
                                                        tables=tables, kernel=SIMT, return_lse=True)
    assert (lse - lse2).abs().max().item() < 5e-2
    # running the same launch twice must give bit-identical results (no races)
    o3 = flash_attention_with_disentangled_varlen(q, k, v, None, None, cu, cu, 1100, 1100, False, scale, 256, 512,
                                                  tables=tables, kernel=UMMA)
    assert torch.equal(o, o3)


def test_umma_bad_cu_seqlens_reported():
    from turbodeberta_b200.ops.flash_attention_varlen import flash_attention_with_disentangled_varlen
    w = _wl([64, 64], None)
    q, k, v, rel, P = util.device_inputs(w, DT)
    tables = util.make_tables(w, rel, P)
    cu = torch.tensor([0, 80, 64], dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError):
        flash_attention_with_disentangled_varlen(q, k, v, None, None, cu, cu, 64, 64, False, 0.07, 256, 512,
                                                 tables=tables, kernel=UMMA)


def test_empty_and_degenerate_inputs():
    """Empty batches, zero-length sequences inside a packed stream and a fully padded row."""
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    from turbodeberta_b200.ops.flash_attention_varlen import flash_attention_with_disentangled_varlen
    w = _wl([130, 5], None)
    q, k, v, rel, P = util.device_inputs(w, DT)
    tables = util.make_tables(w, rel, P)
    scale = 1.0 / (3 * 64) ** 0.5
    # packed stream with empty sequences in front, in the middle and at the end
    cu = torch.tensor([0, 0, 130, 130, 135, 135], dtype=torch.int32, device="cuda")
    o = flash_attention_with_disentangled_varlen(q, k, v, None, None, cu, cu, 130, 130, False, scale, 256, 512,
                                                 tables=tables, kernel=UMMA)
    ref = util.oracle_varlen(q, k, v, tables, np.array([0, 130, 135]), w, sm_scale=scale)
    util.assert_close(o, ref, DT, "packed stream with empty sequences")
    # no tokens at all
    e = torch.empty(0, 2, 64, dtype=DT, device="cuda")
    cu0 = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert flash_attention_with_disentangled_varlen(e, e, e, None, None, cu0, cu0, 0, 0, False, scale, 256, 512,
                                                    tables=tables, kernel=UMMA).shape == (0, 2, 64)
    # empty batch and a batch whose second row is entirely padding
    eb = torch.empty(0, 2, 16, 64, dtype=DT, device="cuda")
    assert flash_attention_with_disentangled(eb, eb, eb, None, None, False, scale, 256, 512, tables=tables,
                                             kernel=UMMA).shape == (0, 2, 16, 64)
    w2 = _wl([100, 100], 100)
    q2, k2, v2, rel2, P2 = util.device_inputs(w2, DT)
    t2 = util.make_tables(w2, rel2, P2)
    lens = torch.tensor([100, 0], dtype=torch.int32, device="cuda")
    o2 = flash_attention_with_disentangled(q2.permute(0, 2, 1, 3), k2.permute(0, 2, 1, 3), v2.permute(0, 2, 1, 3), None,
                                           None, False, scale, 256, 512, seqlens=lens, tables=t2, kernel=UMMA)
    ref2 = util.oracle_fixed(q2, k2, v2, t2, [100, 0], w2, sm_scale=scale)
    util.assert_close(o2.permute(0, 2, 1, 3), ref2, DT, "row of padding only")
    assert torch.count_nonzero(o2[1]).item() == 0


def test_strided_views_and_lse():
    """q, k, v as slices of one fused [B, L, 3, H, D] buffer (non-trivial strides), and the optional LSE output."""
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    w = _wl([200, 77, 129], 200)
    q, k, v, rel, P = util.device_inputs(w, DT)
    tables = util.make_tables(w, rel, P)
    fused = torch.stack([q, k, v], dim=2).contiguous()                     # [B, L, 3, H, D]
    qs, ks, vs = (fused[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    scale = 1.0 / (3 * 64) ** 0.5
    lens = torch.as_tensor(np.asarray(w.lengths), dtype=torch.int32, device="cuda")
    o, lse = flash_attention_with_disentangled(qs, ks, vs, None, None, False, scale, 256, 512, seqlens=lens,
                                               tables=tables, kernel=UMMA, return_lse=True)
    ref = util.oracle_fixed(q, k, v, tables, w.lengths, w, sm_scale=scale)
    util.assert_close(o.permute(0, 2, 1, 3), ref, DT, "strided q/k/v")
    o2, lse2 = flash_attention_with_disentangled(qs, ks, vs, None, None, False, scale, 256, 512, seqlens=lens,
                                                 tables=tables, kernel=SIMT, return_lse=True)
    for b, n in enumerate(w.lengths):
        assert (lse[b, :, :n] - lse2[b, :, :n]).abs().max().item() < 5e-2


@pytest.mark.parametrize("mode", ["large", "negative", "rising"])
def test_umma_reference_exponent_moves(mode):
    """Scores far from zero: the rows have to move their reference exponent (first tile far below zero, later tiles
    far above the earlier ones), which rescales the running output; the small-score cases above never get there."""
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    w = _wl([512, 300], 512, hidden=128, heads=2, seed=77)
    q, k, v, rel, P = util.device_inputs(w, DT)
    tables = util.make_tables(w, rel, P)
    if mode == "large":                       # log2-scaled scores with a spread of tens
        q = (q.float() * 6.0).to(DT)
    elif mode == "negative":                  # every score of a row far below zero
        q = (torch.ones_like(q).float() + 0.05 * q.float()).to(DT)
        k = (-10.0 * torch.ones_like(k).float() + k.float()).to(DT)
    else:                                     # scores grow with the key position: every key tile raises the maximum
        ramp = torch.linspace(0.0, 4.0, k.shape[1], device=k.device)[None, :, None, None]
        q = (torch.ones_like(q).float() + 0.05 * q.float()).to(DT)
        k = (ramp * torch.ones_like(k).float() + 0.1 * k.float()).to(DT)
    scale = 1.0 / (3 * 64) ** 0.5
    lens = torch.as_tensor(np.asarray(w.lengths), dtype=torch.int32, device="cuda")
    o, lse = flash_attention_with_disentangled(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3),
                                               None, None, False, scale, 256, 512, seqlens=lens, tables=tables,
                                               kernel=UMMA, return_lse=True)
    ref = util.oracle_fixed(q, k, v, tables, w.lengths, w, sm_scale=scale)
    util.assert_close(o.permute(0, 2, 1, 3), ref, DT, f"exponent moves ({mode})")
    o2 = flash_attention_with_disentangled(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3),
                                           None, None, False, scale, 256, 512, seqlens=lens, tables=tables, kernel=SIMT)
    assert (o.float() - o2.float()).abs().max().item() < 2e-2
    assert torch.isfinite(lse).all()


def test_umma_many_single_tile_items():
    """Thousands of short sequences: every work item is one key tile, so each tile of the stream is an item's first
    and last at once (deferred epilogue, item hand-over and work ring all turn over at every step)."""
    from turbodeberta_b200.ops.flash_attention_varlen import flash_attention_with_disentangled_varlen
    rng = np.random.default_rng(123)
    lengths = rng.integers(1, 41, 3000)
    lengths[::97] = 0                                   # some empty sequences in between
    lengths[5] = 128; lengths[6] = 129                   # and a few that are exactly one tile / just over
    w = workloads.make_attention_workload("tiny", seed=124, hidden_size=128, num_heads=2, lengths=lengths,
                                          padded_len=None, dtype=DT)
    q, k, v, rel, P = util.device_inputs(w, DT)
    tables = util.make_tables(w, rel, P)
    cu = torch.as_tensor(np.asarray(w.cu_seqlens), dtype=torch.int32, device="cuda")
    scale = 1.0 / (3 * 64) ** 0.5
    mx = int(lengths.max())
    o = flash_attention_with_disentangled_varlen(q, k, v, None, None, cu, cu, mx, mx, False, scale, 256, 512,
                                                 tables=tables, kernel=UMMA)
    o2 = flash_attention_with_disentangled_varlen(q, k, v, None, None, cu, cu, mx, mx, False, scale, 256, 512,
                                                  tables=tables, kernel=SIMT)
    assert torch.isfinite(o.float()).all()
    assert (o.float() - o2.float()).abs().max().item() < 1e-2
    cuh = np.asarray(w.cu_seqlens)
    for b in (0, 5, 6, 1500, 2999):                      # and against the oracle on a few of them
        s, e = int(cuh[b]), int(cuh[b + 1])
        if e > s:
            ref = util.oracle_varlen(q[s:e], k[s:e], v[s:e], tables, np.array([0, e - s]), w, sm_scale=scale)
            util.assert_close(o[s:e], ref, DT, f"tiny sequence {b}")


def test_umma_repeated_runs_are_bitwise_identical():
    """Work items are handed out dynamically, but every tile is computed in a fixed order: the output must not depend
    on which CTA drew which item (a race on a staging row or a tensor-memory buffer would show up here)."""
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    w = _wl([512, 77, 300, 129, 64, 511, 1, 256], 512, hidden=256, heads=4, seed=55)
    q, k, v, rel, P = util.device_inputs(w, DT)
    tables = util.make_tables(w, rel, P)
    lens = torch.as_tensor(np.asarray(w.lengths), dtype=torch.int32, device="cuda")
    args = (q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), None, None, False, 0.0722, 256, 512)
    first = flash_attention_with_disentangled(*args, seqlens=lens, tables=tables, kernel=UMMA).clone()
    for _ in range(5):
        again = flash_attention_with_disentangled(*args, seqlens=lens, tables=tables, kernel=UMMA)
        assert torch.equal(first, again)


def test_padding_of_k_and_v_may_hold_anything():
    """Rows of K and V at or beyond a sequence's length are padding: the caller may leave NaN or infinities there.
    The probabilities of those keys are exact zeros, but 0 x NaN is NaN, so the kernel must not let those rows into the
    P.V product: results on the valid rows equal those with clean padding, bit for bit, in both kernels."""
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    w = _wl([200, 77, 129, 1], 256)
    q, k, v, rel, P = util.device_inputs(w, DT)
    tables = util.make_tables(w, rel, P)
    lens = torch.as_tensor(np.asarray(w.lengths), dtype=torch.int32, device="cuda")
    scale = 1.0 / (3 * 64) ** 0.5
    run = lambda kk, vv, kern: flash_attention_with_disentangled(
        q.permute(0, 2, 1, 3), kk.permute(0, 2, 1, 3), vv.permute(0, 2, 1, 3), None, None, False, scale, 256, 512,
        seqlens=lens, tables=tables, kernel=kern).permute(0, 2, 1, 3)
    kd, vd = k.clone(), v.clone()
    for b, n in enumerate(w.lengths):
        kd[b, n:] = float("nan")
        vd[b, n:] = float("nan")
        if n + 3 < 256:
            vd[b, n + 1] = float("inf")
            kd[b, n + 2] = float("-inf")
    for kern in (UMMA, SIMT):
        clean, dirty = run(k, v, kern), run(kd, vd, kern)
        assert torch.isfinite(dirty.float()).all()
        assert torch.equal(clean, dirty)
    ref = util.oracle_fixed(q, k, v, tables, w.lengths, w, True, True, scale)
    util.assert_close(run(kd, vd, UMMA), ref, DT, "dirty padding")


def test_long_padded_batch_mixes_band_tiles_saturated_tiles_and_dirty_padding():
    """A padded batch long enough for saturated key tiles (all distances of a 128 x 128 tile beyond the bucket table's
    span: their position terms ride in the score product) next to ordinary band tiles, with ragged lengths - so that
    saturated runs start and end inside items, last key tiles are partial, and whole query tiles are padding - and
    with NaN in the padding of K and V.  Valid rows must match the oracle; padded rows are zeros."""
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    lengths = [1536, 1100, 641, 130]
    w = _wl(lengths, 1536)
    q, k, v, rel, P = util.device_inputs(w, DT)
    tables = util.make_tables(w, rel, P)
    lens = torch.as_tensor(np.asarray(w.lengths), dtype=torch.int32, device="cuda")
    scale = 1.0 / (3 * 64) ** 0.5
    kd, vd = k.clone(), v.clone()
    for b, n in enumerate(lengths):
        kd[b, n:] = float("nan")
        vd[b, n:] = float("nan")
    out = flash_attention_with_disentangled(
        q.permute(0, 2, 1, 3), kd.permute(0, 2, 1, 3), vd.permute(0, 2, 1, 3), None, None, False, scale, 256, 512,
        seqlens=lens, tables=tables, kernel=UMMA).permute(0, 2, 1, 3)
    assert torch.isfinite(out.float()).all()
    for b, n in enumerate(lengths):
        assert torch.count_nonzero(out[b, n:]).item() == 0
    ref = util.oracle_fixed(q, k, v, tables, w.lengths, w, True, True, scale)
    util.assert_close(out, ref, DT, "long padded batch")
    simt = flash_attention_with_disentangled(
        q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), None, None, False, scale, 256, 512,
        seqlens=lens, tables=tables, kernel=SIMT).permute(0, 2, 1, 3)
    assert (out.float() - simt.float()).abs().max().item() < 1e-2


@pytest.mark.parametrize("c2p,p2c", [(True, False), (False, True)])
def test_long_sequences_with_one_position_term(c2p, p2c):
    """The long-sequence instantiations with a single position term: saturated tiles fold only that term into the
    score product, band tiles drain only that band."""
    o, ref = _fixed(_wl([1408, 700], 1408, hidden=64, heads=1), c2p=c2p, p2c=p2c)
    util.assert_close(o, ref, DT, f"long sequences, c2p={c2p}, p2c={p2c}")
