"""Pin the numpy restatement (oracle/) against the live eager module and the committed fixtures."""
import os

import numpy as np
import pytest
import torch

from oracle import disentangled_oracle as orc
from oracle import hf_eager
from tests.golden import make_golden as G
from turbodeberta_b200 import workloads

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def bucket_gold():
    return np.load(os.path.join(GOLD, "bucket_index.npz"))


@pytest.fixture(scope="module")
def att_gold():
    return np.load(os.path.join(GOLD, "attention_eager.npz"))


@pytest.mark.parametrize("pair", G.BUCKET_PAIRS)
def test_bucket_index_matches_fixture_and_live(pair, bucket_gold):
    b, m = pair
    dm = int(bucket_gold["delta_max"])
    mine = orc.gather_index_table(dm, b, m)
    assert np.array_equal(mine, bucket_gold[f"b{b}_m{m}"])
    assert np.array_equal(mine, hf_eager.hf_bucket_index(dm, b, m))


def test_bucket_known_answers():
    """Facts of the (256, 512) bucket function used by the kernels' table design."""
    d = np.arange(-8191, 8192)
    b = orc.relative_bucket(d, 256, 512)
    assert np.array_equal(b, -b[::-1])                       # odd function
    assert np.all(np.diff(b) >= 0) and np.all(np.diff(b) <= 1)
    assert np.array_equal(b[np.abs(d) <= 128], d[np.abs(d) <= 128])
    at = lambda x: int(b[x + 8191])
    assert [at(x) for x in (129, 130, 131, 132, 133)] == [129, 130, 131, 131, 132]
    assert at(505) == 254 and at(506) == 255 and at(511) == 255 and at(512) == 256 and at(8191) == 510
    idx = orc.gather_index(d, 256, 512)
    assert idx[506 + 8191] == 511 and idx[-512 + 8191] == 0 and idx[-511 + 8191] == 1 and idx[-506 + 8191] == 1
    assert idx.min() == 0 and idx.max() == 511


def _params_np(w):
    return {k: v.numpy() for k, v in w.params.items()}


@pytest.mark.parametrize("name", sorted(G.SMALL_CASES))
def test_module_restatement_matches_fixture_and_live(name, att_gold):
    spec = G.SMALL_CASES[name]
    w = G.small_workload(name)
    assert bytes(att_gold[name + "__fp"]).decode() == G.fingerprint(w), "seeded inputs drifted"
    rel = w.rel_embeddings.numpy() if len(spec[7]) else None
    mine = orc.self_attention_layer(w.hidden.numpy(), w.lengths, _params_np(w), num_heads=w.num_heads,
                                    position_buckets=w.position_buckets,
                                    max_relative_positions=w.max_relative_positions,
                                    share_att_key=spec[6], pos_att_type=spec[7], rel_embeddings=rel)
    live = hf_eager.attention_module_forward(w, share_att_key=spec[6], pos_att_type=spec[7],
                                             relative_attention=len(spec[7]) > 0).numpy()
    gold = att_gold[name]
    for b, n in enumerate(w.lengths):
        assert np.abs(mine[b, :n] - gold[b, :n]).max() < 2e-6
        assert np.abs(live[b, :n] - gold[b, :n]).max() < 2e-6
        assert np.all(mine[b, n:] == 0)


def test_config1_matches_fixture(att_gold):
    w = workloads.config1()
    assert bytes(att_gold["config1__fp"]).decode() == G.fingerprint(w)
    mine = orc.self_attention_layer(w.hidden.numpy(), w.lengths, _params_np(w), num_heads=12,
                                    position_buckets=256, max_relative_positions=512,
                                    rel_embeddings=w.rel_embeddings.numpy())
    gold = att_gold["config1_every8th"]
    err = np.abs(mine[:, ::8] - gold).max()
    assert err / np.abs(gold).max() < 1e-5


def test_varlen_equals_per_sequence_fixed():
    w = workloads.make_attention_workload("v", seed=5, hidden_size=128, num_heads=2, lengths=[5, 1, 33, 17],
                                          padded_len=None, dtype=torch.float32)
    q, k, v = [t.numpy() for t in workloads.project_qkv(w, dtype=torch.float32)]
    p = _params_np(w)
    rel = w.rel_embeddings.numpy()
    kr = orc.relpos_project(rel, p["key_proj.weight"], p["key_proj.bias"], 2)
    qr = orc.relpos_project(rel, p["query_proj.weight"], p["query_proj.bias"], 2)
    out = orc.attention_varlen(q, k, v, kr, qr, w.cu_seqlens, position_buckets=256, max_relative_positions=512)
    live = hf_eager.attention_module_forward_packed(w).numpy().reshape(out.shape)
    assert np.abs(out - live).max() < 2e-6


def test_layer_norm_matches_torch():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(64, 96, generator=g); wt = torch.randn(96, generator=g); bs = torch.randn(96, generator=g)
    ref = torch.nn.functional.layer_norm(x, (96,), wt, bs, 1e-7).numpy()
    assert np.abs(orc.layer_norm(x.numpy(), wt.numpy(), bs.numpy(), 1e-7) - ref).max() < 1e-5


def test_flop_accounting():
    assert orc.algorithmic_flops([512] * 32, 12, 64, 512) == pytest.approx(51.5e9, rel=2e-3)
    assert orc.algorithmic_flops([4096] * 4, 12, 64, 512) == pytest.approx(231.9e9, rel=2e-3)
    w = workloads.config2()
    assert w.flops() == orc.algorithmic_flops(w.lengths, 12, 64, 512)
    assert w.bytes(2) == orc.algorithmic_bytes(int(w.lengths.sum()), 12, 64, 512, 2, 32)


def test_materialised_scores_form_equals_table_form():
    """Gathering from materialised Q.Kr^T / K.Qr^T (the reference's operator interface, model.py:122-125) is the
    same arithmetic as the table form; the mirrored index differs from it exactly where idx(q-k) != idx(k-q)."""
    rng = np.random.default_rng(5)
    L, H, d, span = 70, 2, 64, 16
    q, k, v = (rng.standard_normal((L, H, d)) for _ in range(3))
    kr, qr = (0.3 * rng.standard_normal((H, 2 * span, d)) for _ in range(2))
    c2p = np.einsum("lhd,hrd->lhr", q, kr)
    p2c = np.einsum("lhd,hrd->lhr", k, qr)
    kw = dict(position_buckets=span, max_relative_positions=64)
    ref = orc.attention_single(q, k, v, kr, qr, **kw)
    got = orc.attention_single_scores(q, k, v, c2p, p2c, **kw)
    np.testing.assert_allclose(got, ref, rtol=0, atol=1e-12)
    only_c2p = orc.attention_single_scores(q, k, v, c2p, None, sm_scale=0.1, **kw)
    np.testing.assert_allclose(only_c2p, orc.attention_single(q, k, v, kr, None, p2c=False, sm_scale=0.1, **kw), atol=1e-12)
    mirrored = orc.attention_single_scores(q, k, v, c2p, p2c, p2c_mirrored=True, **kw)
    assert np.abs(mirrored - ref).max() > 1e-3
    # mirrored p2c of (q, k) equals the plain p2c with the roles of the distance swapped: check one element by hand
    idx = orc.gather_index(np.arange(L)[:, None] - np.arange(L)[None, :], span, 64)
    s_m = q[:, 0] @ k[:, 0].T + np.take_along_axis(c2p[:, 0], idx, 1) + np.take_along_axis(p2c[:, 0], idx, 1).T
    s_m = s_m / np.sqrt(3 * d)
    p = np.exp(s_m - s_m.max(1, keepdims=True)); p /= p.sum(1, keepdims=True)
    np.testing.assert_allclose(mirrored[:, 0], p @ v[:, 0], atol=1e-12)
