"""GPU parity of the CUDA-core attention kernel (the full-precision path) against the oracle."""
import os

import numpy as np
import pytest
import torch

from tests import util
from tests.golden import make_golden as G
from turbodeberta_b200 import workloads

pytestmark = pytest.mark.gpu
SIMT = 1


def _run_fixed(w, dtype, c2p=True, p2c=True, share=True, kernel=SIMT, with_lens=True):
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    q, k, v, rel, P = util.device_inputs(w, dtype)
    tables = util.make_tables(w, rel, P, c2p, p2c, share) if (c2p or p2c) else None
    d = w.head_dim
    scale = 1.0 / (d * (1 + int(c2p) + int(p2c))) ** 0.5
    lens = torch.as_tensor(np.asarray(w.lengths), dtype=torch.int32, device="cuda") if with_lens else None
    o = flash_attention_with_disentangled(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3),
                                          None, None, False, scale, w.position_buckets, w.max_relative_positions,
                                          seqlens=lens, tables=tables, kernel=kernel)
    ref = util.oracle_fixed(q, k, v, tables, w.lengths if with_lens else None, w, c2p, p2c, scale)
    return o.permute(0, 2, 1, 3), ref


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", sorted(G.SMALL_CASES))
def test_simt_small_cases(name, dtype):
    spec = G.SMALL_CASES[name]
    w = G.small_workload(name)
    c2p, p2c = "c2p" in spec[7], "p2c" in spec[7]
    o, ref = _run_fixed(w, dtype, c2p, p2c, share=spec[6])
    util.assert_close(o, ref, dtype, name)


def test_simt_config1_fp32_matches_eager_fixture():
    """Configuration 1 end to end at the op level: fp32, batch 2 x 128, against the committed eager output."""
    w = workloads.config1()
    o, ref = _run_fixed(w, torch.float32)
    util.assert_close(o, ref, torch.float32, "config1 vs oracle")
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "attention_eager.npz"))["config1_every8th"]
    got = o.reshape(2, 128, 768)[:, ::8].float().cpu().numpy()
    assert np.abs(got - gold).max() / np.abs(gold).max() < util.FP32_REL_TOL


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_simt_varlen(dtype):
    from turbodeberta_b200.ops.flash_attention_varlen import flash_attention_with_disentangled_varlen
    w = workloads.make_attention_workload("v", seed=21, hidden_size=128, num_heads=2,
                                          lengths=[5, 1, 33, 17, 128, 129, 600], padded_len=None, dtype=dtype)
    q, k, v, rel, P = util.device_inputs(w, dtype)
    tables = util.make_tables(w, rel, P)
    cu = torch.as_tensor(w.cu_seqlens, device="cuda")
    scale = 1.0 / (3 * 64) ** 0.5
    o, lse = flash_attention_with_disentangled_varlen(q, k, v, None, None, cu, cu, 600, 600, False, scale, 256, 512,
                                                      tables=tables, kernel=SIMT, return_lse=True)
    ref = util.oracle_varlen(q, k, v, tables, w.cu_seqlens, w, sm_scale=scale)
    util.assert_close(o, ref, dtype, "varlen")
    assert torch.isfinite(lse).all()


def test_argument_errors():
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    q = torch.zeros(1, 2, 16, 32, device="cuda")
    with pytest.raises(ValueError):
        flash_attention_with_disentangled(q, q, q, None, None)                  # head_dim 32
    q = torch.zeros(1, 2, 16, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(ValueError):
        flash_attention_with_disentangled(q, q, q, None, None)                  # fp16
    q = torch.zeros(1, 2, 16, 64, device="cuda")
    with pytest.raises(ValueError):
        flash_attention_with_disentangled(q, q, q, torch.zeros(1, 2, 16, 300, device="cuda"), None,
                                          position_buckets=256, max_relative_distance=512)   # 300 columns are neither
    o = flash_attention_with_disentangled(q, q, q, torch.zeros(1, 2, 16, 512, device="cuda"), None,
                                          position_buckets=256, max_relative_distance=512)   # materialised scores
    assert o.shape == q.shape and torch.isfinite(o).all()
    with pytest.raises(RuntimeError):
        flash_attention_with_disentangled(q.cpu(), q.cpu(), q.cpu(), None, None)            # no CPU path
    with pytest.raises(NotImplementedError):
        flash_attention_with_disentangled(q, q, q, None, None, causal=True)


def test_understated_max_seqlen_and_short_offsets_are_reported():
    """The CUDA-core kernel sizes its grid from max_seqlen: a value below the longest sequence, or offsets that stop
    short of the token count, must come back as an error instead of rows that were never written."""
    from turbodeberta_b200.ops.flash_attention_varlen import flash_attention_with_disentangled_varlen
    w = workloads.make_attention_workload("v", seed=22, hidden_size=128, num_heads=2, lengths=[40, 200],
                                          padded_len=None, dtype=torch.float32)
    q, k, v, rel, P = util.device_inputs(w, torch.float32)
    tables = util.make_tables(w, rel, P)
    cu = torch.as_tensor(w.cu_seqlens, device="cuda")
    args = (False, 1.0 / (3 * 64) ** 0.5, 256, 512)
    with pytest.raises(ValueError, match="max_seqlen"):
        flash_attention_with_disentangled_varlen(q, k, v, None, None, cu, cu, 64, 64, *args, tables=tables, kernel=SIMT)
    short = cu.clone()
    short[-1] -= 8
    with pytest.raises(ValueError, match="cu_seqlens"):
        flash_attention_with_disentangled_varlen(q, k, v, None, None, short, short, 200, 200, *args, tables=tables,
                                                 kernel=SIMT)
    other = cu.clone()
    other[1] += 1                                          # key offsets that differ from the query offsets
    with pytest.raises(ValueError, match="key offsets"):
        flash_attention_with_disentangled_varlen(q, k, v, None, None, cu, other, 200, 200, *args, tables=tables)
    o = flash_attention_with_disentangled_varlen(q, k, v, None, None, cu, cu.clone(), 200, 200, *args, tables=tables)
    assert torch.isfinite(o).all()


def test_backward_raises_like_the_reference():
    """Forward-only (the reference raises in backward, ``ops/flash_attention.py:341-343``): a loss built on the output
    must fail loudly instead of training with no gradient through the attention."""
    from turbodeberta_b200.ops.flash_attention import flash_attention_with_disentangled
    from turbodeberta_b200.ops.flash_attention_varlen import flash_attention_with_disentangled_varlen
    q = torch.randn(1, 2, 16, 64, device="cuda", requires_grad=True)
    o = flash_attention_with_disentangled(q, q.detach(), q.detach(), None, None)
    assert o.requires_grad
    with pytest.raises(RuntimeError, match="forward-only"):
        o.sum().backward()
    qp = torch.randn(16, 2, 64, device="cuda", requires_grad=True)
    cu = torch.tensor([0, 16], dtype=torch.int32, device="cuda")
    o = flash_attention_with_disentangled_varlen(qp, qp.detach(), qp.detach(), None, None, cu, cu, 16, 16)
    with pytest.raises(RuntimeError, match="forward-only"):
        o.sum().backward()
    scores = torch.zeros(1, 2, 16, 512, device="cuda")
    with pytest.raises(RuntimeError, match="forward-only"):           # score-tensor form: refused before the launch
        flash_attention_with_disentangled(q, q, q, scores, None, position_buckets=256, max_relative_distance=512)
    with torch.no_grad():
        o = flash_attention_with_disentangled(q, q, q, scores, None, position_buckets=256, max_relative_distance=512)
    assert not o.requires_grad
