"""GPU parity of the once-per-layer kernels: bucket index (bit-exact), projection, expansion."""
import os

import numpy as np
import pytest
import torch

from oracle import disentangled_oracle as orc
from tests.golden import make_golden as G

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("pair", G.BUCKET_PAIRS)
def test_bucket_table_bit_exact(pair):
    from turbodeberta_b200 import relpos
    b, m = pair
    gold = np.load(os.path.join(GOLD, "bucket_index.npz"))
    dm = int(gold["delta_max"])
    t = relpos.bucket_index_table(b, m, dm, "cuda")
    assert np.array_equal(t.cpu().numpy(), gold[f"b{b}_m{m}"])
    assert np.array_equal(t.cpu().numpy(), orc.gather_index_table(dm, b, m))


@pytest.mark.parametrize("pair", [(256, 512), (64, 128), (101, 300), (0, 64), (32, 512)])
def test_saturation_distance_is_safe(pair):
    """Beyond the saturation distance the row index must not change any more."""
    from turbodeberta_b200 import relpos
    b, m = pair
    sat = relpos.saturation_distance(b, m)
    idx = orc.gather_index_table(4 * sat + 64, b, m)
    dm = 4 * sat + 64
    assert np.all(idx[dm + sat:] == idx[-1]) and np.all(idx[: dm - sat + 1] == idx[0])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,heads,two_span", [(128, 2, 512), (768, 12, 512), (192, 3, 100)])
def test_relpos_project(dtype, hidden, heads, two_span):
    from turbodeberta_b200 import relpos
    g = torch.Generator().manual_seed(11)
    rel = (torch.randn(two_span, hidden, generator=g) * 0.5).to("cuda", dtype)
    W = (torch.randn(hidden, hidden, generator=g) * 0.05).to("cuda", dtype)
    bias = (torch.randn(hidden, generator=g) * 0.1).to("cuda", dtype)
    out = relpos.project(rel, W, bias, heads)
    ref = orc.relpos_project(rel.float().cpu().numpy(), W.float().cpu().numpy(), bias.float().cpu().numpy(), heads)
    err = np.abs(out.float().cpu().numpy() - ref).max()
    scale = np.abs(ref).max()
    assert err / scale < (1e-5 if dtype == torch.float32 else 8e-3)
    out2 = relpos.project(rel, W, None, heads)
    ref2 = orc.relpos_project(rel.float().cpu().numpy(), W.float().cpu().numpy(), None, heads)
    assert np.abs(out2.float().cpu().numpy() - ref2).max() / scale < (1e-5 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("pair", [(256, 512), (0, 64), (32, 64)])
def test_relpos_expand(pair):
    from turbodeberta_b200 import relpos
    b, m = pair
    span = b if b > 0 else m
    g = torch.Generator().manual_seed(5)
    table = torch.randn(3, 2 * span, 64, generator=g).to("cuda", torch.bfloat16)
    sat = relpos.saturation_distance(b, m)
    idx = relpos.bucket_index_table(b, m, sat + 1, "cuda")
    edm = sat + 256
    out = relpos.expand(table, idx, edm)
    rows = out.shape[1]
    assert rows % 8 == 0 and rows >= 2 * edm + 1
    delta = np.clip(np.arange(rows) - edm, -(sat + 1), sat + 1)
    rix = orc.gather_index(delta, b, m)
    ref = table.cpu()[:, torch.as_tensor(rix), :]
    assert torch.equal(out.cpu(), ref)
