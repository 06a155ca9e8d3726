"""Helpers shared by the GPU parity tests: run an op through the package and compare with the oracle."""
import numpy as np
import torch

from oracle import disentangled_oracle as orc
from turbodeberta_b200 import workloads

BF16_ABS_TOL = 2e-2       # bf16 outputs vs the fp32/fp64 result on the same bf16-rounded inputs
FP32_REL_TOL = 1e-4       # fp32 outputs: max |x - ref| / max |ref|
# Whole models.  fp32: 24 layers of fp32 GEMMs on two different devices (different summation orders) on top of the
# attention's 1e-4; measured differences sit near 1e-5, the bound leaves one order of magnitude.
MODEL_FP32_REL_TOL = 5e-4
# bf16: every layer rounds its activations to 8 bits of mantissa, so a 24-layer bf16 model is some 1e-2..1e-1 away
# from the fp32 model whatever the attention kernel.  The yardstick is therefore the eager model ITSELF run in bf16:
# the fused model may be at most this factor further from the fp32 result than eager-bf16 is (max abs and RMS), which
# is what "the fused attention adds no error of its own" means at model level.
MODEL_BF16_VS_EAGER_FACTOR = 1.5


def f64(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy().astype(np.float64)


def device_inputs(w, dtype, device="cuda"):
    """q, k, v ([..., H, D], token-major) and tables computed on the device in `dtype`."""
    from turbodeberta_b200 import relpos
    q, k, v = workloads.project_qkv(w, device=device, dtype=dtype)
    rel = w.rel_embeddings.to(device=device, dtype=dtype)
    P = {n: t.to(device=device, dtype=dtype) for n, t in w.params.items()}
    return q, k, v, rel, P


def make_tables(w, rel, P, c2p=True, p2c=True, share=True):
    from turbodeberta_b200 import relpos
    kn, qn = ("key_proj", "query_proj") if share else ("pos_key_proj", "pos_query_proj")
    return relpos.build_tables(rel, num_heads=w.num_heads, position_buckets=w.position_buckets,
                               max_relative_positions=w.max_relative_positions,
                               key_weight=P[kn + ".weight"], key_bias=P[kn + ".bias"],
                               query_weight=P[qn + ".weight"], query_bias=P[qn + ".bias"], c2p=c2p, p2c=p2c)


def oracle_fixed(q, k, v, tables, lengths, w, c2p=True, p2c=True, sm_scale=None):
    kr = f64(tables.kr) if (c2p and tables is not None) else None
    qr = f64(tables.qr) if (p2c and tables is not None) else None
    return orc.attention_fixed(f64(q), f64(k), f64(v), kr, qr, lengths, position_buckets=w.position_buckets,
                               max_relative_positions=w.max_relative_positions, c2p=c2p, p2c=p2c, sm_scale=sm_scale)


def oracle_varlen(q, k, v, tables, cu, w, c2p=True, p2c=True, sm_scale=None):
    kr = f64(tables.kr) if (c2p and tables is not None) else None
    qr = f64(tables.qr) if (p2c and tables is not None) else None
    return orc.attention_varlen(f64(q), f64(k), f64(v), kr, qr, cu, position_buckets=w.position_buckets,
                                max_relative_positions=w.max_relative_positions, c2p=c2p, p2c=p2c, sm_scale=sm_scale)


def assert_close(out: torch.Tensor, ref: np.ndarray, dtype, what=""):
    got = f64(out)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite values in the output"
    err = np.abs(got - ref).max() if got.size else 0.0
    if dtype == torch.float32:
        rel = err / max(np.abs(ref).max(), 1e-30)
        assert rel <= FP32_REL_TOL, f"{what}: fp32 max rel error {rel:.3e} > {FP32_REL_TOL}"
    else:
        assert err <= BF16_ABS_TOL, f"{what}: bf16 max abs error {err:.3e} > {BF16_ABS_TOL}"
    return err
