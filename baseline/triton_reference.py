#!/usr/bin/env python
"""Times the reference's own Triton kernels on this GPU, next to the sm_100a kernels of this repository.

    python baseline/triton_reference.py [--cases c2full,c4layer,c3] [--steps K] [--warmup W]

The reference package is imported, unmodified, from ``baseline/_ref/src`` (a plain copy of its ``src`` tree made by
``__graft_entry__.build()``; git-ignored).  What is timed is the reference's public operator call, as its attention
module makes it (``model.py:122-137`` fixed, ``:143-182`` packed):

* ``fixed``: ``flash_attention_with_disentangled(q, k, v, pos_key, pos_query, ...)`` on contiguous ``(B, H, L, D)``
  tensors, once with the two materialised ``(B, H, L, 2*span)`` score tensors prepared outside the timer and once
  with the two batched matmuls that build them (``model.py:122-125``) inside it;
* ``varlen``: ``flash_attention_with_disentangled_varlen`` on the packed stream.  TIMING ONLY: that kernel is
  numerically wrong upstream (``ops/flash_attention_varlen.py:111`` masks keys by the batch maximum, ``:152``
  advances the position pointer by the wrong stride).  Its stray reads stay below 64 token rows past the end of its
  inputs, so every input is allocated with 64 spare rows.

Results are NOT compared with the eager module (the reference kernel mirrors the position->content index).
One JSON object is printed.  Nothing of this repository's kernels runs in this process.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF_SRC = os.path.join(HERE, "_ref", "src")


def _time(fn, steps, warmup, flush):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return {"ms_median": ts[len(ts) // 2], "ms_min": ts[0]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", default="c2full,c4layer,c3")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    if not os.path.isdir(os.path.join(REF_SRC, "turbodeberta")):
        print(json.dumps({"unavailable": "baseline/_ref/src is missing (made by __graft_entry__.build() where the reference tree is present)"}))
        return
    sys.path.insert(0, ROOT)            # turbodeberta_b200.workloads: the seeded inputs (no kernels of this repo)
    sys.path.insert(0, REF_SRC)         # ... and ahead of it the reference, so `turbodeberta` is the reference's package
    import numpy as np
    import torch
    out = {"triton": None, "device": None, "cases": {}}
    try:
        import triton
        out["triton"] = triton.__version__
        import turbodeberta.ops.flash_attention as fa
        import turbodeberta.ops.flash_attention_varlen as fav
        assert os.path.abspath(fa.__file__).startswith(os.path.abspath(REF_SRC)), fa.__file__
    except Exception as e:
        print(json.dumps({"unavailable": f"importing the reference failed: {type(e).__name__}: {e}"}))
        return
    from turbodeberta_b200 import workloads
    dev = torch.device("cuda", 0)
    out["device"] = torch.cuda.get_device_name(0)
    dt = torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    scale = 1.0 / (3 * 64) ** 0.5

    def tables_of(w):
        """Projected relative tables [1, H, 2*span, D] computed with torch (what model.py:95-100 does)."""
        rel = w.rel_embeddings.to(dev, dt)
        H, D = w.num_heads, w.head_dim
        kr = torch.nn.functional.linear(rel, w.params["key_proj.weight"].to(dev, dt), w.params["key_proj.bias"].to(dev, dt))
        qr = torch.nn.functional.linear(rel, w.params["query_proj.weight"].to(dev, dt), w.params["query_proj.bias"].to(dev, dt))
        f = lambda t: t.view(1, -1, H, D).permute(0, 2, 1, 3).contiguous()
        return f(kr), f(qr)

    def fixed_case(name, w):
        q, k, v = workloads.project_qkv(w, device=dev, dtype=dt)                     # [B, L, H, D]
        q, k, v = (t.permute(0, 2, 1, 3).contiguous() for t in (q, k, v))            # the reference's transform()
        kr, qr = tables_of(w)
        B, H, L, D = q.shape
        cfg = fa.get_fwd_config(B, H, L, L, D, False)
        pos_key = torch.matmul(q, kr.transpose(-1, -2))
        pos_query = torch.matmul(k, qr.transpose(-1, -2))
        call = lambda pk, pq: fa.flash_attention_with_disentangled(q, k, v, pk, pq, False, scale, w.position_buckets,
                                                                   w.max_relative_positions)
        o = call(pos_key, pos_query)
        torch.cuda.synchronize()
        finite = bool(torch.isfinite(o.float()).all())
        t_k = _time(lambda: call(pos_key, pos_query), a.steps, a.warmup, flush)

        def with_bias():
            pk = torch.matmul(q, kr.transpose(-1, -2))
            pq = torch.matmul(k, qr.transpose(-1, -2))
            return call(pk, pq)
        t_b = _time(with_bias, a.steps, a.warmup, flush)
        fl = w.flops()
        out["cases"][name] = {
            "workload": w.name, "op": "flash_attention_with_disentangled (ops/flash_attention.py:345)",
            "tile_config_block_m_n_stages_warps": list(cfg), "output_finite": finite,
            "kernel_only": dict(t_k, algorithmic_tflops=fl / (t_k["ms_median"] * 1e-3) / 1e12),
            "with_bias_materialisation": dict(t_b, algorithmic_tflops=fl / (t_b["ms_median"] * 1e-3) / 1e12),
            "bias_tensors_bytes": 2 * pos_key.numel() * 2, "algorithmic_flops": fl}

    def varlen_case(name, w):
        q, k, v = workloads.project_qkv(w, device=dev, dtype=dt)                     # [T, H, D]
        T, H, D = q.shape
        PADR = 64                                                                     # rows the kernel's stray reads may touch

        def padded(t):
            buf = torch.zeros((T + PADR,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev)
            buf[:T] = t
            return buf[:T]
        q, k, v = padded(q), padded(k), padded(v)
        kr, qr = tables_of(w)
        cu = torch.as_tensor(w.cu_seqlens, device=dev)
        mx = int(w.lengths.max())
        pos_key = padded(torch.einsum("qhd,hmd->qhm", q, kr[0]))
        pos_query = padded(torch.einsum("qhd,hmd->qhm", k, qr[0]))
        aM = T // len(w.lengths)
        cfg = fav.get_fwd_config(aM, D, False)
        call = lambda: fav.flash_attention_with_disentangled_varlen(q, k, v, pos_key, pos_query, cu, cu, mx, mx, False,
                                                                     scale, w.position_buckets, w.max_relative_positions)
        call()
        torch.cuda.synchronize()
        t_k = _time(call, a.steps, a.warmup, flush)
        fl = w.flops()
        out["cases"][name] = {
            "workload": w.name, "op": "flash_attention_with_disentangled_varlen (ops/flash_attention_varlen.py:348)",
            "tile_config_block_m_n_stages_warps": list(cfg),
            "note": "timing only: numerically incorrect upstream; includes the operator's host loop over sequences "
                    "(one device->host read per sequence) and its two host->device copies",
            "kernel_only": dict(t_k, algorithmic_tflops=fl / (t_k["ms_median"] * 1e-3) / 1e12),
            "bias_tensors_bytes": 2 * pos_key.numel() * 2, "algorithmic_flops": fl}

    for case in a.cases.split(","):
        try:
            if case == "c2full":
                w = workloads.config2(seed=1002)
                w.lengths = np.full_like(w.lengths, 512)
                w.name = "c2_base_bf16_b32_l512_allvalid"
                fixed_case(case, w)
            elif case == "c4layer":
                w = workloads.make_attention_workload("c4_one_layer_b256_l512_h16", seed=1004, hidden_size=1024, num_heads=16,
                                                      lengths=[512] * 256, padded_len=512, dtype=dt)
                fixed_case(case, w)
            elif case == "c3":
                varlen_case(case, workloads.config3(seed=1003))
            else:
                out["cases"][case] = {"unavailable": "unknown case"}
        except Exception as e:                                   # compile or launch error: record it, do not retry
            out["cases"][case] = {"unavailable": f"{type(e).__name__}: {str(e)[:300]}"}
            if "CUDA" in str(e) or "illegal" in str(e).lower():
                break                                            # the context may be gone: stop here
        torch.cuda.empty_cache()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
