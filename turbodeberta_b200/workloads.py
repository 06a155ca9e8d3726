"""Seeded synthetic inputs for the five benchmark/parity configurations.

Everything is drawn on the CPU (``torch.Generator`` for tensors, ``numpy.random.default_rng`` for
lengths) so that values do not depend on the device; callers cast and move afterwards.
No dataset is involved: hidden states ~N(0,1), weights ~N(0,0.02), biases zero, relative
embeddings ~N(0,0.02), as the configurations prescribe.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class AttentionWorkload:
    """One attention-layer problem: module parameters plus hidden states and valid lengths."""
    name: str
    hidden_size: int
    num_heads: int
    head_dim: int
    position_buckets: int
    max_relative_positions: int
    lengths: np.ndarray                 # valid length of each sequence
    padded_len: int | None              # L for the fixed (padded) form, None for packed
    hidden: torch.Tensor                # fixed: [B, L, hidden]; packed: [T, hidden]   (fp32, CPU)
    params: dict = field(default_factory=dict)   # HF parameter names -> fp32 CPU tensors
    rel_embeddings: torch.Tensor | None = None   # [2*span, hidden] as handed to the module (post LayerNorm)
    dtype: torch.dtype = torch.bfloat16

    @property
    def two_span(self) -> int:
        return 2 * (self.position_buckets if self.position_buckets > 0 else self.max_relative_positions)

    @property
    def cu_seqlens(self) -> np.ndarray:
        return np.concatenate([[0], np.cumsum(self.lengths)]).astype(np.int32)

    def flops(self) -> float:
        """4 L^2 d + 4 L R d per sequence and head, R = min(2*span, 2L-1)."""
        tot = 0.0
        for L in self.lengths:
            L = int(L)
            R = min(self.two_span, max(2 * L - 1, 0))
            tot += 4.0 * L * L * self.head_dim + 4.0 * L * R * self.head_dim
        return tot * self.num_heads

    def bytes(self, elem: int) -> float:
        T = int(np.sum(self.lengths))
        return elem * (4.0 * T * self.num_heads * self.head_dim
                       + 2.0 * self.two_span * self.num_heads * self.head_dim) + 4.0 * (len(self.lengths) + 1)


def _module_params(gen: torch.Generator, hidden: int, share_att_key: bool = True) -> dict:
    p = {}
    names = ["query_proj", "key_proj", "value_proj"]
    if not share_att_key:
        names += ["pos_key_proj", "pos_query_proj"]
    for n in names:
        p[n + ".weight"] = torch.randn(hidden, hidden, generator=gen) * 0.02
        p[n + ".bias"] = torch.zeros(hidden)
    return p


def make_attention_workload(name: str, *, seed: int, hidden_size: int, num_heads: int, lengths,
                            padded_len: int | None, position_buckets: int = 256,
                            max_relative_positions: int = 512, share_att_key: bool = True,
                            dtype: torch.dtype = torch.bfloat16) -> AttentionWorkload:
    gen = torch.Generator().manual_seed(seed)
    lengths = np.asarray(lengths, dtype=np.int64)
    if padded_len is None:
        hidden = torch.randn(int(lengths.sum()), hidden_size, generator=gen)
    else:
        hidden = torch.randn(len(lengths), padded_len, hidden_size, generator=gen)
    span = position_buckets if position_buckets > 0 else max_relative_positions
    rel = torch.randn(2 * span, hidden_size, generator=gen) * 0.02
    params = _module_params(gen, hidden_size, share_att_key)
    return AttentionWorkload(name=name, hidden_size=hidden_size, num_heads=num_heads,
                             head_dim=hidden_size // num_heads, position_buckets=position_buckets,
                             max_relative_positions=max_relative_positions, lengths=lengths,
                             padded_len=padded_len, hidden=hidden, params=params,
                             rel_embeddings=rel, dtype=dtype)


def config1() -> AttentionWorkload:
    """v3-base layer, fp32, batch 2 x seq 128, all-ones mask."""
    return make_attention_workload("c1_base_fp32_b2_l128", seed=1001, hidden_size=768, num_heads=12,
                                   lengths=[128, 128], padded_len=128, dtype=torch.float32)


def config2(batch: int = 32, seq: int = 512, seed: int = 1002) -> AttentionWorkload:
    """v3-base heads, bf16, batch 32 x seq 512, valid lengths uniform in [64, 512], right padded."""
    rng = np.random.default_rng(seed)
    lengths = rng.integers(64, seq + 1, batch)
    return make_attention_workload(f"c2_base_bf16_b{batch}_l{seq}_padded", seed=seed, hidden_size=768,
                                   num_heads=12, lengths=lengths, padded_len=seq)


def config3(n_seqs: int = 256, seed: int = 1003) -> AttentionWorkload:
    """v3-large heads, bf16, 256 packed sequences with lengths log-uniform in [16, 1024]."""
    rng = np.random.default_rng(seed)
    lengths = np.floor(np.exp(rng.uniform(math.log(16), math.log(1024), n_seqs))).astype(np.int64)
    return make_attention_workload(f"c3_large_bf16_{n_seqs}seqs_packed", seed=seed, hidden_size=1024,
                                   num_heads=16, lengths=lengths, padded_len=None)


def config5_fixed(batch: int = 4, seq: int = 4096, seed: int = 1005) -> AttentionWorkload:
    """v3-base heads, bf16, batch 4 x seq 4096, all valid."""
    return make_attention_workload(f"c5_base_bf16_b{batch}_l{seq}", seed=seed, hidden_size=768, num_heads=12,
                                   lengths=[seq] * batch, padded_len=seq)


def config5_varlen(n_seqs: int = 64, seed: int = 1005, lo: int = 2048, hi: int = 8192) -> AttentionWorkload:
    """v3-base heads, bf16, 64 packed sequences with lengths uniform in [2048, 8192]."""
    rng = np.random.default_rng(seed)
    lengths = rng.integers(lo, hi + 1, n_seqs)
    return make_attention_workload(f"c5_base_bf16_{n_seqs}seqs_packed", seed=seed, hidden_size=768,
                                   num_heads=12, lengths=lengths, padded_len=None)


def project_qkv(w: AttentionWorkload, device="cpu", dtype=None):
    """Q, K, V = the three Linear projections of the hidden states, shaped ``[..., H, d]``
    (token-major, heads split by a view, no transposition), plus the per-head relative tables
    input ``rel_embeddings`` cast to the same dtype."""
    dtype = dtype or w.dtype
    h = w.hidden.to(device=device, dtype=dtype)
    out = []
    for n in ("query_proj", "key_proj", "value_proj"):
        W = w.params[n + ".weight"].to(device=device, dtype=dtype)
        b = w.params[n + ".bias"].to(device=device, dtype=dtype)
        y = torch.nn.functional.linear(h, W, b)
        out.append(y.view(*y.shape[:-1], w.num_heads, w.head_dim))
    return out
