"""The reference's eager CPU path, driven directly (TEST INFRASTRUCTURE ONLY).

The reference package subclasses ``transformers``' ``DisentangledSelfAttention`` and
``DebertaV2Model`` (``src/turbodeberta/model.py:30,232``); their un-patched eager forward is the
behaviour the fused kernels must reproduce.  This wrapper builds those modules from a
seeded workload and runs them on the host.  Used by the tests (to pin the numpy
restatement and as the live checker), by ``tests/golden/make_golden.py`` and by the
CPU-baseline / reference legs of the benchmark.  The shipped package never imports it.
"""
from __future__ import annotations

import numpy as np
import torch


def _hf():
    from transformers import DebertaV2Config
    from transformers.models.deberta_v2 import modeling_deberta_v2 as m
    return DebertaV2Config, m


def hf_bucket_index(delta_max: int, position_buckets: int, max_relative_positions: int) -> np.ndarray:
    """clamp(bucket(delta)+span, 0, 2span-1) for delta in [-delta_max, delta_max], from the live
    ``make_log_bucket_position`` (modeling_deberta_v2.py:56-69) and the clamp at :317."""
    _, m = _hf()
    d = torch.arange(-delta_max, delta_max + 1, dtype=torch.long)
    if position_buckets > 0 and max_relative_positions > 0:
        b = m.make_log_bucket_position(d, position_buckets, max_relative_positions).to(torch.long)
    else:
        b = d
    span = position_buckets if position_buckets > 0 else max_relative_positions
    return torch.clamp(b + span, 0, 2 * span - 1).to(torch.int16).numpy()


def build_attention_module(w, share_att_key=True, pos_att_type=("c2p", "p2c"), relative_attention=True):
    """``DisentangledSelfAttention`` (fp32, eval) carrying the workload's parameters."""
    DebertaV2Config, m = _hf()
    cfg = DebertaV2Config(hidden_size=w.hidden_size, num_attention_heads=w.num_heads,
                          relative_attention=relative_attention, position_buckets=w.position_buckets,
                          max_relative_positions=w.max_relative_positions, share_att_key=share_att_key,
                          pos_att_type=list(pos_att_type), norm_rel_ebd="layer_norm",
                          hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
                          max_position_embeddings=max(512, w.max_relative_positions))
    mod = m.DisentangledSelfAttention(cfg).eval()
    sd = {k: v.clone() for k, v in w.params.items() if k in mod.state_dict()}
    missing = set(mod.state_dict()) - set(sd)
    if missing:
        raise KeyError(f"workload lacks parameters {sorted(missing)}")
    mod.load_state_dict(sd)
    return mod


@torch.no_grad()
def attention_module_forward(w, hidden=None, share_att_key=True, pos_att_type=("c2p", "p2c"),
                             relative_attention=True, module=None) -> torch.Tensor:
    """Eager forward on a padded workload: hidden ``[B, L, hidden]`` fp32, mask = m (x) m^T as the
    encoder builds it (modeling_deberta_v2.py:603-610).  Returns ``[B, L, hidden]`` fp32; rows of padded
    queries hold the eager module's uniform average and must be ignored by callers."""
    mod = module or build_attention_module(w, share_att_key, pos_att_type, relative_attention)
    x = (w.hidden if hidden is None else hidden).float()
    B, L, _ = x.shape
    lens = torch.as_tensor(np.asarray(w.lengths[:B]), dtype=torch.long)
    m2 = (torch.arange(L)[None, :] < lens[:, None])
    mask4 = (m2[:, None, :, None] & m2[:, None, None, :])
    rel = w.rel_embeddings.float() if relative_attention else None
    out, _ = mod(x, mask4, relative_pos=None, rel_embeddings=rel)
    return out


@torch.no_grad()
def attention_module_forward_packed(w, share_att_key=True, pos_att_type=("c2p", "p2c")) -> torch.Tensor:
    """Eager forward on a packed workload, one sequence at a time (hidden ``[T, hidden]``) -> ``[T, hidden]``."""
    mod = build_attention_module(w, share_att_key, pos_att_type)
    outs = []
    cu = w.cu_seqlens
    rel = w.rel_embeddings.float()
    for b in range(len(w.lengths)):
        x = w.hidden[cu[b]:cu[b + 1]].float()[None]
        L = x.shape[1]
        mask4 = torch.ones(1, 1, L, L, dtype=torch.bool)
        o, _ = mod(x, mask4, relative_pos=None, rel_embeddings=rel)
        outs.append(o[0])
    return torch.cat(outs, 0)
