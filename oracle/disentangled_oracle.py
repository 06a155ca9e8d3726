"""CPU restatement of DeBERTa-v2/v3 disentangled self-attention (TEST INFRASTRUCTURE ONLY).

This module is the parity checker for the CUDA kernels.  It is never imported by the
shipped package: only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark may use it.  It restates, in plain numpy, the arithmetic that the reference
package (Ingvarstep/TurboDeBERTa) inherits from its third-party dependency
``transformers`` (``models/deberta_v2/modeling_deberta_v2.py``, pinned here to the
installed release 5.5.0; the reference itself only constrains ``transformers>=4.30.0``
in ``pyproject.toml:12``).  Line numbers below written ``HF:n`` refer to that file;
``model.py`` / ``ops/...`` refer to files under ``src/turbodeberta/`` of the reference.

Pinning: ``tests/test_oracle_cpu.py`` checks every function here against the live
``transformers`` module (bucket indices exactly, attention to 2e-6) and against the
committed fixtures in ``tests/golden/`` that were generated from that module by
``tests/golden/make_golden.py``.  The reference ships no tests or golden vectors.

Deliberate deviation from the reference's Triton kernels: ``ops/flash_attention.py:127``
indexes the position->content term with ``span - bucket(q-k)`` whereas the eager module
the reference subclasses (HF:327-343) reduces to ``span + bucket(q-k)``.  The parity
target is the eager module, so this restatement follows HF.
"""
from __future__ import annotations

import math

import numpy as np

__all__ = [
    "make_log_bucket_position",
    "relative_bucket",
    "gather_index",
    "gather_index_table",
    "layer_norm",
    "relpos_project",
    "attention_single",
    "attention_varlen",
    "attention_fixed",
    "self_attention_layer",
    "algorithmic_flops",
    "algorithmic_bytes",
]


# --------------------------------------------------------------------------- buckets
def make_log_bucket_position(relative_pos: np.ndarray, bucket_size: int, max_position: int) -> np.ndarray:
    """Float32 log-bucket of signed distances, following HF:56-69 operation by operation.

    ``relative_pos`` is an integer array of q-k distances.  Every intermediate is float32,
    as in the eager module (the integer distance is divided by ``mid`` in float32, the
    denominator is the float32 rounding of the python double ``(max_position-1)/mid``).
    The reference's kernels restate the same formula per score element
    (``ops/flash_attention.py:100-115``, ``ops/flash_attention_varlen.py:118-133``).
    """
    rel = np.asarray(relative_pos, dtype=np.int64)
    sign = np.sign(rel).astype(np.float32)
    mid = bucket_size // 2
    abs_pos = np.where((rel < mid) & (rel > -mid), mid - 1, np.abs(rel)).astype(np.int64)
    ratio = abs_pos.astype(np.float32) / np.float32(mid)
    denom = np.log(np.float32((max_position - 1) / mid))
    with np.errstate(divide="ignore", invalid="ignore"):
        log_pos = np.ceil(np.log(ratio) / denom * np.float32(mid - 1)) + np.float32(mid)
    log_pos = log_pos.astype(np.float32)
    return np.where(abs_pos <= mid, rel.astype(np.float32), log_pos * sign).astype(np.float32)


def relative_bucket(delta: np.ndarray, position_buckets: int, max_relative_positions: int) -> np.ndarray:
    """Integer bucket of q-k distances (HF:72-101): log-bucketed when both sizes are > 0,
    otherwise the distance itself; truncated to int64 like ``.to(torch.long)``."""
    delta = np.asarray(delta, dtype=np.int64)
    if position_buckets > 0 and max_relative_positions > 0:
        return make_log_bucket_position(delta, position_buckets, max_relative_positions).astype(np.int64)
    return delta


def att_span(position_buckets: int, max_relative_positions: int) -> int:
    """Half-width of the relative-embedding table the module uses (HF:168-174)."""
    return position_buckets if position_buckets > 0 else max_relative_positions


def gather_index(delta: np.ndarray, position_buckets: int, max_relative_positions: int) -> np.ndarray:
    """Row of the projected relative-embedding tables used for distance ``delta = q - k``.

    HF:317 computes ``clamp(bucket(q-k) + span, 0, 2*span-1)`` for the content->position term.
    For position->content HF:336 computes ``clamp(-bucket(k-q) + span, ...)`` on the transposed
    matrix, and because the bucket function is odd this is the same number, so one index
    serves both terms.
    """
    span = att_span(position_buckets, max_relative_positions)
    b = relative_bucket(delta, position_buckets, max_relative_positions)
    return np.clip(b + span, 0, 2 * span - 1).astype(np.int64)


def gather_index_table(delta_max: int, position_buckets: int, max_relative_positions: int) -> np.ndarray:
    """``gather_index`` for every delta in [-delta_max, delta_max] as int16 (entry i is delta = i - delta_max)."""
    d = np.arange(-delta_max, delta_max + 1, dtype=np.int64)
    return gather_index(d, position_buckets, max_relative_positions).astype(np.int16)


# --------------------------------------------------------------------------- relative tables
def layer_norm(x: np.ndarray, weight: np.ndarray, bias: np.ndarray, eps: float) -> np.ndarray:
    """LayerNorm over the last axis, biased variance (the encoder applies it to the relative
    embeddings when ``norm_rel_ebd`` contains ``layer_norm``: HF:597-601, ``model.py:224-227``)."""
    x = np.asarray(x, dtype=np.float64)
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * np.asarray(weight, np.float64) + np.asarray(bias, np.float64)


def relpos_project(rel: np.ndarray, w: np.ndarray, b: np.ndarray | None, num_heads: int) -> np.ndarray:
    """Project (already normalised) relative embeddings ``[2*span, hidden]`` with a Linear layer
    ``w [H*d, hidden]``, ``b [H*d]`` and split heads -> ``[H, 2*span, d]``.

    Follows ``model.py:92-110`` (``key_proj``/``query_proj`` when ``share_att_key`` else
    ``pos_key_proj``/``pos_query_proj``) and HF:296-311."""
    rel = np.asarray(rel, np.float64)
    y = rel @ np.asarray(w, np.float64).T
    if b is not None:
        y = y + np.asarray(b, np.float64)
    two_span = rel.shape[0]
    return np.ascontiguousarray(y.reshape(two_span, num_heads, -1).transpose(1, 0, 2))


# --------------------------------------------------------------------------- attention
def attention_single(q, k, v, kr, qr, *, position_buckets, max_relative_positions,
                     sm_scale=None, c2p=True, p2c=True, dtype=np.float64):
    """Disentangled attention for ONE sequence.

    q, k, v: ``[L, H, d]`` (q may have a different length than k is NOT supported: self-attention
    only, as in ``model.py:116-137``).  kr, qr: ``[H, 2*span, d]`` projected relative tables
    (either may be None when its term is disabled).  Returns ``[L, H, d]``.

    score[q,k] = (Q[q].K[k] + Q[q].Kr[idx(q-k)] + K[k].Qr[idx(q-k)]) * sm_scale
    with ``sm_scale = 1/sqrt(d * (1 + c2p + p2c))`` (``model.py:84-90``; HF:237-243, 324, 343),
    then softmax over k and P.V (HF:259-262).
    """
    q = np.asarray(q, dtype); k = np.asarray(k, dtype); v = np.asarray(v, dtype)
    L, H, d = q.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d * (1 + int(bool(c2p)) + int(bool(p2c))))
    out = np.empty((L, H, d), dtype)
    if L == 0:
        return out
    pos = np.arange(L, dtype=np.int64)
    idx = gather_index(pos[:, None] - pos[None, :], position_buckets, max_relative_positions)  # [Lq, Lk]
    for h in range(H):
        qh, kh, vh = q[:, h, :], k[:, h, :], v[:, h, :]
        s = qh @ kh.T
        if c2p:
            full = qh @ np.asarray(kr[h], dtype).T             # [Lq, 2span]   (model.py:122-123)
            s = s + np.take_along_axis(full, idx, axis=1)      # HF:315-324
        if p2c:
            full = kh @ np.asarray(qr[h], dtype).T             # [Lk, 2span]   (model.py:124-125)
            s = s + np.take_along_axis(full, idx.T, axis=1).T  # HF:327-343, index by key row
        s = s * dtype(sm_scale)
        s = s - s.max(axis=1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=1, keepdims=True)
        out[:, h, :] = p @ vh
    return out


def attention_single_scores(q, k, v, c2p_scores, p2c_scores, *, position_buckets, max_relative_positions,
                            sm_scale=None, p2c_mirrored=False, dtype=np.float64):
    """ONE sequence, legacy operator form: the position products arrive materialised, ``c2p_scores[t, h, r] =
    Q[t].Kr[r]`` and ``p2c_scores[t, h, r] = K[t].Qr[r]`` (``model.py:122-125``), and are only gathered.

    score[q,k] = (Q[q].K[k] + c2p_scores[q, idx(q-k)] + p2c_scores[k, idx(q-k)]) * sm_scale   (HF:315-343)
    With ``p2c_mirrored`` the last term is read at ``idx(k-q)``, the index the reference kernel forms
    (``ops/flash_attention.py:126-132``: ``-bucket(q-k) + span``; the bucket function is odd).
    q, k, v ``[L, H, d]``; scores ``[L, H, 2*span]`` or None.  Returns ``[L, H, d]``."""
    q = np.asarray(q, dtype); k = np.asarray(k, dtype); v = np.asarray(v, dtype)
    L, H, d = q.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d * (1 + int(c2p_scores is not None) + int(p2c_scores is not None)))
    out = np.empty((L, H, d), dtype)
    if L == 0:
        return out
    pos = np.arange(L, dtype=np.int64)
    idx = gather_index(pos[:, None] - pos[None, :], position_buckets, max_relative_positions)  # [a, b] -> idx(a-b)
    for h in range(H):
        s = q[:, h, :] @ k[:, h, :].T
        if c2p_scores is not None:
            s = s + np.take_along_axis(np.asarray(c2p_scores, dtype)[:, h, :], idx, axis=1)
        if p2c_scores is not None:
            full = np.asarray(p2c_scores, dtype)[:, h, :]                      # [Lk, 2span], row = key
            by_key = idx if p2c_mirrored else idx.T                            # [k, q] -> idx(k-q) or idx(q-k)
            s = s + np.take_along_axis(full, by_key, axis=1).T
        s = s * dtype(sm_scale)
        s = s - s.max(axis=1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=1, keepdims=True)
        out[:, h, :] = p @ v[:, h, :]
    return out


def attention_varlen(q, k, v, kr, qr, cu_seqlens, **kw):
    """Packed form: q, k, v ``[T, H, d]``; ``cu_seqlens`` int ``[B+1]``.  Relative positions restart
    at every sequence (``ops/flash_attention_varlen.py:70,118``).  Returns ``[T, H, d]``."""
    q = np.asarray(q); out = np.zeros(q.shape, kw.get("dtype", np.float64))
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    for b in range(len(cu) - 1):
        s, e = int(cu[b]), int(cu[b + 1])
        if e > s:
            out[s:e] = attention_single(q[s:e], k[s:e], v[s:e], kr, qr, **kw)
    return out


def attention_fixed(q, k, v, kr, qr, seqlens=None, **kw):
    """Padded form: q, k, v ``[B, L, H, d]``; ``seqlens`` int ``[B]`` valid prefix lengths (None = all L).
    Keys at or beyond the length are masked (HF:256-257).  Query rows at or beyond the length are
    returned as zeros, which is what the reference's re-padding produces (``padding.py:11-15``,
    ``model.py:183``); the eager module returns a uniform average there, and neither is meaningful."""
    q = np.asarray(q)
    B, L = q.shape[:2]
    out = np.zeros(q.shape, kw.get("dtype", np.float64))
    for b in range(B):
        n = L if seqlens is None else int(seqlens[b])
        if n > 0:
            out[b, :n] = attention_single(q[b, :n], k[b, :n], v[b, :n], kr, qr, **kw)
    return out


def self_attention_layer(hidden, seqlens, params, *, num_heads, position_buckets, max_relative_positions,
                         share_att_key=True, pos_att_type=("c2p", "p2c"), rel_embeddings=None):
    """Whole attention module (``model.py:34-186`` == HF:191-274) on padded input.

    hidden ``[B, L, hidden]``; ``params`` maps HF parameter names (``query_proj.weight`` ...) to arrays;
    ``rel_embeddings`` ``[>=2*span, hidden]`` as handed to the module (already LayerNorm'd by the encoder).
    Returns ``[B, L, hidden]`` float64 with zero rows for padded queries."""
    hidden = np.asarray(hidden, np.float64)
    B, L, hs = hidden.shape

    def lin(x, name):
        y = x @ np.asarray(params[name + ".weight"], np.float64).T
        if name + ".bias" in params and params[name + ".bias"] is not None:
            y = y + np.asarray(params[name + ".bias"], np.float64)
        return y

    q = lin(hidden, "query_proj").reshape(B, L, num_heads, -1)
    k = lin(hidden, "key_proj").reshape(B, L, num_heads, -1)
    v = lin(hidden, "value_proj").reshape(B, L, num_heads, -1)
    c2p, p2c = "c2p" in pos_att_type, "p2c" in pos_att_type
    kr = qr = None
    if rel_embeddings is not None and (c2p or p2c):
        span = att_span(position_buckets, max_relative_positions)
        rel = np.asarray(rel_embeddings, np.float64)[: 2 * span]
        if share_att_key:
            kr = relpos_project(rel, params["key_proj.weight"], params.get("key_proj.bias"), num_heads)
            qr = relpos_project(rel, params["query_proj.weight"], params.get("query_proj.bias"), num_heads)
        else:
            if c2p:
                kr = relpos_project(rel, params["pos_key_proj.weight"], params.get("pos_key_proj.bias"), num_heads)
            if p2c:
                qr = relpos_project(rel, params["pos_query_proj.weight"], params.get("pos_query_proj.bias"), num_heads)
    else:
        c2p = p2c = False
    d = q.shape[-1]
    scale = 1.0 / math.sqrt(d * (1 + int("c2p" in pos_att_type) + int("p2c" in pos_att_type)))
    out = attention_fixed(q, k, v, kr, qr, seqlens, position_buckets=position_buckets,
                          max_relative_positions=max_relative_positions, sm_scale=scale, c2p=c2p, p2c=p2c)
    return out.reshape(B, L, -1)


# --------------------------------------------------------------------------- work accounting
def algorithmic_flops(lengths, num_heads: int, head_dim: int, two_span: int) -> float:
    """Contract FLOP count: per sequence and head ``4 L^2 d`` (QK^T, PV) plus ``4 L R d``
    (the two position terms against the R = min(2*span, 2L-1) table rows a length-L sequence can reach)."""
    total = 0.0
    for L in lengths:
        L = int(L)
        R = min(two_span, max(2 * L - 1, 0))
        total += 4.0 * L * L * head_dim + 4.0 * L * R * head_dim
    return total * num_heads


def algorithmic_bytes(total_tokens: int, num_heads: int, head_dim: int, two_span: int, elem: int, n_seqs: int) -> float:
    """Contract byte count: read Q, K, V once, write O once, read both tables once, read the offsets."""
    return elem * (4.0 * total_tokens * num_heads * head_dim + 2.0 * two_span * num_heads * head_dim) + 4.0 * (n_seqs + 1)
