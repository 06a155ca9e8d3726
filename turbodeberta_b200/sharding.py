"""Replica sharding for multi-GPU inference: the path has no exchange step, so ranks get disjoint sequences.

Padded batches are cut into contiguous slices; packed streams are cut at sequence boundaries with a greedy
longest-first assignment that balances attention cost (sum of L^2, tie-broken by sum of L).  The only
collective is the gather of final outputs, which callers run over NCCL (GPU) or gloo (CPU tests).
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


def shard_batch(n: int, world: int, rank: int) -> slice:
    """Contiguous slice of ``range(n)`` owned by ``rank``; sizes differ by at most one."""
    if not (0 <= rank < world):
        raise ValueError("rank outside the world")
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def shard_packed(lengths, world: int) -> list[list[int]]:
    """Sequence indices per rank: longest first, each to the rank with the least accumulated ``L^2``
    (then least tokens).  Indices inside a rank are returned in increasing order."""
    lengths = np.asarray(lengths, dtype=np.int64)
    order = np.argsort(-lengths, kind="stable")
    cost = np.zeros(world)
    toks = np.zeros(world)
    out: list[list[int]] = [[] for _ in range(world)]
    for i in order:
        r = int(np.lexsort((toks, cost))[0])
        out[r].append(int(i))
        cost[r] += float(lengths[i]) ** 2
        toks[r] += float(lengths[i])
    return [sorted(x) for x in out]


def gather_padded(local: torch.Tensor, n_total: int, group=None) -> torch.Tensor:
    """All ranks contribute their contiguous batch slice ``[n_r, ...]`` (``shard_batch`` order); every rank gets
    ``[n_total, ...]``.  Uneven slices are padded to the largest one for the collective and trimmed after."""
    world = dist.get_world_size(group)
    sizes = [shard_batch(n_total, world, r) for r in range(world)]
    biggest = max(s.stop - s.start for s in sizes)
    buf = local
    if local.shape[0] != biggest:
        buf = torch.zeros(biggest, *local.shape[1:], dtype=local.dtype, device=local.device)
        buf[: local.shape[0]] = local
    out = torch.empty(world * biggest, *local.shape[1:], dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, buf.contiguous(), group=group)
    if world * biggest == n_total:                 # even slices: the collective's output already is the result
        return out
    parts = [out[r * biggest: r * biggest + (s.stop - s.start)] for r, s in enumerate(sizes)]
    return torch.cat(parts, 0)


def gather_packed(local: torch.Tensor, lengths, assignment: list[list[int]], group=None) -> torch.Tensor:
    """Inverse of ``shard_packed``: ``local`` holds this rank's sequences back to back (in the order of
    ``assignment[rank]``); returns the full packed stream ``[sum(lengths), ...]`` in original sequence order."""
    world = dist.get_world_size(group)
    lengths = np.asarray(lengths, dtype=np.int64)
    tok = [int(lengths[a].sum()) if len(a) else 0 for a in assignment]
    biggest = max(max(tok), 1)
    buf = torch.zeros(biggest, *local.shape[1:], dtype=local.dtype, device=local.device)
    buf[: local.shape[0]] = local
    out = torch.empty(world * biggest, *local.shape[1:], dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, buf, group=group)
    cu = np.concatenate([[0], np.cumsum(lengths)])
    full = torch.empty(int(cu[-1]), *local.shape[1:], dtype=local.dtype, device=local.device)
    for r, seqs in enumerate(assignment):
        off = r * biggest
        for s in seqs:
            n = int(lengths[s])
            full[int(cu[s]): int(cu[s]) + n] = out[off: off + n]
            off += n
    return full
