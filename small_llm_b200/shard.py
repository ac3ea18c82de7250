"""Batch sharding of independent sequences over the GPUs of one box.

Generation of a sequence depends only on its own tokens, the replicated weights and its own draws,
so the token loop needs no collective: rank r takes a contiguous block of sequences, runs them on its
own engine, and the only exchange is the gather of the finished token streams to rank 0 (NCCL over
NVLink on GPUs; the same code runs over gloo on CPU for the tests).  The reference has no multi-device
code of any kind; this is the path's natural extension.
"""
from __future__ import annotations

import numpy as np


def shard_range(n_seq: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous block [begin, end) of rank `rank`; blocks differ by at most one sequence."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank / world size")
    base, extra = divmod(n_seq, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def balanced_assignment(lengths, world: int) -> list[np.ndarray]:
    """Sequences dealt to ranks so that every rank gets the same count (within one) and nearly the same total
    length: sorted by length, longest first, dealt in a snake (0..world-1, world-1..0, ...).  At large batch a decode
    iteration's time follows the KV bytes a rank streams, i.e. the sum of its sequences' lengths, and the job ends
    with its slowest rank.  Returns, per rank, the global indices it owns (ascending)."""
    if world < 1:
        raise ValueError("bad world size")
    lengths = np.asarray(lengths)
    order = np.argsort(-lengths, kind="stable")
    owners: list[list[int]] = [[] for _ in range(world)]
    for k, idx in enumerate(order):
        rnd, col = divmod(k, world)
        owners[col if rnd % 2 == 0 else world - 1 - col].append(int(idx))
    return [np.array(sorted(o), dtype=np.int64) for o in owners]


def gather_streams(streams: list[np.ndarray], n_seq_total: int, max_len: int, group=None, dst: int = 0, device=None,
                   assignment: list[np.ndarray] | None = None):
    """Gathers per-rank lists of token streams to `dst` in global sequence order.

    assignment[r] = global indices of rank r's sequences, in the order of its `streams` (default: the contiguous
    blocks of shard_range).

    Every rank contributes a fixed-shape block (sequences padded to max_len, shard padded to the largest
    shard) plus the lengths, so one gather of int32 [rows, max_len + 1] suffices.  Returns the list of
    n_seq_total uint32 arrays on `dst`, None elsewhere."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    rows = -(-n_seq_total // world) if assignment is None else max(len(a) for a in assignment)
    block = np.zeros((rows, max_len + 1), dtype=np.int32)
    for i, s in enumerate(streams):
        if len(s) > max_len:
            raise ValueError("stream longer than max_len")
        block[i, 0] = len(s)
        block[i, 1:1 + len(s)] = np.asarray(s, dtype=np.uint32).astype(np.int32)
    t = torch.from_numpy(block)
    if device is not None:
        t = t.to(device)
    if world == 1:
        parts = [t]
    else:
        parts = [torch.empty_like(t) for _ in range(world)] if rank == dst else None
        dist.gather(t, parts, dst=dst, group=group)
        if rank != dst:
            return None
    out: list = [None] * n_seq_total
    for r, p in enumerate(parts):
        if assignment is None:
            b, e = shard_range(n_seq_total, world, r)
            owned = range(b, e)
        else:
            owned = assignment[r]
        a = p.cpu().numpy()
        for i, g in enumerate(owned):
            out[int(g)] = a[i, 1:1 + a[i, 0]].astype(np.uint32)
    return out
