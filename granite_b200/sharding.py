"""Sharding of attention work across the GPUs of one box.

Every (sequence, KV head) pair is independent - softmax is per query head and a GQA group reads
exactly one KV head - so attention needs no exchange step.  Sequences are dealt to ranks by
longest-processing-time-first on their context length (the cost of decode is the bytes of K/V
read); each rank's page manager owns only its sequences' pages.  The only collective is the gather
of per-rank output rows, after which `unshard` restores the caller's sequence order.

When the KV-head count is a multiple of the rank count there is a second split: every rank holds
ALL sequences but only `Hkv / ranks` KV heads (pool shard [pages * 16, Hkv / ranks, D]) and the
query heads of their GQA groups.  Block tables are replicated - they index tokens, not heads - and
the split is perfectly balanced whatever the lengths are; the gather then interleaves head slices
([B, Hq / ranks, D] per rank -> [B, Hq, D]).  `choose_split` picks per call whichever of the two the
plan predicts to finish first.
"""
from __future__ import annotations

import numpy as np


def lpt_assign(lengths, n_ranks: int) -> list[np.ndarray]:
    """Indices of the sequences each rank owns.  Deterministic: ties broken by index, so every
    rank computes the same plan from the same lengths without talking to the others."""
    lengths = np.asarray(lengths, np.int64)
    order = np.lexsort((np.arange(len(lengths)), -lengths))  # by length desc, then index
    load = np.zeros(n_ranks, np.int64)
    owned: list[list[int]] = [[] for _ in range(n_ranks)]
    for i in order:
        r = int(np.argmin(load))  # first minimum: lowest rank wins ties
        owned[r].append(int(i))
        load[r] += int(lengths[i])
    return [np.array(sorted(o), np.int64) for o in owned]


def imbalance(lengths, plan) -> float:
    """max rank load / mean rank load."""
    lengths = np.asarray(lengths, np.int64)
    loads = np.array([int(lengths[p].sum()) for p in plan], np.float64)
    return float(loads.max() / max(loads.mean(), 1.0))


def padded_rows(plan) -> int:
    """Rows every rank contributes to an all-gather (ranks own different numbers of sequences)."""
    return max((len(p) for p in plan), default=0)


def unshard(gathered: np.ndarray, plan, n_sequences: int) -> np.ndarray:
    """gathered: [n_ranks, padded_rows, ...] as all-gather returns it -> [n_sequences, ...] in the
    caller's order."""
    out = np.zeros((n_sequences,) + tuple(gathered.shape[2:]), gathered.dtype)
    for r, idx in enumerate(plan):
        out[idx] = gathered[r, : len(idx)]
    return out


# ---------------------------------------------------------------------------- split by KV head
def head_split(num_heads: int, num_kv_heads: int, n_ranks: int):
    """Per rank (first KV head, KV heads, first query head, query heads), or None when the KV heads
    do not divide evenly among the ranks."""
    if n_ranks < 1 or num_kv_heads % n_ranks != 0 or num_heads % num_kv_heads != 0:
        return None
    hkv = num_kv_heads // n_ranks
    group = num_heads // num_kv_heads
    return [(r * hkv, hkv, r * hkv * group, hkv * group) for r in range(n_ranks)]


def shard_pool_by_head(pool, rank: int, n_ranks: int):
    """pool [rows, Hkv, D] (numpy or torch) -> this rank's contiguous [rows, Hkv / ranks, D] shard.
    Row numbers are unchanged, so every rank uses the same block tables."""
    hkv = pool.shape[1] // n_ranks
    part = pool[:, rank * hkv:(rank + 1) * hkv]
    return part.contiguous() if hasattr(part, "contiguous") else np.ascontiguousarray(part)


def shard_queries_by_head(q, rank: int, n_ranks: int):
    """q [B, Hq, D] -> the query heads of this rank's KV heads, [B, Hq / ranks, D]."""
    hq = q.shape[1] // n_ranks
    part = q[:, rank * hq:(rank + 1) * hq]
    return part.contiguous() if hasattr(part, "contiguous") else np.ascontiguousarray(part)


def unshard_heads(gathered: np.ndarray) -> np.ndarray:
    """gathered [n_ranks, B, Hq / ranks, D] as an all-gather of head slices returns it -> [B, Hq, D]."""
    n, b, hq, d = gathered.shape
    return np.ascontiguousarray(gathered.transpose(1, 0, 2, 3)).reshape(b, n * hq, d)


# Throughput of the decode kernel with this many KV heads per page box, relative to eight (32 KB
# boxes).  With fewer heads the warps of a head share its pages instead of its query heads, which keeps
# the kernel near its rate down to two heads; one-head pages are 4 KB boxes, bound by how fast they can be
# issued.  Measured on B200 on the long-context lengths, 4.8 GB of K/V per call: 6.89, 6.67, 6.27 and 5.04 TB/s.
HEADS_PER_BOX_EFFICIENCY = {8: 1.0, 4: 0.97, 2: 0.91, 1: 0.73}


def predicted_cost(lengths, num_kv_heads: int, n_ranks: int, split: str) -> float:
    """Tokens x KV heads the slowest rank reads, divided by the kernel's relative throughput."""
    lengths = np.asarray(lengths, np.int64)
    if split == "sequence":
        plan = lpt_assign(lengths, n_ranks)
        worst = max((int(lengths[p].sum()) for p in plan), default=0)
        return worst * num_kv_heads / HEADS_PER_BOX_EFFICIENCY.get(min(num_kv_heads, 8), 1.0)
    if split == "kv_head":
        if num_kv_heads % n_ranks != 0:
            return float("inf")
        local = num_kv_heads // n_ranks
        return int(lengths.sum()) * local / HEADS_PER_BOX_EFFICIENCY.get(min(local, 8), 1.0)
    raise ValueError(split)


def choose_split(lengths, num_kv_heads: int, n_ranks: int) -> str:
    """"kv_head" when the heads divide evenly and that split is predicted faster, else "sequence"."""
    if n_ranks <= 1:
        return "sequence"
    by_seq = predicted_cost(lengths, num_kv_heads, n_ranks, "sequence")
    by_head = predicted_cost(lengths, num_kv_heads, n_ranks, "kv_head")
    return "kv_head" if by_head < by_seq else "sequence"
