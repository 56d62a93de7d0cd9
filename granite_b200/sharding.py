"""Sharding of attention work across the GPUs of one box.

Every (sequence, KV head) pair is independent - softmax is per query head and a GQA group reads
exactly one KV head - so attention needs no exchange step.  Sequences are dealt to ranks by
longest-processing-time-first on their context length (the cost of decode is the bytes of K/V
read); each rank's page manager owns only its sequences' pages.  The only collective is the gather
of per-rank output rows, after which `unshard` restores the caller's sequence order.
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
