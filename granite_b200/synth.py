"""Seeded synthetic workloads with the shapes of the benchmark configurations.

Granite measures this path only on synthetic tensors (tools/benchmark_attention.mm:153-176) and
on model files it does not ship, so every input here is synthetic: lengths, page permutation
and tree shapes come from numpy's PCG64 seeded per case; K/V/Q are i.i.d. N(0,1), generated
either on the host (small parity cases, bit-identical inputs for the CPU checker) or directly in
HBM with a seeded torch generator (full-size cases).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

PAGE = 16


@dataclass
class PagedCase:
    """A batch of sequences in a paged fp16 pool.  Arrays are numpy unless `device` was given,
    in which case q/k_pool/v_pool are torch tensors on that device."""
    seq_lens: np.ndarray      # [B] int32
    tables: np.ndarray        # [B, max_blocks] int32, -1 padded
    num_blocks: int
    q: object                 # [B, Hq, D] fp32
    k_pool: object            # [num_blocks*PAGE, Hkv, D] fp16
    v_pool: object
    num_heads: int
    num_kv_heads: int
    head_dim: int

    @property
    def batch(self) -> int:
        return int(self.seq_lens.shape[0])

    @property
    def max_blocks(self) -> int:
        return int(self.tables.shape[1])

    @property
    def total_tokens(self) -> int:
        return int(self.seq_lens.sum())

    def algorithmic_bytes(self) -> int:
        """K+V once per element, the table entries and lengths read, Q read, O written."""
        hkv, d, hq = self.num_kv_heads, self.head_dim, self.num_heads
        pages = int(((self.seq_lens + PAGE - 1) // PAGE).sum())
        return (self.total_tokens * hkv * d * 2 * 2 + pages * 4 + self.batch * 4
                + self.batch * hq * d * 4 * 2)


def draw_lengths(rng: np.random.Generator, batch: int, lo: int, hi: int, dist: str) -> np.ndarray:
    if dist == "uniform":
        return rng.integers(lo, hi + 1, size=batch).astype(np.int32)
    if dist == "loguniform":
        return np.rint(np.exp(rng.uniform(np.log(lo), np.log(hi), size=batch))).astype(np.int32)
    raise ValueError(dist)


def build_tables(rng: np.random.Generator, seq_lens: np.ndarray, spare_blocks: int = 0):
    """One seeded permutation of [0, num_blocks) dealt to the sequences in order."""
    pages = (seq_lens.astype(np.int64) + PAGE - 1) // PAGE
    num_blocks = int(pages.sum()) + spare_blocks
    perm = rng.permutation(num_blocks).astype(np.int32)
    max_blocks = max(int(pages.max()) if len(pages) else 1, 1)
    tables = np.full((len(seq_lens), max_blocks), -1, np.int32)
    off = 0
    for b, n in enumerate(pages):
        tables[b, :n] = perm[off:off + n]
        off += int(n)
    return tables, max(num_blocks, 1)


def paged_case(seed: int, batch: int, len_lo: int, len_hi: int, num_heads: int = 32,
               num_kv_heads: int = 8, head_dim: int = 128, dist: str = "uniform",
               device=None, seq_lens=None, spare_blocks: int = 0) -> PagedCase:
    rng = np.random.default_rng(seed)
    if seq_lens is None:
        seq_lens = draw_lengths(rng, batch, len_lo, len_hi, dist)
    seq_lens = np.asarray(seq_lens, np.int32)
    tables, num_blocks = build_tables(np.random.default_rng(seed + 100), seq_lens, spare_blocks)
    rows = num_blocks * PAGE
    if device is None:
        q = np.random.default_rng(seed + 200).standard_normal((len(seq_lens), num_heads, head_dim), np.float32)
        k = np.random.default_rng(seed + 300).standard_normal((rows, num_kv_heads, head_dim), np.float32).astype(np.float16)
        v = np.random.default_rng(seed + 400).standard_normal((rows, num_kv_heads, head_dim), np.float32).astype(np.float16)
    else:
        import torch
        g = torch.Generator(device=device)
        g.manual_seed(seed + 200)
        q = torch.randn((len(seq_lens), num_heads, head_dim), dtype=torch.float32, device=device, generator=g)
        k = torch.empty((rows, num_kv_heads, head_dim), dtype=torch.float16, device=device)
        v = torch.empty_like(k)
        g.manual_seed(seed + 300)
        k.normal_(generator=g)
        g.manual_seed(seed + 400)
        v.normal_(generator=g)
    return PagedCase(seq_lens, tables, num_blocks, q, k, v, num_heads, num_kv_heads, head_dim)


def tree_parents(seed: int, num_nodes: int = 64, max_children: int = 4, max_depth: int = 8) -> np.ndarray:
    """Random draft tree: parent[0] = -1; node i > 0 picks a parent uniformly among earlier nodes
    that still have fewer than `max_children` children and depth < max_depth (root depth 0), so a
    parent always precedes its children, as SpeculationTree::add_node builds them."""
    rng = np.random.default_rng(seed)
    parents = np.full(num_nodes, -1, np.int32)
    depth = np.zeros(num_nodes, np.int32)
    kids = np.zeros(num_nodes, np.int32)
    for i in range(1, num_nodes):
        cand = [j for j in range(i) if kids[j] < max_children and depth[j] < max_depth]
        p = int(cand[rng.integers(0, len(cand))])
        parents[i] = p
        depth[i] = depth[p] + 1
        kids[p] += 1
    return parents


# Shapes of the benchmark configurations.
CONFIGS = {
    "decode_contiguous_ctx512": dict(seed=1001, batch=1, ctx=512, num_heads=32, num_kv_heads=8, head_dim=128),
    "prefill_causal_s2048": dict(seed=1002, seq=2048, num_heads=32, num_kv_heads=8, head_dim=128),
    "paged_decode_b64": dict(seed=1003, batch=64, len_lo=1024, len_hi=32768, dist="uniform",
                             num_heads=32, num_kv_heads=8, head_dim=128),
    "tree_verify_b16": dict(seed=1004, batch=16, prefix=4096, nodes=64, max_children=4, max_depth=8,
                            num_heads=32, num_kv_heads=8, head_dim=128),
    "paged_decode_long_b256": dict(seed=1005, batch=256, len_lo=4096, len_hi=131072, dist="loguniform",
                                   num_heads=64, num_kv_heads=8, head_dim=128),
}
