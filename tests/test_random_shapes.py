"""Seeded random shapes for the three attention entry points: head counts and group sizes that are
not powers of two, ragged lengths around every tile and page boundary, offsets, stale cache rows
poisoned with NaN - each case against the CPU checker."""
import numpy as np
import pytest

from conftest import assert_attention_close
from granite_b200 import synth
import test_prefill as TP
import test_tree_verify as TT

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_random_prefill_shapes(compute):
    rng = np.random.default_rng(101)
    for _ in range(16):
        hkv = int(rng.choice([1, 2, 3, 4, 8]))
        hq = hkv * int(rng.choice([1, 2, 3, 4, 5, 8]))
        seq_q = int(rng.integers(2, 520))
        start = int(rng.choice([0, 0, int(rng.integers(0, 700))]))
        seq_kv = start + seq_q
        max_seq = seq_kv + int(rng.choice([0, 0, 1, 77, 200]))
        q_fp16, out_fp16 = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        q, k, v = TP._case(int(rng.integers(1 << 30)), seq_q, seq_kv, max_seq, hq, hkv)
        got = TP._run(compute, q, k, v, seq_kv, start, q_fp16, out_fp16)
        ref = TP._oracle(q, k, v, seq_kv, start, q_fp16)
        assert_attention_close(got, ref, f"prefill Hq={hq} Hkv={hkv} seq_q={seq_q} start={start} max_seq={max_seq} "
                                         f"q16={q_fp16} out16={out_fp16}")


def test_random_tree_shapes(compute):
    import torch
    from oracle import pyoracle
    rng = np.random.default_rng(202)
    for _ in range(12):
        hkv = int(rng.choice([1, 2, 4, 8]))
        hq = hkv * int(rng.choice([1, 2, 3, 4, 6, 8]))
        batch, n = int(rng.integers(1, 5)), int(rng.integers(1, 65))
        lens = np.array(rng.choice([0, 1, 15, 16, 17, 100, 127, 128, 129, 300, 1000], size=batch), np.int32)
        q_fp16 = bool(rng.integers(0, 2))
        case = synth.paged_case(int(rng.integers(1 << 30)), batch, 0, 0, hq, hkv, seq_lens=lens, spare_blocks=2)
        q, kt, vt, _ = TT._tree_inputs(int(rng.integers(1 << 30)), batch, n, hq, hkv)
        parents = np.stack([synth.tree_parents(int(rng.integers(1 << 30)), n) for _ in range(batch)])
        if q_fp16:
            q = q.astype(np.float16).astype(np.float32)
        k_np, v_np = case.k_pool.view(np.uint16).copy(), case.v_pool.view(np.uint16).copy()
        live = np.zeros(case.num_blocks * synth.PAGE, bool)
        for b, length in enumerate(lens):
            for pos in range(int(length)):
                live[case.tables[b, pos // synth.PAGE] * synth.PAGE + pos % synth.PAGE] = True
        k_np[~live] = 0x7E00
        v_np[~live] = 0x7E00
        tables = np.where(case.tables < 0, 0, case.tables).astype(np.int32)
        out = torch.full((batch, hq, n, 128), float("nan"), device=DEV)
        compute.attention_tree(torch.from_numpy(q.astype(np.float16) if q_fp16 else q).to(DEV),
                               torch.from_numpy(k_np.view(np.float16)).to(DEV), torch.from_numpy(v_np.view(np.float16)).to(DEV),
                               torch.from_numpy(kt).to(DEV), torch.from_numpy(vt).to(DEV), torch.from_numpy(parents).to(DEV),
                               out, hq, hkv, n, 0, 128, 1.0 / np.sqrt(128.0), batch_size=batch,
                               block_tables=torch.from_numpy(tables).to(DEV), max_blocks_per_seq=case.max_blocks,
                               num_blocks=case.num_blocks, cache_lens=torch.from_numpy(lens).to(DEV), q_dtype=int(q_fp16))
        compute.sync()
        got = out.cpu().numpy()
        for b in range(batch):
            kr, _ = pyoracle.paged_gather(k_np, tables[b], int(lens[b]), synth.PAGE)
            vr, _ = pyoracle.paged_gather(v_np, tables[b], int(lens[b]), synth.PAGE)
            ref = TT._oracle_one(q[b], pyoracle.f16_bits_to_f32(kr), pyoracle.f16_bits_to_f32(vr), kt[b], vt[b], parents[b])
            assert_attention_close(got[b], ref, f"tree Hq={hq} Hkv={hkv} N={n} prefix={int(lens[b])} q16={q_fp16}")


def test_random_decode_shapes(compute):
    import torch
    from oracle import pyoracle
    rng = np.random.default_rng(303)
    for _ in range(12):
        hkv = int(rng.choice([1, 2, 4, 8, 16]))
        hq = hkv * int(rng.choice([1, 2, 3, 4, 8, 16]))
        if hq > 64:
            hq = hkv * 2
        batch = int(rng.integers(1, 40))
        lens = np.array(rng.choice([0, 1, 2, 15, 16, 17, 31, 32, 33, 100, 500, 1000, 2047, 2048], size=batch), np.int32)
        case = synth.paged_case(int(rng.integers(1 << 30)), batch, 0, 0, hq, hkv, seq_lens=lens, spare_blocks=1)
        out = torch.full((batch, hq, 128), float("nan"), device=DEV)
        compute.batched_paged_attention_decode(torch.from_numpy(case.q).to(DEV), torch.from_numpy(case.k_pool).to(DEV),
                                               torch.from_numpy(case.v_pool).to(DEV), torch.from_numpy(case.tables).to(DEV),
                                               torch.from_numpy(lens).to(DEV), out, batch, hq, hkv, 128, synth.PAGE,
                                               case.max_blocks, 1.0 / np.sqrt(128.0), num_blocks=case.num_blocks)
        compute.sync()
        ref, bad = pyoracle.paged_decode_batch(case.q, case.k_pool.view(np.uint16), case.v_pool.view(np.uint16),
                                               np.where(case.tables < 0, 0, case.tables), lens, synth.PAGE)
        assert bad == 0
        assert_attention_close(out.cpu().numpy(), ref, f"decode Hq={hq} Hkv={hkv} lens={lens.tolist()}")
