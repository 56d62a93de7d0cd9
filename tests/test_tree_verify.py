"""Tree-masked verification attention (tcgen05/TMEM kernel) against the CPU checker.

Reference: MetalCompute::attention_tree (include/granite/metal_compute.h:830-844); correctness is
the CPU loop src/llm/transformer.mm:2044-2126 with the ancestor mask of :823-840.  The mask is
checked bit for bit, the outputs within the path's tolerance.
"""
import numpy as np
import pytest

from conftest import assert_attention_close
from granite_b200 import synth

pytestmark = pytest.mark.gpu
D = 128


def _tree_inputs(seed, batch, n, hq, hkv, same_tree=False):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((batch, hq, n, D), np.float32)
    kt = rng.standard_normal((batch, hkv, n, D), np.float32).astype(np.float16)
    vt = rng.standard_normal((batch, hkv, n, D), np.float32).astype(np.float16)
    parents = np.stack([synth.tree_parents(seed + (0 if same_tree else b), n) for b in range(batch)])
    return q, kt, vt, parents


def _oracle_one(q_b, kp, vp, kt_b, vt_b, parents_b):
    """q_b [Hq,N,D] fp32; kp/vp [L,Hkv,D] fp32; kt_b/vt_b [Hkv,N,D] fp16 -> [Hq,N,D]."""
    from oracle import pyoracle
    q4 = np.ascontiguousarray(q_b.transpose(1, 0, 2))[None]                  # [1,N,Hq,D]
    kt = np.ascontiguousarray(kt_b.astype(np.float32).transpose(1, 0, 2))[None]  # [1,N,Hkv,D]
    vt = np.ascontiguousarray(vt_b.astype(np.float32).transpose(1, 0, 2))[None]
    out = pyoracle.attention_tree(q4, kp, vp, kt, vt, parents_b)
    return out[0].transpose(1, 0, 2)


@pytest.mark.parametrize("n,cache_len,hq,hkv,q_fp16", [
    (64, 512, 32, 8, False), (64, 512, 32, 8, True), (16, 300, 8, 2, False), (1, 40, 4, 1, False),
    (33, 0, 8, 2, False), (64, 128, 4, 4, True), (7, 1000, 16, 2, False), (64, 129, 6, 2, True)])
def test_contiguous_prefix_reference_layout(compute, n, cache_len, hq, hkv, q_fp16):
    """batch 1, cache [Hkv, cache_len, D] with stride cache_len: the reference's own call."""
    import torch
    from oracle import pyoracle
    q, kt, vt, parents = _tree_inputs(50 + n + cache_len, 1, n, hq, hkv)
    if q_fp16:
        q = q.astype(np.float16).astype(np.float32)
    rng = np.random.default_rng(3)
    kc = rng.standard_normal((hkv, max(cache_len, 1), D), np.float32).astype(np.float16)
    vc = rng.standard_normal((hkv, max(cache_len, 1), D), np.float32).astype(np.float16)
    dev = "cuda:0"
    out = torch.full((hq, n, D), float("nan"), device=dev)
    qd = torch.from_numpy(q[0].astype(np.float16) if q_fp16 else q[0]).to(dev)
    compute.attention_tree(qd, torch.from_numpy(kc).to(dev), torch.from_numpy(vc).to(dev),
                           torch.from_numpy(kt[0]).to(dev), torch.from_numpy(vt[0]).to(dev),
                           torch.from_numpy(parents[0]).to(dev), out, hq, hkv, n, cache_len, D,
                           1.0 / np.sqrt(D), q_dtype=int(q_fp16))
    compute.sync()
    kp = pyoracle.cache_to_fp32(kc.view(np.uint16), cache_len) if cache_len else np.zeros((0, hkv, D), np.float32)
    vp = pyoracle.cache_to_fp32(vc.view(np.uint16), cache_len) if cache_len else np.zeros((0, hkv, D), np.float32)
    ref = _oracle_one(q[0], kp, vp, kt[0], vt[0], parents[0])
    assert_attention_close(out.cpu().numpy(), ref, f"tree n={n} cache={cache_len}")


@pytest.mark.parametrize("batch,n,lens,hq,hkv", [(3, 64, [700, 16, 2049], 32, 8), (2, 20, [0, 333], 8, 2),
                                                 (4, 64, [512] * 4, 16, 2)])
def test_paged_prefix_batch(compute, batch, n, lens, hq, hkv):
    """Prefix in the paged pool (block table), one tree per sequence, stale NaN rows in the pool."""
    import torch
    from oracle import pyoracle
    q, kt, vt, parents = _tree_inputs(90 + n, batch, n, hq, hkv)
    case = synth.paged_case(seed=77, batch=batch, len_lo=0, len_hi=0, num_heads=hq, num_kv_heads=hkv,
                            seq_lens=np.array(lens, np.int32), spare_blocks=2)
    k_np = case.k_pool.view(np.uint16).copy()
    v_np = case.v_pool.view(np.uint16).copy()
    live = np.zeros(case.num_blocks * synth.PAGE, bool)
    for b, L in enumerate(lens):
        for pos in range(L):
            live[case.tables[b, pos // 16] * 16 + pos % 16] = True
    k_np[~live] = 0x7E00
    v_np[~live] = 0x7E00
    dev = "cuda:0"
    out = torch.full((batch, hq, n, D), float("nan"), device=dev)
    compute.attention_tree(torch.from_numpy(q).to(dev), torch.from_numpy(k_np.view(np.float16)).to(dev),
                           torch.from_numpy(v_np.view(np.float16)).to(dev), torch.from_numpy(kt).to(dev),
                           torch.from_numpy(vt).to(dev), torch.from_numpy(parents).to(dev), out, hq, hkv, n, 0, D,
                           1.0 / np.sqrt(D), batch_size=batch, block_tables=torch.from_numpy(case.tables).to(dev),
                           cache_lens=torch.from_numpy(case.seq_lens).to(dev), max_blocks_per_seq=case.max_blocks,
                           num_blocks=case.num_blocks)
    compute.sync()
    got = out.cpu().numpy()
    tables = np.where(case.tables < 0, 0, case.tables)
    for b, L in enumerate(lens):
        kr, bad = pyoracle.paged_gather(k_np, tables[b], L, 16)
        vr, _ = pyoracle.paged_gather(v_np, tables[b], L, 16)
        assert bad == 0
        ref = _oracle_one(q[b], pyoracle.f16_bits_to_f32(kr), pyoracle.f16_bits_to_f32(vr), kt[b], vt[b], parents[b])
        assert_attention_close(got[b], ref, f"paged tree seq {b} len {L}")


def test_tree_mask_is_bit_exact(compute):
    import torch
    from oracle import pyoracle
    dev = "cuda:0"
    for n in (1, 2, 17, 64):
        parents = np.stack([synth.tree_parents(1004 + b, n) for b in range(5)])
        parents[4] = -1                       # a forest of roots
        if n > 2:
            parents[3] = np.arange(-1, n - 1)  # a chain: node i sees 0..i
        masks = torch.zeros((5, n), dtype=torch.int64, device=dev)
        compute.build_tree_mask(torch.from_numpy(parents).to(dev), masks, 5, n)
        compute.sync()
        got = masks.cpu().numpy().view(np.uint64)
        for b in range(5):
            ref = pyoracle.tree_mask(parents[b])
            bits = ((got[b][:, None] >> np.arange(n, dtype=np.uint64)[None, :]) & np.uint64(1)).astype(np.uint8)
            assert np.array_equal(bits, ref)


def test_parent_out_of_range_is_reported(compute):
    import torch
    import granite_b200 as g
    parents = np.array([[-1, 0, 9]], np.int32)  # 9 >= num_nodes (src/llm/transformer.mm:806-813)
    masks = torch.zeros((1, 3), dtype=torch.int64, device="cuda:0")
    compute.build_tree_mask(torch.from_numpy(parents).to("cuda:0"), masks, 1, 3)
    with pytest.raises(g.GraniteCudaError) as ei:
        compute.sync()
    assert ei.value.code == g.ErrorCode.InvalidArgument
    compute.sync()


def test_full_tree_config_sample(compute):
    """The benchmark configuration: 16 sequences x (4096-token paged prefix + 64-node tree), Hq 32,
    Hkv 8; K/V generated in HBM; the CPU checker evaluates sequences 0 and 15."""
    import torch
    from oracle import pyoracle
    cfg = synth.CONFIGS["tree_verify_b16"]
    batch, n, hq, hkv, L = cfg["batch"], cfg["nodes"], cfg["num_heads"], cfg["num_kv_heads"], cfg["prefix"]
    dev = "cuda:0"
    case = synth.paged_case(cfg["seed"], batch, 0, 0, hq, hkv, seq_lens=np.full(batch, L, np.int32), device=dev)
    q, kt, vt, parents = _tree_inputs(cfg["seed"] + 500, batch, n, hq, hkv)
    q = q.astype(np.float16).astype(np.float32)  # fp16-representable queries
    out = torch.zeros((batch, hq, n, D), device=dev)
    tables = torch.from_numpy(case.tables).to(dev)
    compute.attention_tree(torch.from_numpy(q.astype(np.float16)).to(dev), case.k_pool, case.v_pool,
                           torch.from_numpy(kt).to(dev), torch.from_numpy(vt).to(dev),
                           torch.from_numpy(parents).to(dev), out, hq, hkv, n, L, D, 1.0 / np.sqrt(D),
                           batch_size=batch, block_tables=tables, max_blocks_per_seq=case.max_blocks,
                           num_blocks=case.num_blocks, q_dtype=1)
    compute.sync()
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    for b in (0, batch - 1):
        rows = (torch.from_numpy(case.tables[b]).to(dev).long()[:, None] * 16 + torch.arange(16, device=dev)[None]).reshape(-1)[:L]
        kr = case.k_pool[rows].cpu().numpy().astype(np.float32)
        vr = case.v_pool[rows].cpu().numpy().astype(np.float32)
        ref = _oracle_one(q[b], kr, vr, kt[b], vt[b], parents[b])
        assert_attention_close(got[b], ref, f"tree config, sequence {b}")


@pytest.mark.parametrize("lens,hq,hkv,n,q_fp16", [
    ([4096] * 4, 32, 8, 64, True),                 # few equal items
    ([9000, 16, 0, 1300, 2049, 40], 16, 4, 64, True),   # ragged: one long prefix among short and empty ones
    ([5000, 1200], 8, 2, 33, False),               # fp32 queries (hi + lo tiles)
    ([1100] * 30, 8, 8, 16, True),                 # many items of nine steps, four heads per tile
    ([20000], 4, 1, 64, True),                     # one long sequence, one KV head
])
def test_long_and_ragged_prefixes(compute, lens, hq, hkv, n, q_fp16):
    """Few work items with long, ragged or empty paged prefixes; every sequence against the CPU checker, and a
    second call on the same compute object must pass as well."""
    import torch
    from oracle import pyoracle
    batch = len(lens)
    q, kt, vt, parents = _tree_inputs(300 + n + batch, batch, n, hq, hkv)
    if q_fp16:
        q = q.astype(np.float16).astype(np.float32)
    case = synth.paged_case(seed=78, batch=batch, len_lo=0, len_hi=0, num_heads=hq, num_kv_heads=hkv,
                            seq_lens=np.array(lens, np.int32), spare_blocks=2)
    dev = "cuda:0"
    k_np, v_np = case.k_pool.view(np.uint16), case.v_pool.view(np.uint16)
    args = (torch.from_numpy(q.astype(np.float16) if q_fp16 else q).to(dev), torch.from_numpy(case.k_pool).to(dev),
            torch.from_numpy(case.v_pool).to(dev), torch.from_numpy(kt).to(dev), torch.from_numpy(vt).to(dev),
            torch.from_numpy(parents).to(dev))
    tables_d = torch.from_numpy(case.tables).to(dev)
    lens_d = torch.from_numpy(case.seq_lens).to(dev)
    outs = []
    for _ in range(2):
        out = torch.full((batch, hq, n, D), float("nan"), device=dev)
        compute.attention_tree(*args, out, hq, hkv, n, 0, D, 1.0 / np.sqrt(D), batch_size=batch, block_tables=tables_d,
                               cache_lens=lens_d, max_blocks_per_seq=case.max_blocks, num_blocks=case.num_blocks,
                               q_dtype=int(q_fp16))
        compute.sync()
        outs.append(out.cpu().numpy())
    tables = np.where(case.tables < 0, 0, case.tables)
    for b, L in enumerate(lens):
        kr, bad = pyoracle.paged_gather(k_np, tables[b], L, 16)
        vr, _ = pyoracle.paged_gather(v_np, tables[b], L, 16)
        assert bad == 0
        ref = _oracle_one(q[b], pyoracle.f16_bits_to_f32(kr), pyoracle.f16_bits_to_f32(vr), kt[b], vt[b], parents[b])
        assert_attention_close(outs[0][b], ref, f"sequence {b} of lens {lens}")
        assert_attention_close(outs[1][b], ref, f"second call, sequence {b} of lens {lens}")
