"""Paged / contiguous decode attention on the GPU against the CPU checker (through the C ABI).

Shapes follow tools/test_paged_flash_attention.mm:158-174 (Hq 32, Hkv 8|4, D 128, block 16,
shuffled block table) plus the edge cases the reference kernels special-case: one token, a
length that is not a multiple of the block, an empty sequence, ragged batches.
"""
import numpy as np
import pytest

from conftest import assert_attention_close
from granite_b200 import synth

pytestmark = pytest.mark.gpu


def _run_paged(compute, case, poison_unused=False):
    import torch
    dev = "cuda:0"
    k_np = case.k_pool.view(np.uint16).copy()
    v_np = case.v_pool.view(np.uint16).copy()
    if poison_unused:
        # every row that no live token maps to becomes NaN: the kernel must never let it leak
        live = np.zeros(case.num_blocks * synth.PAGE, bool)
        for b, n in enumerate(case.seq_lens):
            for pos in range(int(n)):
                live[case.tables[b, pos // synth.PAGE] * synth.PAGE + pos % synth.PAGE] = True
        k_np[~live] = 0x7E00
        v_np[~live] = 0x7E00
    q = torch.from_numpy(case.q).to(dev)
    k = torch.from_numpy(k_np.view(np.float16)).to(dev)
    v = torch.from_numpy(v_np.view(np.float16)).to(dev)
    tables = torch.from_numpy(case.tables).to(dev)
    lens = torch.from_numpy(case.seq_lens).to(dev)
    out = torch.full((case.batch, case.num_heads, case.head_dim), float("nan"), device=dev)
    scale = 1.0 / np.sqrt(case.head_dim)
    compute.batched_paged_attention_decode(q, k, v, tables, lens, out, case.batch, case.num_heads,
                                           case.num_kv_heads, case.head_dim, synth.PAGE,
                                           case.max_blocks, scale, num_blocks=case.num_blocks)
    compute.sync()
    return out.cpu().numpy(), k_np, v_np


def _oracle(case, k_np, v_np):
    from oracle import pyoracle
    tables = np.where(case.tables < 0, 0, case.tables)
    ref, bad = pyoracle.paged_decode_batch(case.q, k_np, v_np, tables, case.seq_lens, synth.PAGE)
    assert bad == 0
    return ref


@pytest.mark.parametrize("hq,hkv", [(32, 8), (32, 4), (64, 8), (8, 8), (16, 2), (8, 1), (32, 16),
                                    # few KV heads: the warps of a head share its pages (groups up to 16) ...
                                    (16, 1), (9, 1), (1, 1), (4, 4), (64, 4),
                                    # ... or, with larger groups, its query heads
                                    (64, 2), (40, 1),
                                    # head counts that are not 1, 2, 4 or 8k: tiles of the largest of 4, 2, 1 that divides
                                    (12, 3), (24, 12), (14, 7), (6, 6), (40, 10)])
def test_paged_decode_matches_cpu(compute, hq, hkv):
    case = synth.paged_case(seed=7 + hq + hkv, batch=5, len_lo=1, len_hi=700, num_heads=hq, num_kv_heads=hkv)
    got, k_np, v_np = _run_paged(compute, case)
    assert_attention_close(got, _oracle(case, k_np, v_np), f"Hq={hq} Hkv={hkv}")


@pytest.mark.parametrize("lens", [[1], [15], [16], [17], [512], [4097], [1, 16, 33, 2048, 5], [0, 40, 0], [3000] * 3])
def test_paged_decode_edge_lengths(compute, lens):
    case = synth.paged_case(seed=11, batch=len(lens), len_lo=0, len_hi=0, seq_lens=np.array(lens, np.int32),
                            spare_blocks=3)
    got, k_np, v_np = _run_paged(compute, case, poison_unused=True)
    ref = _oracle(case, k_np, v_np)
    assert_attention_close(got, ref, f"lens={lens}")
    for b, n in enumerate(lens):
        if n == 0:
            assert not got[b].any()


def test_paged_decode_many_short_sequences(compute):
    rng = np.random.default_rng(5)
    lens = rng.integers(1, 40, size=600).astype(np.int32)
    case = synth.paged_case(seed=12, batch=len(lens), len_lo=0, len_hi=0, seq_lens=lens)
    got, k_np, v_np = _run_paged(compute, case)
    assert_attention_close(got, _oracle(case, k_np, v_np), "600 short sequences")


@pytest.mark.parametrize("hq,hkv,d", [(32, 8, 128), (32, 16, 128), (32, 4, 128), (14, 2, 64), (64, 8, 64)])
def test_cut_sequences_merged_inside_the_decode_kernel(compute, hq, hkv, d):
    """Batches large enough for the in-kernel merge (the warp that finishes a cut sequence's last pages
    combines its partials): one sequence cut by almost every CTA among short and empty ones, and a
    batch of mid-sized sequences cut two or three times each.  Same bits on a second run."""
    rng = np.random.default_rng(hq * 100 + hkv)
    skewed = rng.integers(0, 200, size=48).astype(np.int32)
    skewed[17] = 20000
    skewed[3] = 0
    middling = rng.integers(1500, 4000, size=40).astype(np.int32)
    for name, lens in (("one long among short", skewed), ("forty mid-sized", middling)):
        case = synth.paged_case(seed=21, batch=len(lens), len_lo=0, len_hi=0, num_heads=hq, num_kv_heads=hkv,
                                head_dim=d, seq_lens=lens)
        got, k_np, v_np = _run_paged(compute, case)
        assert_attention_close(got, _oracle(case, k_np, v_np), f"{name}, Hq={hq} Hkv={hkv} D={d}")
        again, _, _ = _run_paged(compute, case)
        assert np.array_equal(got, again), name


@pytest.mark.parametrize("hq,hkv,d", [(32, 8, 128), (32, 4, 128), (16, 2, 128), (16, 1, 128), (12, 3, 128), (32, 8, 64)])
def test_one_launch_decode_of_small_batches(compute, hq, hkv, d):
    """Small batches of short sequences (at most 128 pages) take the one-launch path: a few CTAs per
    (sequence, KV head) with an equal share of the pages each, the last one to arrive combining their partials.
    Lengths around the share boundaries, sequences with fewer pages than CTAs (empty shares), empty sequences,
    the same bits on a second run, and calls of different shapes one after the other (the arrival counters
    must be back at zero after every launch)."""
    for lens in ([1], [16], [17], [63], [64], [65], [512], [2047], [2048], [0], [5, 0, 2048], [100, 1999], [777, 33, 1, 1200]):
        case = synth.paged_case(seed=41 + len(lens), batch=len(lens), len_lo=0, len_hi=0, num_heads=hq, num_kv_heads=hkv,
                                head_dim=d, seq_lens=np.array(lens, np.int32), spare_blocks=2)
        got, k_np, v_np = _run_paged(compute, case, poison_unused=True)
        assert_attention_close(got, _oracle(case, k_np, v_np), f"lens={lens} Hq={hq} Hkv={hkv} D={d}")
        again, _, _ = _run_paged(compute, case, poison_unused=True)
        assert np.array_equal(got, again), f"lens={lens}"


@pytest.mark.parametrize("name,lens,d", [("in-kernel merge", [0] + [3000, 40, 1] * 15 + [20000, 0], 128),
                                         ("merge pass", [700, 0, 33, 5000, 16], 128),
                                         ("one launch", [700, 0, 33, 2048, 16], 128),
                                         ("head_dim 64", list(range(1, 1200, 29)), 64),
                                         ("plain kernel", [100, 0, 900], 96)])
def test_decode_with_fused_gather(compute, name, lens, d):
    """The decode that also stores every final row into gather buffers (here two buffers on the same
    GPU standing in for peers): rows row_offset .. row_offset + batch hold exactly the output, every
    other row is untouched.  Covers rows written by the decode kernel itself, by the warp that merges a
    cut sequence, by the separate merge pass, by the one-launch path's last CTA, the zero rows of empty
    sequences and the plain kernel."""
    import torch
    dev = "cuda:0"
    case = synth.paged_case(seed=31, batch=len(lens), len_lo=0, len_hi=0, head_dim=d, seq_lens=np.array(lens, np.int32))
    q = torch.from_numpy(case.q).to(dev)
    k = torch.from_numpy(case.k_pool).to(dev)
    v = torch.from_numpy(case.v_pool).to(dev)
    tables = torch.from_numpy(case.tables).to(dev)
    seq_lens = torch.from_numpy(case.seq_lens).to(dev)
    out = torch.full((case.batch, case.num_heads, d), float("nan"), device=dev)
    total, offset = case.batch + 11, 7
    gathered = [torch.full((total, case.num_heads, d), float("nan"), device=dev) for _ in range(2)]
    compute.batched_paged_attention_decode(q, k, v, tables, seq_lens, out, case.batch, case.num_heads, case.num_kv_heads,
                                           d, synth.PAGE, case.max_blocks, 1.0 / np.sqrt(d), num_blocks=case.num_blocks,
                                           gather_ptrs=[g.data_ptr() for g in gathered], gather_row_offset=offset)
    compute.sync()
    got = out.cpu().numpy()
    ref = _oracle(case, case.k_pool.view(np.uint16), case.v_pool.view(np.uint16))
    assert_attention_close(got, ref, name)
    for g in gathered:
        assert torch.equal(g[offset:offset + case.batch], out), name
        assert torch.isnan(g[:offset]).all() and torch.isnan(g[offset + case.batch:]).all(), name


@pytest.mark.parametrize("lens", [[700, 0, 33, 2048, 16], list(range(1, 3000, 61))])
def test_decode_gather_into_pinned_host_memory(compute, lens):
    """A gather destination may be pinned host memory: the kernel stores the rows over PCIe itself, and after the
    stream is drained the host buffer holds exactly the device output (one-launch path and in-kernel merge)."""
    import torch
    dev = "cuda:0"
    case = synth.paged_case(seed=37, batch=len(lens), len_lo=0, len_hi=0, seq_lens=np.array(lens, np.int32))
    q = torch.from_numpy(case.q).to(dev)
    k = torch.from_numpy(case.k_pool).to(dev)
    v = torch.from_numpy(case.v_pool).to(dev)
    tables = torch.from_numpy(case.tables).to(dev)
    seq_lens = torch.from_numpy(case.seq_lens).to(dev)
    out = torch.full((case.batch, case.num_heads, 128), float("nan"), device=dev)
    host = torch.full((case.batch + 3, case.num_heads, 128), float("nan")).pin_memory()
    compute.batched_paged_attention_decode(q, k, v, tables, seq_lens, out, case.batch, case.num_heads, case.num_kv_heads,
                                           128, synth.PAGE, case.max_blocks, 1.0 / np.sqrt(128.0), num_blocks=case.num_blocks,
                                           gather_ptrs=[host.data_ptr()], gather_row_offset=2)
    compute.sync()
    assert_attention_close(out.cpu().numpy(), _oracle(case, case.k_pool.view(np.uint16), case.v_pool.view(np.uint16)), "host gather")
    assert torch.equal(host[2:2 + case.batch], out.cpu())
    assert torch.isnan(host[:2]).all() and torch.isnan(host[2 + case.batch:]).all()


@pytest.mark.parametrize("ranks,hq,hkv", [(2, 32, 8), (4, 32, 8), (8, 64, 8), (2, 16, 16)])
def test_decode_sharded_by_kv_head(compute, ranks, hq, hkv):
    """Every GPU holds all sequences and num_kv_heads / ranks heads: pool shard [rows, Hkv / ranks, D], the same
    block tables, its groups' query heads.  The ranks run here one after the other on one GPU, each storing its
    head slice into the gathered [B, Hq, D] buffer through the fused gather; the assembled rows must match the
    CPU checker on the unsharded problem and - bit for bit - the unsharded decode when each rank's tile still
    holds whole KV heads."""
    import torch
    from granite_b200 import sharding
    dev = "cuda:0"
    rng = np.random.default_rng(ranks)
    lens = rng.integers(0, 900, size=41).astype(np.int32)
    lens[7] = 6000
    lens[3] = 0
    case = synth.paged_case(seed=51, batch=len(lens), len_lo=0, len_hi=0, num_heads=hq, num_kv_heads=hkv, seq_lens=lens)
    d = case.head_dim
    tables = torch.from_numpy(case.tables).to(dev)
    seq_lens = torch.from_numpy(case.seq_lens).to(dev)
    gathered = torch.full((case.batch + 5, hq, d), float("nan"), device=dev)
    split = sharding.head_split(hq, hkv, ranks)
    assert split is not None and len(split) == ranks
    for r, (kv0, n_kv, q0, n_q) in enumerate(split):
        k = torch.from_numpy(sharding.shard_pool_by_head(case.k_pool, r, ranks)).to(dev)
        v = torch.from_numpy(sharding.shard_pool_by_head(case.v_pool, r, ranks)).to(dev)
        q = torch.from_numpy(sharding.shard_queries_by_head(case.q, r, ranks)).to(dev)
        assert k.shape[1] == n_kv and q.shape[1] == n_q and q0 == r * n_q
        local = torch.full((case.batch, n_q, d), float("nan"), device=dev)
        compute.batched_paged_attention_decode(q, k, v, tables, seq_lens, local, case.batch, n_q, n_kv, d, synth.PAGE,
                                               case.max_blocks, 1.0 / np.sqrt(d), num_blocks=case.num_blocks,
                                               gather_ptrs=[gathered.data_ptr()], gather_row_offset=2,
                                               gather_num_heads=hq, gather_head_offset=q0)
        compute.sync()
        assert torch.equal(gathered[2:2 + case.batch, q0:q0 + n_q], local)
    ref = _oracle(case, case.k_pool.view(np.uint16), case.v_pool.view(np.uint16))
    got = gathered[2:2 + case.batch].cpu().numpy()
    assert_attention_close(got, ref, f"{ranks} ranks by KV head")
    assert torch.isnan(gathered[:2]).all() and torch.isnan(gathered[2 + case.batch:]).all()


def test_head_sharded_gather_is_refused_outside_the_tuned_shapes(compute):
    import torch
    import granite_b200 as g
    dev = "cuda:0"
    case = synth.paged_case(seed=52, batch=2, len_lo=10, len_hi=50, num_heads=6, num_kv_heads=3, head_dim=96)
    out = torch.zeros((2, 6, 96), device=dev)
    gathered = torch.zeros((2, 12, 96), device=dev)
    args = [torch.from_numpy(x).to(dev) for x in (case.q, case.k_pool, case.v_pool, case.tables, case.seq_lens)]
    with pytest.raises(g.GraniteCudaError) as ei:
        compute.batched_paged_attention_decode(*args, out, 2, 6, 3, 96, synth.PAGE, case.max_blocks, 0.1,
                                               num_blocks=case.num_blocks, gather_ptrs=[gathered.data_ptr()],
                                               gather_num_heads=12, gather_head_offset=6)
    assert ei.value.code == g.ErrorCode.InvalidArgument
    with pytest.raises(g.GraniteCudaError):  # the slice would run past the destination row
        compute.batched_paged_attention_decode(*args, out, 2, 6, 3, 96, synth.PAGE, case.max_blocks, 0.1,
                                               num_blocks=case.num_blocks, gather_ptrs=[gathered.data_ptr()],
                                               gather_num_heads=8, gather_head_offset=4)


def test_single_sequence_paged_decode(compute):
    import torch
    case = synth.paged_case(seed=13, batch=1, len_lo=0, len_hi=0, seq_lens=np.array([777], np.int32))
    dev = "cuda:0"
    q = torch.from_numpy(case.q).to(dev)
    k = torch.from_numpy(case.k_pool).to(dev)
    v = torch.from_numpy(case.v_pool).to(dev)
    table = torch.from_numpy(case.tables[0]).to(dev)
    out = torch.zeros((case.num_heads, case.head_dim), device=dev)
    compute.paged_attention_decode(q, k, v, table, out, case.num_heads, case.num_kv_heads, 777,
                                   case.head_dim, synth.PAGE, 1.0 / np.sqrt(128.0), num_blocks=case.num_blocks)
    compute.sync()
    ref = _oracle(case, case.k_pool.view(np.uint16), case.v_pool.view(np.uint16))
    assert_attention_close(out.cpu().numpy()[None], ref, "single sequence")


def test_bad_table_entry_is_reported_not_fatal(compute):
    import granite_b200 as g
    case = synth.paged_case(seed=14, batch=2, len_lo=100, len_hi=200)
    case.tables[1, 2] = case.num_blocks + 5
    with pytest.raises(g.GraniteCudaError) as ei:
        _run_paged(compute, case)
    assert ei.value.code == g.ErrorCode.InvalidArgument
    compute.sync()  # status word was cleared; the context is still usable
    case.tables[1, 2] = 0
    _run_paged(compute, case)


@pytest.mark.parametrize("batch", [37, 64, 192, 193, 300])
def test_batches_around_the_self_planning_limit(compute, batch):
    """Up to 192 sequences every CTA of the decode kernel builds the page prefix sums itself (no plan kernel, the
    page counters reset themselves); larger batches launch the plan kernel.  Ragged lengths with empty sequences,
    twice (the second run needs the counters back at zero), then a different batch size on the same object."""
    rng = np.random.default_rng(900 + batch)
    lens = rng.integers(0, 1500, size=batch).astype(np.int32)
    lens[::7] = 0
    lens[1] = 9000  # cut by many CTAs
    case = synth.paged_case(seed=43, batch=batch, len_lo=0, len_hi=0, seq_lens=lens)
    got, k_np, v_np = _run_paged(compute, case, poison_unused=True)
    ref = _oracle(case, k_np, v_np)
    assert_attention_close(got, ref, f"batch {batch}")
    assert not got[lens == 0].any()
    again, _, _ = _run_paged(compute, case, poison_unused=True)
    assert np.array_equal(got, again)
    other = synth.paged_case(seed=44, batch=50, len_lo=200, len_hi=3000)
    got2, k2, v2 = _run_paged(compute, other)
    assert_attention_close(got2, _oracle(other, k2, v2), "batch 50 after it")


def test_self_planned_batch_of_empty_sequences_and_a_bad_length(compute):
    import granite_b200 as g
    case = synth.paged_case(seed=45, batch=64, len_lo=0, len_hi=0, seq_lens=np.zeros(64, np.int32), spare_blocks=4)
    got, _, _ = _run_paged(compute, case)
    assert not got.any()  # every row is defined to be zero
    case = synth.paged_case(seed=46, batch=64, len_lo=100, len_hi=400)
    good = case.seq_lens.copy()
    case.seq_lens[5] = case.max_blocks * synth.PAGE + 1
    with pytest.raises(g.GraniteCudaError) as ei:
        _run_paged(compute, case)
    assert ei.value.code == g.ErrorCode.InvalidArgument
    compute.sync()
    case.seq_lens[:] = good
    got, k_np, v_np = _run_paged(compute, case)
    assert_attention_close(got, _oracle(case, k_np, v_np), "after the bad length")


def test_unsupported_shapes_are_rejected(compute):
    import torch
    import granite_b200 as g
    t = torch.zeros(16, device="cuda:0")
    # (head_dim 64, 32-token pages or 3 KV heads are not errors: the plain kernel takes them)
    for kw in (dict(head_dim=100), dict(head_dim=512), dict(num_kv_heads=5), dict(block_size=0)):
        args = dict(batch_size=1, num_heads=32, num_kv_heads=8, head_dim=128, block_size=16)
        args.update(kw)
        with pytest.raises(g.GraniteCudaError) as ei:
            compute.batched_paged_attention_decode(t, t, t, t, t, t, args["batch_size"], args["num_heads"],
                                                   args["num_kv_heads"], args["head_dim"], args["block_size"],
                                                   4, 0.1, num_blocks=4)
        assert ei.value.code == g.ErrorCode.InvalidArgument


@pytest.mark.parametrize("seq_kv,max_seq,hq,hkv", [(512, 512, 32, 8), (1, 64, 32, 8), (100, 256, 32, 8), (2048, 4096, 32, 8),
                                                   (333, 333, 32, 8),
                                                   # few KV heads: the warps of a head share its pages
                                                   (3000, 4096, 8, 1), (700, 1024, 16, 2), (129, 256, 32, 4), (900, 900, 12, 3)])
def test_contiguous_decode_matches_cpu(compute, seq_kv, max_seq, hq, hkv):
    """multihead_attention with seq_q == 1 (config: batch 1, Hq 32, Hkv 8, D 128, ctx 512)."""
    import torch
    from oracle import pyoracle
    d = 128
    rng = np.random.default_rng(1001 + seq_kv)
    q = rng.standard_normal((hq, d), np.float32)
    k = rng.standard_normal((hkv, max_seq, d), np.float32).astype(np.float16)
    v = rng.standard_normal((hkv, max_seq, d), np.float32).astype(np.float16)
    # rows past seq_kv are stale cache contents: make them hostile
    k.view(np.uint16)[:, seq_kv:] = 0x7E00
    v.view(np.uint16)[:, seq_kv:] = 0x7E00
    dev = "cuda:0"
    out = torch.zeros((hq, d), device=dev)
    compute.multihead_attention(torch.from_numpy(q).to(dev), torch.from_numpy(k).to(dev),
                                torch.from_numpy(v).to(dev), out, hq, hkv, 1, seq_kv, d,
                                1.0 / np.sqrt(d), max_seq)
    compute.sync()
    kf = pyoracle.cache_to_fp32(k.view(np.uint16), seq_kv)
    vf = pyoracle.cache_to_fp32(v.view(np.uint16), seq_kv)
    ref = pyoracle.attention(q[None, None], kf, vf, start_pos=seq_kv - 1)[0, 0]
    assert_attention_close(out.cpu().numpy(), ref, f"contiguous seq_kv={seq_kv}")


@pytest.mark.parametrize("hq,hkv", [(32, 8), (32, 4), (14, 2), (8, 8), (16, 1), (64, 8)])
def test_paged_decode_head_dim_64(compute, hq, hkv):
    """The same split-KV kernel built for head_dim 64 (one 128-byte swizzle block per row, 16 KB pages
    of eight heads, a 14-deep ring)."""
    case = synth.paged_case(seed=90 + hq + hkv, batch=7, len_lo=0, len_hi=0, num_heads=hq, num_kv_heads=hkv, head_dim=64,
                            seq_lens=np.array([1, 15, 16, 17, 700, 0, 3001], np.int32), spare_blocks=2)
    got, k_np, v_np = _run_paged(compute, case, poison_unused=True)
    assert_attention_close(got, _oracle(case, k_np, v_np), f"D=64 Hq={hq} Hkv={hkv}")
    assert not got[5].any()


def test_contiguous_decode_head_dim_64(compute):
    import torch
    from oracle import pyoracle
    hq, hkv, d, seq_kv, max_seq = 32, 8, 64, 777, 1024
    rng = np.random.default_rng(3)
    q = rng.standard_normal((hq, d), dtype=np.float32)
    k = rng.standard_normal((hkv, max_seq, d), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((hkv, max_seq, d), dtype=np.float32).astype(np.float16)
    k.view(np.uint16)[:, seq_kv:] = 0x7E00
    v.view(np.uint16)[:, seq_kv:] = 0x7E00
    out = torch.zeros((hq, d), device="cuda:0")
    compute.multihead_attention(torch.from_numpy(q).to("cuda:0"), torch.from_numpy(k).to("cuda:0"),
                                torch.from_numpy(v).to("cuda:0"), out, hq, hkv, 1, seq_kv, d, 1.0 / np.sqrt(d), max_seq)
    compute.sync()
    ref = pyoracle.attention(q[None, None], pyoracle.cache_to_fp32(k.view(np.uint16), seq_kv),
                             pyoracle.cache_to_fp32(v.view(np.uint16), seq_kv), start_pos=seq_kv - 1, scale=1.0 / np.sqrt(d))[0, 0]
    assert_attention_close(out.cpu().numpy(), ref, "contiguous decode D=64")
