"""RoPE, the fused RoPE + paged K/V write, the tree commit copy and chunked prefill over the paged
cache, on the GPU through the C ABI, against the CPU checker.

Rotated values, cache bytes and committed rows are compared bit for bit (the rotation follows
src/llm/rope.cpp:52-86 with the host-built tables, the narrowing src/llm/math_ops.cpp:45-54, the
addressing include/granite/metal_compute.h:853-861); attention outputs within the path's tolerance.
"""
import numpy as np
import pytest

from conftest import assert_attention_close
from granite_b200 import synth
from granite_b200.capi import ErrorCode, GraniteCudaError

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _dev_table(compute, max_seq, d, theta=10000.0):
    import torch
    cos_p, sin_p = compute.rope_table_create(max_seq, d, theta)
    n = max_seq * (d // 2)
    cos = np.empty(n, np.float32)
    sin = np.empty(n, np.float32)
    compute.read_buffer(cos, cos_p, n * 4)
    compute.read_buffer(sin, sin_p, n * 4)
    compute.sync()
    return cos_p, sin_p, cos.reshape(max_seq, d // 2), sin.reshape(max_seq, d // 2)


@pytest.mark.parametrize("max_seq,d,theta", [(4096, 128, 10000.0), (300, 64, 500000.0), (7, 2, 10000.0)])
def test_rope_table_has_the_cpu_bits(compute, max_seq, d, theta):
    from oracle import pyoracle
    cos_p, sin_p, cos, sin = _dev_table(compute, max_seq, d, theta)
    ref_cos, ref_sin = pyoracle.rope_table(max_seq, d, theta)
    assert np.array_equal(cos.view(np.uint32), ref_cos.view(np.uint32))
    assert np.array_equal(sin.view(np.uint32), ref_sin.view(np.uint32))
    compute.destroy_buffer(cos_p)
    compute.destroy_buffer(sin_p)


@pytest.mark.parametrize("seq,hq,hk,d,start", [(1, 32, 8, 128, 511), (5, 32, 8, 128, 700), (3, 4, 4, 64, 0), (2, 8, 0, 16, 3)])
def test_rope_multihead_is_bit_exact(compute, seq, hq, hk, d, start):
    import torch
    from oracle import pyoracle
    rng = np.random.default_rng(seq * 100 + hq)
    max_seq = 1024
    cos_p, sin_p, cos, sin = _dev_table(compute, max_seq, d)
    q = rng.standard_normal((seq, hq, d), dtype=np.float32)
    k = rng.standard_normal((seq, max(hk, 1), d), dtype=np.float32)
    qd = torch.from_numpy(q).to(DEV)
    kd = torch.from_numpy(k).to(DEV)
    compute.rope_multihead(qd, kd if hk else None, hq, hk, seq, d, start, cos_p, sin_p, max_seq)
    compute.sync()
    assert np.array_equal(qd.cpu().numpy().view(np.uint32), pyoracle.rope_apply(q, start, cos, sin).view(np.uint32))
    if hk:
        assert np.array_equal(kd.cpu().numpy().view(np.uint32), pyoracle.rope_apply(k, start, cos, sin).view(np.uint32))
    else:
        assert np.array_equal(kd.cpu().numpy(), k)
    # positions past the table are refused on the host, as RoPECache::apply does (rope.cpp:34-38)
    with pytest.raises(GraniteCudaError) as e:
        compute.rope_multihead(qd, None, hq, 0, seq, d, max_seq - seq + 1, cos_p, sin_p, max_seq)
    assert e.value.code == ErrorCode.InvalidArgument
    compute.destroy_buffer(cos_p)
    compute.destroy_buffer(sin_p)


def _append_case(seed, batch, new_len, hq, hkv, d, len_hi):
    rng = np.random.default_rng(seed)
    old_lens = rng.integers(0, len_hi, size=batch).astype(np.int32)
    case = synth.paged_case(seed, batch, 0, 0, hq, hkv, d, seq_lens=old_lens + new_len, spare_blocks=3)
    q = rng.standard_normal((batch, new_len, hq, d), dtype=np.float32)
    k = rng.standard_normal((batch, new_len, hkv, d), dtype=np.float32)
    v = rng.standard_normal((batch, new_len, hkv, d), dtype=np.float32)
    # values that exercise the truncating cast: tiny (flushed), huge (clamped), negative zero
    k[0, 0, 0, :4] = [1e-8, -1e-8, 1e6, -0.0]
    v[0, 0, 0, :4] = [7e4, -7e4, 6e-5, 5.96e-8]
    return case, old_lens, q, k, v


@pytest.mark.parametrize("batch,new_len,hq,hkv", [(64, 1, 32, 8), (5, 1, 32, 4), (3, 37, 32, 8), (1, 300, 8, 8), (2, 16, 0, 2)])
def test_rope_paged_append_writes_the_cpu_bytes(compute, batch, new_len, hq, hkv):
    import torch
    from oracle import pyoracle
    d = 128
    case, old_lens, q, k, v = _append_case(31 + batch + new_len, batch, new_len, max(hq, 1), hkv, d, 400)
    max_seq = 1024
    cos_p, sin_p, cos, sin = _dev_table(compute, max_seq, d)
    k_np = case.k_pool.view(np.uint16).copy()
    v_np = case.v_pool.view(np.uint16).copy()
    kd = torch.from_numpy(k_np.view(np.float16)).to(DEV)
    vd = torch.from_numpy(v_np.view(np.float16)).to(DEV)
    tables = np.where(case.tables < 0, 0, case.tables).astype(np.int32)
    qd = torch.from_numpy(q).to(DEV) if hq else None
    newk, newv = torch.from_numpy(k).to(DEV), torch.from_numpy(v).to(DEV)
    compute.rope_paged_kv_cache_append(qd, newk, newv, cos_p, sin_p, kd, vd, torch.from_numpy(tables).to(DEV),
                                       torch.from_numpy(old_lens).to(DEV), batch, new_len, hq, hkv, d, synth.PAGE,
                                       case.max_blocks, case.num_blocks, max_seq)
    compute.sync()
    q_ref, bad = pyoracle.rope_paged_append(q if hq else None, k, v, cos, sin, k_np, v_np, tables, old_lens, synth.PAGE)
    assert bad == 0
    assert np.array_equal(kd.cpu().numpy().view(np.uint16), k_np)
    assert np.array_equal(vd.cpu().numpy().view(np.uint16), v_np)
    if hq:
        assert np.array_equal(qd.cpu().numpy().view(np.uint32), q_ref.view(np.uint32))
    assert np.array_equal(newk.cpu().numpy(), k) and np.array_equal(newv.cpu().numpy(), v)  # inputs untouched
    compute.destroy_buffer(cos_p)
    compute.destroy_buffer(sin_p)


def test_decode_step_append_then_attend(compute):
    """One decode step of a batch as Granite runs it (src/llm/transformer.mm:2975-3000): rotate, write
    the new token's K/V into the pages, attend over the grown sequences."""
    import torch
    from oracle import pyoracle
    batch, hq, hkv, d = 9, 32, 8, 128
    case, old_lens, q, k, v = _append_case(77, batch, 1, hq, hkv, d, 900)
    k[0, 0, 0, :4] = 0.5
    v[0, 0, 0, :4] = 0.25
    max_seq = 1024
    cos_p, sin_p, cos, sin = _dev_table(compute, max_seq, d)
    k_np = case.k_pool.view(np.uint16).copy()
    v_np = case.v_pool.view(np.uint16).copy()
    kd = torch.from_numpy(k_np.view(np.float16)).to(DEV)
    vd = torch.from_numpy(v_np.view(np.float16)).to(DEV)
    tables = np.where(case.tables < 0, 0, case.tables).astype(np.int32)
    td = torch.from_numpy(tables).to(DEV)
    qd = torch.from_numpy(q).to(DEV)
    compute.rope_paged_kv_cache_append(qd, torch.from_numpy(k).to(DEV), torch.from_numpy(v).to(DEV), cos_p, sin_p,
                                       kd, vd, td, torch.from_numpy(old_lens).to(DEV), batch, 1, hq, hkv, d,
                                       synth.PAGE, case.max_blocks, case.num_blocks, max_seq)
    new_lens = (old_lens + 1).astype(np.int32)
    out = torch.full((batch, hq, d), float("nan"), device=DEV)
    compute.batched_paged_attention_decode(qd, kd, vd, td, torch.from_numpy(new_lens).to(DEV), out, batch, hq, hkv, d,
                                           synth.PAGE, case.max_blocks, 1.0 / np.sqrt(d), num_blocks=case.num_blocks)
    compute.sync()
    q_ref, bad = pyoracle.rope_paged_append(q, k, v, cos, sin, k_np, v_np, tables, old_lens, synth.PAGE)
    ref, bad2 = pyoracle.paged_decode_batch(q_ref.reshape(batch, hq, d), k_np, v_np, tables, new_lens, synth.PAGE)
    assert bad == 0 and bad2 == 0
    assert_attention_close(out.cpu().numpy(), ref, "decode step")
    compute.destroy_buffer(cos_p)
    compute.destroy_buffer(sin_p)


def test_rope_paged_append_reports_bad_positions_and_entries(compute):
    import torch
    batch, hq, hkv, d = 3, 4, 2, 128
    case, old_lens, q, k, v = _append_case(5, batch, 1, hq, hkv, d, 40)
    max_seq = 64
    cos_p, sin_p, _, _ = _dev_table(compute, max_seq, d)
    kd = torch.from_numpy(case.k_pool.copy()).to(DEV)
    vd = torch.from_numpy(case.v_pool.copy()).to(DEV)
    before = kd.clone()
    tables = np.where(case.tables < 0, 0, case.tables).astype(np.int32)

    def run(tab, pos):
        compute.rope_paged_kv_cache_append(torch.from_numpy(q).to(DEV), torch.from_numpy(k).to(DEV),
                                           torch.from_numpy(v).to(DEV), cos_p, sin_p, kd, vd,
                                           torch.from_numpy(tab).to(DEV), torch.from_numpy(pos).to(DEV), batch, 1, hq,
                                           hkv, d, synth.PAGE, case.max_blocks, case.num_blocks, max_seq)
        compute.sync()

    bad_tab = tables.copy()
    bad_tab[:, :] = case.num_blocks  # every entry outside the pool: nothing may be written
    with pytest.raises(GraniteCudaError) as e:
        run(bad_tab, old_lens)
    assert e.value.code == ErrorCode.InvalidArgument
    assert torch.equal(kd, before)
    with pytest.raises(GraniteCudaError) as e:
        run(tables, np.full(batch, max_seq, np.int32))  # past the RoPE table
    assert e.value.code == ErrorCode.InvalidArgument
    assert torch.equal(kd, before)
    run(tables, old_lens)  # the object is still usable
    compute.destroy_buffer(cos_p)
    compute.destroy_buffer(sin_p)


@pytest.mark.parametrize("batch,n,max_acc", [(16, 64, 9), (3, 7, 7), (1, 1, 1)])
def test_tree_commit_moves_the_accepted_rows(compute, batch, n, max_acc):
    import torch
    from oracle import pyoracle
    hkv, d = 8, 128
    rng = np.random.default_rng(batch * 10 + n)
    cache_lens = rng.integers(0, 300, size=batch).astype(np.int32)
    case = synth.paged_case(3, batch, 0, 0, 32, hkv, d, seq_lens=cache_lens + max_acc, spare_blocks=2)
    tables = np.where(case.tables < 0, 0, case.tables).astype(np.int32)
    k_tree = rng.integers(0, 65536, size=(batch, hkv, n, d)).astype(np.uint16)
    v_tree = rng.integers(0, 65536, size=(batch, hkv, n, d)).astype(np.uint16)
    num_acc = rng.integers(0, max_acc + 1, size=batch).astype(np.int32)
    num_acc[0] = max_acc
    accepted = np.full((batch, max_acc), -1, np.int32)
    for b in range(batch):  # a root-first path visits increasing node indices
        accepted[b, :num_acc[b]] = np.sort(rng.permutation(n)[:num_acc[b]])
    k_np = case.k_pool.view(np.uint16).copy()
    v_np = case.v_pool.view(np.uint16).copy()
    kd = torch.from_numpy(k_np.view(np.float16)).to(DEV)
    vd = torch.from_numpy(v_np.view(np.float16)).to(DEV)
    compute.tree_commit(torch.from_numpy(k_tree.view(np.float16)).to(DEV), torch.from_numpy(v_tree.view(np.float16)).to(DEV),
                        kd, vd, torch.from_numpy(tables).to(DEV), torch.from_numpy(cache_lens).to(DEV),
                        torch.from_numpy(accepted).to(DEV), torch.from_numpy(num_acc).to(DEV), batch, n, max_acc, hkv, d,
                        synth.PAGE, case.max_blocks, case.num_blocks)
    compute.sync()
    assert pyoracle.tree_commit(k_tree, v_tree, k_np, v_np, tables, cache_lens, accepted, num_acc, synth.PAGE) == 0
    assert np.array_equal(kd.cpu().numpy().view(np.uint16), k_np)
    assert np.array_equal(vd.cpu().numpy().view(np.uint16), v_np)


def _paged_sequence(seed, total, hq, hkv, d):
    case = synth.paged_case(seed, 1, 0, 0, hq, hkv, d, seq_lens=np.array([total], np.int32), spare_blocks=4)
    k_np = case.k_pool.view(np.uint16).copy()
    v_np = case.v_pool.view(np.uint16).copy()
    # rows no live token maps to are NaN: nothing past the sequence may leak into the result
    live = np.zeros(case.num_blocks * synth.PAGE, bool)
    for pos in range(total):
        live[case.tables[0, pos // synth.PAGE] * synth.PAGE + pos % synth.PAGE] = True
    k_np[~live] = 0x7E00
    v_np[~live] = 0x7E00
    return case, k_np, v_np


@pytest.mark.parametrize("start,seq_q,hq,hkv,q16", [(0, 200, 32, 8, True), (128, 128, 32, 8, True), (300, 77, 32, 8, False),
                                                    (1000, 1, 8, 8, True), (513, 400, 16, 4, True)])
def test_chunked_prefill_over_pages_matches_cpu(compute, start, seq_q, hq, hkv, q16):
    import torch
    from oracle import pyoracle
    d = 128
    total = start + seq_q
    case, k_np, v_np = _paged_sequence(start + seq_q, total, hq, hkv, d)
    rng = np.random.default_rng(start)
    q = rng.standard_normal((seq_q, hq, d), dtype=np.float32)
    if q16:
        q = q.astype(np.float16).astype(np.float32)
    table = np.where(case.tables[0] < 0, 0, case.tables[0]).astype(np.int32)
    qd = torch.from_numpy(q.astype(np.float16) if q16 else q).to(DEV)
    out = torch.full((seq_q, hq, d), float("nan"), device=DEV)
    compute.paged_prefill_attention(qd, torch.from_numpy(k_np.view(np.float16)).to(DEV),
                                    torch.from_numpy(v_np.view(np.float16)).to(DEV), torch.from_numpy(table).to(DEV), out,
                                    hq, hkv, seq_q, start, d, synth.PAGE, case.max_blocks, case.num_blocks,
                                    1.0 / np.sqrt(d), q_dtype=1 if q16 else 0, out_dtype=0)
    compute.sync()
    k_rows, bad = pyoracle.paged_gather(k_np, table, total, synth.PAGE)
    v_rows, bad2 = pyoracle.paged_gather(v_np, table, total, synth.PAGE)
    assert bad == 0 and bad2 == 0
    ref = pyoracle.attention(q[None], pyoracle.f16_bits_to_f32(k_rows), pyoracle.f16_bits_to_f32(v_rows), start)
    assert_attention_close(out.cpu().numpy(), ref.reshape(seq_q, hq, d), f"chunk at {start}")


def test_chunked_prefill_rejects_a_chunk_beyond_the_table(compute):
    import torch
    d, hq, hkv = 128, 8, 8
    case, k_np, v_np = _paged_sequence(1, 64, hq, hkv, d)
    q = torch.zeros((32, hq, d), device=DEV)
    with pytest.raises(GraniteCudaError) as e:
        compute.paged_prefill_attention(q, torch.from_numpy(k_np.view(np.float16)).to(DEV),
                                        torch.from_numpy(v_np.view(np.float16)).to(DEV),
                                        torch.from_numpy(case.tables[0].copy()).to(DEV), torch.zeros_like(q), hq, hkv, 32,
                                        case.max_blocks * synth.PAGE - 16, d, synth.PAGE, case.max_blocks, case.num_blocks,
                                        0.1)
    assert e.value.code == ErrorCode.InvalidArgument


def test_verify_commit_then_decode(compute):
    """The speculative step end to end: verify a tree against the paged prefix, keep an accepted
    path with the commit copy, and decode the next token over the grown cache - the committed rows
    must serve exactly as if they had been appended one by one."""
    import torch
    from oracle import pyoracle
    from test_tree_verify import _tree_inputs
    batch, n, hq, hkv, d = 4, 64, 32, 8, 128
    rng = np.random.default_rng(21)
    cache_lens = np.array([100, 16, 333, 0], np.int32)
    max_acc = 8
    case = synth.paged_case(55, batch, 0, 0, hq, hkv, d, seq_lens=cache_lens + max_acc, spare_blocks=2)
    tables = np.where(case.tables < 0, 0, case.tables).astype(np.int32)
    q, kt, vt, parents = _tree_inputs(9, batch, n, hq, hkv)
    k_np = case.k_pool.view(np.uint16).copy()
    v_np = case.v_pool.view(np.uint16).copy()
    kd = torch.from_numpy(k_np.view(np.float16)).to(DEV)
    vd = torch.from_numpy(v_np.view(np.float16)).to(DEV)
    td = torch.from_numpy(tables).to(DEV)
    ktd, vtd = torch.from_numpy(kt).to(DEV), torch.from_numpy(vt).to(DEV)
    out = torch.zeros((batch, hq, n, d), device=DEV)
    compute.attention_tree(torch.from_numpy(q).to(DEV), kd, vd, ktd, vtd, torch.from_numpy(parents).to(DEV), out, hq, hkv,
                           n, 0, d, 1.0 / np.sqrt(d), batch_size=batch, block_tables=td, max_blocks_per_seq=case.max_blocks,
                           num_blocks=case.num_blocks, cache_lens=torch.from_numpy(cache_lens).to(DEV))
    # accepted path per sequence: a root-to-node chain of the tree (what find_accepted_nodes returns)
    accepted = np.full((batch, max_acc), -1, np.int32)
    num_acc = np.zeros(batch, np.int32)
    for b in range(batch):
        node = int(rng.integers(0, n))
        chain = []
        while node >= 0:
            chain.append(node)
            node = int(parents[b, node])
        chain = chain[::-1][:max_acc]
        accepted[b, :len(chain)] = chain
        num_acc[b] = len(chain)
    compute.tree_commit(ktd, vtd, kd, vd, td, torch.from_numpy(cache_lens).to(DEV), torch.from_numpy(accepted).to(DEV),
                        torch.from_numpy(num_acc).to(DEV), batch, n, max_acc, hkv, d, synth.PAGE, case.max_blocks,
                        case.num_blocks)
    new_lens = (cache_lens + num_acc).astype(np.int32)
    q1 = rng.standard_normal((batch, hq, d), dtype=np.float32)
    out1 = torch.zeros((batch, hq, d), device=DEV)
    compute.batched_paged_attention_decode(torch.from_numpy(q1).to(DEV), kd, vd, td, torch.from_numpy(new_lens).to(DEV), out1,
                                           batch, hq, hkv, d, synth.PAGE, case.max_blocks, 1.0 / np.sqrt(d),
                                           num_blocks=case.num_blocks)
    compute.sync()
    # checker: the same commit on the host copies, then decode; and the verification itself per sequence
    assert pyoracle.tree_commit(kt.view(np.uint16), vt.view(np.uint16), k_np, v_np, tables, cache_lens, accepted, num_acc,
                                synth.PAGE) == 0
    assert np.array_equal(kd.cpu().numpy().view(np.uint16), k_np)
    ref1, bad = pyoracle.paged_decode_batch(q1, k_np, v_np, tables, new_lens, synth.PAGE)
    assert bad == 0
    assert_attention_close(out1.cpu().numpy(), ref1, "decode after commit")
    # the last accepted node's verification output equals plain causal attention over prefix + path
    got = out.cpu().numpy()
    for b in range(batch):
        if num_acc[b] == 0:
            continue
        last = int(accepted[b, num_acc[b] - 1])
        rows_k, _ = pyoracle.paged_gather(k_np, tables[b], int(new_lens[b]), synth.PAGE)
        rows_v, _ = pyoracle.paged_gather(v_np, tables[b], int(new_lens[b]), synth.PAGE)
        ref = pyoracle.attention(q[b, :, last][None, None], pyoracle.f16_bits_to_f32(rows_k), pyoracle.f16_bits_to_f32(rows_v),
                                 int(new_lens[b]) - 1)
        assert_attention_close(got[b, :, last], ref[0, 0], f"sequence {b}: tree output of the path's last node")


def test_push_rows_copies_to_every_destination(compute):
    """The output gather's push kernel, with local buffers standing in for the peers' memory."""
    import torch
    src = torch.randn((64, 32, 128), device=DEV)
    dsts = [torch.full((4 * 64, 32, 128), float("nan"), device=DEV) for _ in range(3)]
    nbytes = src.numel() * 4
    compute.push_rows(src, dsts, 2 * nbytes, nbytes)
    compute.sync()
    for d in dsts:
        assert torch.equal(d[128:192], src)
        assert torch.isnan(d[:128]).all() and torch.isnan(d[192:]).all()
    with pytest.raises(GraniteCudaError) as e:
        compute.push_rows(src, dsts, 8, nbytes)  # offset not 16-byte aligned
    assert e.value.code == ErrorCode.InvalidArgument
    with pytest.raises(GraniteCudaError) as e:
        compute.push_rows(src, [dsts[0]] * 17, 0, nbytes)
    assert e.value.code == ErrorCode.InvalidArgument


def test_an_expired_device_wait_ends_as_an_error_code(compute):
    """The safety net under every pipeline: a wait whose signal never comes expires, the status word
    reaches the host as Timeout, a second waiter leaves through the abort flag, and the same compute
    object goes on working."""
    import torch
    released = torch.zeros(1, dtype=torch.int32, device=DEV)
    compute.selftest_bounded_wait(2_000_000, released)  # about one millisecond
    with pytest.raises(GraniteCudaError) as e:
        compute.sync()
    assert e.value.code == ErrorCode.Timeout
    assert int(released.item()) == 1
    compute.sync()  # cleared
    src = torch.arange(1024, dtype=torch.float32, device=DEV)
    dst = torch.zeros_like(src)
    compute.push_rows(src, [dst], 0, 4096)
    compute.sync()
    assert torch.equal(src, dst)
    with pytest.raises(GraniteCudaError) as e:
        compute.selftest_bounded_wait(10**10, released)  # limits above 0.1 s are refused
    assert e.value.code == ErrorCode.InvalidArgument
