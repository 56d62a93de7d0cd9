"""Shapes beside the benchmarked ones through the same entry points and the same checker: head_dim
64 (which the reference's GPU path also serves, src/backend/metal/metal_compute.mm:2550-2561) on the
tuned kernels; head_dim 96 / 256 and 32-token pages on the plain fp32 kernel; odd KV-head counts."""
import numpy as np
import pytest

from conftest import assert_attention_close
import test_prefill as TP
import test_tree_verify as TT

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _paged(rng, lens, hkv, d, bs):
    pages = [(int(n) + bs - 1) // bs for n in lens]
    num_blocks = sum(pages) + 2
    perm = rng.permutation(num_blocks).astype(np.int32)
    max_blocks = max(max(pages), 1)
    tables = np.zeros((len(lens), max_blocks), np.int32)
    off = 0
    for b, n in enumerate(pages):
        tables[b, :n] = perm[off:off + n]
        off += n
    k = rng.standard_normal((num_blocks * bs, hkv, d), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((num_blocks * bs, hkv, d), dtype=np.float32).astype(np.float16)
    return tables, num_blocks, k, v


@pytest.mark.parametrize("hq,hkv,d,bs", [(32, 8, 64, 16), (8, 2, 64, 32), (12, 3, 128, 16), (32, 8, 128, 32), (4, 4, 256, 16),
                                         (6, 6, 96, 8)])
def test_paged_decode_other_shapes(compute, hq, hkv, d, bs):
    import torch
    from oracle import pyoracle
    rng = np.random.default_rng(hq * 100 + d + bs)
    lens = np.array([1, bs, bs + 1, 300, 0, 1000], np.int32)
    tables, num_blocks, k, v = _paged(rng, lens, hkv, d, bs)
    q = rng.standard_normal((len(lens), hq, d), dtype=np.float32)
    out = torch.full((len(lens), hq, d), float("nan"), device=DEV)
    compute.batched_paged_attention_decode(torch.from_numpy(q).to(DEV), torch.from_numpy(k).to(DEV), torch.from_numpy(v).to(DEV),
                                           torch.from_numpy(tables).to(DEV), torch.from_numpy(lens).to(DEV), out, len(lens),
                                           hq, hkv, d, bs, tables.shape[1], 1.0 / np.sqrt(d), num_blocks=num_blocks)
    compute.sync()
    ref, bad = pyoracle.paged_decode_batch(q, k.view(np.uint16), v.view(np.uint16), tables, lens, bs, scale=1.0 / np.sqrt(d))
    assert bad == 0
    got = out.cpu().numpy()
    assert_attention_close(got, ref, f"decode Hq={hq} Hkv={hkv} D={d} page={bs}")
    assert not got[4].any()  # the empty sequence


@pytest.mark.parametrize("seq_q,start,hq,hkv,d,q16,out16", [(200, 0, 8, 2, 64, True, True), (77, 300, 6, 3, 64, False, False),
                                                            (130, 5, 4, 1, 256, True, False)])
def test_prefill_other_head_dims(compute, seq_q, start, hq, hkv, d, q16, out16):
    seq_kv = start + seq_q
    q, k, v = TP._case(seq_q + d, seq_q, seq_kv, seq_kv + 9, hq, hkv, d=d)
    got = TP._run(compute, q, k, v, seq_kv, start, q16, out16)
    import torch  # noqa: F401
    from oracle import pyoracle
    qq = q.astype(np.float16).astype(np.float32) if q16 else q
    kf = pyoracle.cache_to_fp32(k.view(np.uint16), seq_kv)
    vf = pyoracle.cache_to_fp32(v.view(np.uint16), seq_kv)
    ref = pyoracle.attention(qq[None], kf, vf, start_pos=start, scale=1.0 / np.sqrt(d))[0]
    assert_attention_close(got, ref, f"prefill D={d}")


@pytest.mark.parametrize("d,bs,n,hq,hkv", [(64, 16, 64, 8, 2), (64, 32, 20, 4, 4), (128, 32, 33, 8, 2)])
def test_tree_other_shapes(compute, d, bs, n, hq, hkv):
    import torch
    from oracle import pyoracle
    from granite_b200 import synth
    rng = np.random.default_rng(d + bs + n)
    lens = np.array([0, 100, 333], np.int32)
    batch = len(lens)
    tables, num_blocks, k, v = _paged(rng, lens, hkv, d, bs)
    q = rng.standard_normal((batch, hq, n, d), dtype=np.float32)
    kt = rng.standard_normal((batch, hkv, n, d), dtype=np.float32).astype(np.float16)
    vt = rng.standard_normal((batch, hkv, n, d), dtype=np.float32).astype(np.float16)
    parents = np.stack([synth.tree_parents(int(rng.integers(1 << 30)), n) for _ in range(batch)])
    out = torch.full((batch, hq, n, d), float("nan"), device=DEV)
    compute.attention_tree(torch.from_numpy(q).to(DEV), torch.from_numpy(k).to(DEV), torch.from_numpy(v).to(DEV),
                           torch.from_numpy(kt).to(DEV), torch.from_numpy(vt).to(DEV), torch.from_numpy(parents).to(DEV), out,
                           hq, hkv, n, 0, d, 1.0 / np.sqrt(d), batch_size=batch, block_tables=torch.from_numpy(tables).to(DEV),
                           cache_lens=torch.from_numpy(lens).to(DEV), block_size=bs, max_blocks_per_seq=tables.shape[1],
                           num_blocks=num_blocks)
    compute.sync()
    got = out.cpu().numpy()
    for b in range(batch):
        kr, _ = pyoracle.paged_gather(k.view(np.uint16), tables[b], int(lens[b]), bs)
        vr, _ = pyoracle.paged_gather(v.view(np.uint16), tables[b], int(lens[b]), bs)
        q4 = np.ascontiguousarray(q[b].transpose(1, 0, 2))[None]
        ktb = np.ascontiguousarray(kt[b].astype(np.float32).transpose(1, 0, 2))[None]
        vtb = np.ascontiguousarray(vt[b].astype(np.float32).transpose(1, 0, 2))[None]
        ref = pyoracle.attention_tree(q4, pyoracle.f16_bits_to_f32(kr), pyoracle.f16_bits_to_f32(vr), ktb, vtb, parents[b],
                                      scale=1.0 / np.sqrt(d))[0].transpose(1, 0, 2)
        assert_attention_close(got[b], ref, f"tree D={d} page={bs} N={n} prefix={int(lens[b])}")


@pytest.mark.parametrize("seq_q,start,hq,hkv,q16,out16", [(300, 0, 8, 2, True, True), (129, 0, 4, 4, False, False),
                                                          (77, 500, 12, 3, True, False), (1024, 0, 8, 1, True, True),
                                                          (2, 0, 2, 1, False, True)])
def test_prefill_head_dim_64_on_the_tensor_kernel(compute, seq_q, start, hq, hkv, q16, out16):
    """head_dim 64 runs on the tcgen05 kernel too (half of every tile slot, four score steps, 64 output
    columns); stale cache rows are NaN."""
    from oracle import pyoracle
    d = 64
    seq_kv = start + seq_q
    q, k, v = TP._case(seq_q * 3 + hq, seq_q, seq_kv, seq_kv + 50, hq, hkv, d=d)
    got = TP._run(compute, q, k, v, seq_kv, start, q16, out16)
    qq = q.astype(np.float16).astype(np.float32) if q16 else q
    ref = pyoracle.attention(qq[None], pyoracle.cache_to_fp32(k.view(np.uint16), seq_kv),
                             pyoracle.cache_to_fp32(v.view(np.uint16), seq_kv), start_pos=start, scale=1.0 / np.sqrt(d))[0]
    assert_attention_close(got, ref, f"prefill D=64 seq_q={seq_q} start={start}")


@pytest.mark.parametrize("n,hq,hkv,q16", [(64, 32, 8, True), (16, 8, 2, False), (33, 6, 6, True), (5, 16, 2, True)])
def test_tree_and_chunked_prefill_head_dim_64(compute, n, hq, hkv, q16):
    import torch
    from oracle import pyoracle
    from granite_b200 import synth
    d, bs = 64, 16
    rng = np.random.default_rng(n * 7 + hq)
    lens = np.array([0, 130, 1000], np.int32)
    batch = len(lens)
    tables, num_blocks, k, v = _paged(rng, lens, hkv, d, bs)
    k_bits, v_bits = k.view(np.uint16).copy(), v.view(np.uint16).copy()
    live = np.zeros(num_blocks * bs, bool)
    for b, length in enumerate(lens):
        for pos in range(int(length)):
            live[tables[b, pos // bs] * bs + pos % bs] = True
    k_bits[~live] = 0x7E00
    v_bits[~live] = 0x7E00
    kd, vd = torch.from_numpy(k_bits.view(np.float16)).to(DEV), torch.from_numpy(v_bits.view(np.float16)).to(DEV)
    q = rng.standard_normal((batch, hq, n, d), dtype=np.float32)
    if q16:
        q = q.astype(np.float16).astype(np.float32)
    kt = rng.standard_normal((batch, hkv, n, d), dtype=np.float32).astype(np.float16)
    vt = rng.standard_normal((batch, hkv, n, d), dtype=np.float32).astype(np.float16)
    parents = np.stack([synth.tree_parents(int(rng.integers(1 << 30)), n) for _ in range(batch)])
    out = torch.full((batch, hq, n, d), float("nan"), device=DEV)
    compute.attention_tree(torch.from_numpy(q.astype(np.float16) if q16 else q).to(DEV), kd, vd, torch.from_numpy(kt).to(DEV),
                           torch.from_numpy(vt).to(DEV), torch.from_numpy(parents).to(DEV), out, hq, hkv, n, 0, d,
                           1.0 / np.sqrt(d), batch_size=batch, block_tables=torch.from_numpy(tables).to(DEV),
                           cache_lens=torch.from_numpy(lens).to(DEV), block_size=bs, max_blocks_per_seq=tables.shape[1],
                           num_blocks=num_blocks, q_dtype=int(q16))
    compute.sync()
    got = out.cpu().numpy()
    for b in range(batch):
        kr, _ = pyoracle.paged_gather(k_bits, tables[b], int(lens[b]), bs)
        vr, _ = pyoracle.paged_gather(v_bits, tables[b], int(lens[b]), bs)
        q4 = np.ascontiguousarray(q[b].transpose(1, 0, 2))[None]
        ktb = np.ascontiguousarray(kt[b].astype(np.float32).transpose(1, 0, 2))[None]
        vtb = np.ascontiguousarray(vt[b].astype(np.float32).transpose(1, 0, 2))[None]
        ref = pyoracle.attention_tree(q4, pyoracle.f16_bits_to_f32(kr), pyoracle.f16_bits_to_f32(vr), ktb, vtb, parents[b],
                                      scale=1.0 / np.sqrt(d))[0].transpose(1, 0, 2)
        assert_attention_close(got[b], ref, f"tree D=64 N={n} prefix={int(lens[b])}")
    # a chunk of the longest sequence through the block table
    start, seq_q = 700, 300
    cq = rng.standard_normal((seq_q, hq, d), dtype=np.float32).astype(np.float16)
    cout = torch.full((seq_q, hq, d), float("nan"), device=DEV)
    compute.paged_prefill_attention(torch.from_numpy(cq).to(DEV), kd, vd, torch.from_numpy(tables[2].copy()).to(DEV), cout, hq,
                                    hkv, seq_q, start, d, bs, tables.shape[1], num_blocks, 1.0 / np.sqrt(d), q_dtype=1, out_dtype=0)
    compute.sync()
    kr, _ = pyoracle.paged_gather(k_bits, tables[2], start + seq_q, bs)
    vr, _ = pyoracle.paged_gather(v_bits, tables[2], start + seq_q, bs)
    ref = pyoracle.attention(cq.astype(np.float32)[None], pyoracle.f16_bits_to_f32(kr), pyoracle.f16_bits_to_f32(vr),
                             start_pos=start, scale=1.0 / np.sqrt(d))[0]
    assert_attention_close(cout.cpu().numpy(), ref, "chunked prefill D=64")
