"""The compute object's cache of TMA descriptors under churn.

Descriptors are cached per (buffer, shape); the cache is bounded, and a launcher holds up to six
descriptor pointers while it fetches the next one.  A serving loop with changing Q / output / K / V
buffers walks through hundreds of keys, so eviction must never drop an entry that the current call
already holds.  One compute object of its own is pushed through more than 300 distinct buffers -
prefill, tree verification and paged decode in turn - and every result is checked against the CPU
checker.
"""
import numpy as np
import pytest

from conftest import assert_attention_close
from granite_b200 import synth

pytestmark = pytest.mark.gpu
D = 128


def test_descriptor_cache_survives_hundreds_of_distinct_buffers():
    import torch
    import granite_b200 as g
    from oracle import pyoracle
    torch.cuda.set_device(0)
    dev = "cuda:0"
    c = g.CudaCompute(0, torch.cuda.current_stream().cuda_stream)
    keep = []  # every buffer stays alive, so every iteration brings new addresses
    rng = np.random.default_rng(88)
    scale = 1.0 / np.sqrt(D)
    hq, hkv = 4, 1
    page_case = synth.paged_case(seed=31, batch=2, len_lo=40, len_hi=300, num_heads=hq, num_kv_heads=hkv)
    kpool = torch.from_numpy(page_case.k_pool).to(dev)
    vpool = torch.from_numpy(page_case.v_pool).to(dev)
    tables = torch.from_numpy(np.where(page_case.tables < 0, 0, page_case.tables).astype(np.int32)).to(dev)
    lens = torch.from_numpy(page_case.seq_lens).to(dev)
    k_bits, v_bits = page_case.k_pool.view(np.uint16), page_case.v_pool.view(np.uint16)
    dec_ref, bad = pyoracle.paged_decode_batch(page_case.q, k_bits, v_bits, np.where(page_case.tables < 0, 0, page_case.tables),
                                               page_case.seq_lens, synth.PAGE)
    assert bad == 0
    try:
        for it in range(120):
            # causal prefill, fp32 Q (two descriptors for Q's hi/lo halves, one each for K and V)
            seq = int(rng.integers(2, 140))
            q = rng.standard_normal((seq, hq, D), np.float32)
            k = rng.standard_normal((hkv, seq, D), np.float32).astype(np.float16)
            v = rng.standard_normal((hkv, seq, D), np.float32).astype(np.float16)
            qd, kd, vd = (torch.from_numpy(x).to(dev) for x in (q, k, v))
            out = torch.full((seq, hq, D), float("nan"), device=dev)
            keep += [qd, kd, vd, out]
            c.multihead_attention(qd, kd, vd, out, hq, hkv, seq, seq, D, scale, seq, q_dtype=0, out_dtype=0)
            c.sync()
            ref = pyoracle.attention(q[None], pyoracle.cache_to_fp32(k.view(np.uint16), seq),
                                     pyoracle.cache_to_fp32(v.view(np.uint16), seq), start_pos=0)[0]
            assert_attention_close(out.cpu().numpy(), ref, f"prefill, iteration {it}")

            # tree verification over the paged prefix of sequence 0 (six descriptors per call)
            n = int(rng.integers(1, 65))
            parents = synth.tree_parents(1000 + it, n)
            tq = rng.standard_normal((1, hq, n, D), np.float32)
            tk = rng.standard_normal((1, hkv, n, D), np.float32).astype(np.float16)
            tv = rng.standard_normal((1, hkv, n, D), np.float32).astype(np.float16)
            tqd, tkd, tvd = (torch.from_numpy(x).to(dev) for x in (tq, tk, tv))
            pd = torch.from_numpy(parents[None].copy()).to(dev)
            tout = torch.full((1, hq, n, D), float("nan"), device=dev)
            keep += [tqd, tkd, tvd, pd, tout]
            clen = int(page_case.seq_lens[0])
            c.attention_tree(tqd, kpool, vpool, tkd, tvd, pd, tout, hq, hkv, n, clen, D, scale, batch_size=1,
                             block_tables=tables[:1].contiguous(), max_blocks_per_seq=page_case.max_blocks,
                             num_blocks=page_case.num_blocks)
            c.sync()
            kr, _ = pyoracle.paged_gather(k_bits, np.where(page_case.tables[0] < 0, 0, page_case.tables[0]), clen, synth.PAGE)
            vr, _ = pyoracle.paged_gather(v_bits, np.where(page_case.tables[0] < 0, 0, page_case.tables[0]), clen, synth.PAGE)
            tref = pyoracle.attention_tree(np.ascontiguousarray(tq[0].transpose(1, 0, 2))[None], pyoracle.f16_bits_to_f32(kr),
                                           pyoracle.f16_bits_to_f32(vr),
                                           np.ascontiguousarray(tk[0].astype(np.float32).transpose(1, 0, 2))[None],
                                           np.ascontiguousarray(tv[0].astype(np.float32).transpose(1, 0, 2))[None], parents)
            assert_attention_close(tout.cpu().numpy()[0], tref[0].transpose(1, 0, 2), f"tree, iteration {it}")

            # paged decode: its two descriptors were cached at iteration 0 and must survive or be rebuilt
            if it % 10 == 0:
                dq = torch.from_numpy(page_case.q).to(dev)
                dout = torch.full((page_case.batch, hq, D), float("nan"), device=dev)
                keep += [dq, dout]
                c.batched_paged_attention_decode(dq, kpool, vpool, tables, lens, dout, page_case.batch, hq, hkv, D, synth.PAGE,
                                                 page_case.max_blocks, scale, num_blocks=page_case.num_blocks)
                c.sync()
                assert_attention_close(dout.cpu().numpy(), dec_ref, f"decode, iteration {it}")
        assert len(keep) > 300
    finally:
        c.shutdown()
