"""Causal prefill attention (tcgen05/TMEM kernel) against the CPU checker, through the C ABI.

The reference path is MetalCompute::multihead_attention with seq_q > 1 (Q and output
[seq, Hq, D], K/V cache [Hkv, max_seq, D] fp16); correctness is defined by the CPU loop of
src/llm/transformer.mm:1779-1840 with the causal rule k_pos > start_pos + q_pos.
"""
import numpy as np
import pytest

from conftest import assert_attention_close

pytestmark = pytest.mark.gpu


def _case(seed, seq_q, seq_kv, max_seq, hq, hkv, d=128, poison=True):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((seq_q, hq, d), np.float32)
    k = rng.standard_normal((hkv, max_seq, d), np.float32).astype(np.float16)
    v = rng.standard_normal((hkv, max_seq, d), np.float32).astype(np.float16)
    if poison and max_seq > seq_kv:
        k.view(np.uint16)[:, seq_kv:] = 0x7E00  # stale rows of the cache: NaN
        v.view(np.uint16)[:, seq_kv:] = 0x7E00
    return q, k, v


def _run(compute, q, k, v, seq_kv, start_pos, q_fp16, out_fp16):
    import torch
    dev = "cuda:0"
    seq_q, hq, d = q.shape
    hkv, max_seq, _ = k.shape
    qd = torch.from_numpy(q.astype(np.float16) if q_fp16 else q).to(dev)
    out = torch.full((seq_q, hq, d), float("nan"), device=dev, dtype=torch.float16 if out_fp16 else torch.float32)
    compute.multihead_attention(qd, torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev), out, hq, hkv,
                                seq_q, seq_kv, d, 1.0 / np.sqrt(d), max_seq, q_dtype=int(q_fp16),
                                out_dtype=int(out_fp16), start_pos=start_pos)
    compute.sync()
    return out.float().cpu().numpy()


def _oracle(q, k, v, seq_kv, start_pos, q_fp16, heads=None):
    from oracle import pyoracle
    hq, hkv = q.shape[1], k.shape[0]
    qq = q.astype(np.float16).astype(np.float32) if q_fp16 else q
    kf = pyoracle.cache_to_fp32(k.view(np.uint16), seq_kv)
    vf = pyoracle.cache_to_fp32(v.view(np.uint16), seq_kv)
    if heads is not None:  # a slice of query heads that share KV head 0
        qq, kf, vf = qq[:, heads], kf[:, :1], vf[:, :1]
    return pyoracle.attention(qq[None], kf, vf, start_pos=start_pos)[0]


@pytest.mark.parametrize("seq,hq,hkv", [(128, 4, 1), (256, 8, 2), (300, 8, 2), (2, 4, 1), (77, 4, 2), (129, 2, 2),
                                        (200, 6, 2), (512, 32, 8)])
def test_prefill_matches_cpu_fp16_io(compute, seq, hq, hkv):
    q, k, v = _case(100 + seq, seq, seq, seq, hq, hkv)
    got = _run(compute, q, k, v, seq, 0, True, True)
    assert_attention_close(got, _oracle(q, k, v, seq, 0, True), f"prefill seq={seq} Hq={hq} Hkv={hkv}")


@pytest.mark.parametrize("q_fp16,out_fp16", [(False, False), (True, False), (False, True)])
def test_prefill_dtypes_and_stale_cache_rows(compute, q_fp16, out_fp16):
    """fp32 Q / fp32 output is the reference's own layout; rows past seq_kv hold NaN."""
    seq, max_seq = 333, 512
    q, k, v = _case(7, seq, seq, max_seq, 8, 2)
    got = _run(compute, q, k, v, seq, 0, q_fp16, out_fp16)
    assert_attention_close(got, _oracle(q, k, v, seq, 0, q_fp16), f"q_fp16={q_fp16} out_fp16={out_fp16}")


@pytest.mark.parametrize("seq_q,start_pos", [(100, 256), (128, 128), (37, 3), (256, 1000)])
def test_chunked_prefill_start_pos(compute, seq_q, start_pos):
    """start_pos = chunk_start, seq_kv = chunk_start + chunk_len (src/llm/transformer.mm:3682-3692)."""
    seq_kv = start_pos + seq_q
    q, k, v = _case(9 + seq_q, seq_q, seq_kv, seq_kv + 64, 8, 2)
    got = _run(compute, q, k, v, seq_kv, start_pos, False, False)
    assert_attention_close(got, _oracle(q, k, v, seq_kv, start_pos, False), f"chunk {seq_q}@{start_pos}")


def test_prefill_full_config_slice(compute):
    """The benchmark configuration (seq 2048, Hq 32, Hkv 8, D 128, fp16 in/out); the CPU checker
    evaluates the four query heads of KV head 0 and the four of KV head 7."""
    seq, hq, hkv = 2048, 32, 8
    q, k, v = _case(1002, seq, seq, seq, hq, hkv)
    got = _run(compute, q, k, v, seq, 0, True, True)
    assert np.isfinite(got).all()
    ref0 = _oracle(q, k, v, seq, 0, True, heads=slice(0, 4))
    assert_attention_close(got[:, 0:4], ref0, "config slice, KV head 0")
    from oracle import pyoracle
    kf = pyoracle.cache_to_fp32(k.view(np.uint16)[7:8], seq)
    vf = pyoracle.cache_to_fp32(v.view(np.uint16)[7:8], seq)
    ref7 = pyoracle.attention(q.astype(np.float16).astype(np.float32)[None, :, 28:32], kf, vf, start_pos=0)[0]
    assert_attention_close(got[:, 28:32], ref7, "config slice, KV head 7")
    # causality as a size-independent property: the first row attends to key 0 only
    assert_attention_close(got[0], np.repeat(v[:, 0].astype(np.float32), hq // hkv, axis=0), "row 0 equals V[0]")


@pytest.mark.parametrize("batch,seq_q,seq_kv,max_seq,start_pos,q_fp16", [(3, 200, 200, 200, 0, True), (2, 128, 300, 384, 172, False),
                                                                       (5, 1, 77, 128, 0, False)])
def test_batched_sequences(compute, batch, seq_q, seq_kv, max_seq, start_pos, q_fp16):
    """A leading batch dimension on every buffer (beyond the reference, which takes one sequence per
    call): every sequence must come out as if it had been run alone.  seq_q == 1 is the decode path."""
    import torch
    dev = "cuda:0"
    hq, hkv, d = 8, 2, 128
    cases = [_case(40 + b, seq_q, seq_kv, max_seq, hq, hkv) for b in range(batch)]
    q = np.stack([c[0] for c in cases])
    k = np.stack([c[1] for c in cases])
    v = np.stack([c[2] for c in cases])
    decode = seq_q == 1
    qd = torch.from_numpy(q.astype(np.float16) if q_fp16 else q).to(dev)
    out = torch.full((batch, seq_q, hq, d), float("nan"), device=dev)
    compute.multihead_attention(qd, torch.from_numpy(k).to(dev), torch.from_numpy(v).to(dev), out, hq, hkv, seq_q, seq_kv,
                                d, 1.0 / np.sqrt(d), max_seq, q_dtype=int(q_fp16), out_dtype=0,
                                start_pos=0 if decode else start_pos, batch_size=batch)
    compute.sync()
    got = out.cpu().numpy()
    for b in range(batch):
        ref = _oracle(q[b], k[b], v[b], seq_kv, seq_kv - 1 if decode else start_pos, q_fp16)
        assert_attention_close(got[b], ref, f"sequence {b} of {batch}")
