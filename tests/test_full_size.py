"""The paged-decode benchmark configurations at full size, through the C ABI.

The CPU checker evaluates a sample of the sequences; the rest of the batch is covered by properties
that do not depend on size: the result may not depend on where the pages physically lie (a permuted
pool with remapped tables gives the same bits), nor change from run to run.
"""
import numpy as np
import pytest

from conftest import assert_attention_close
from granite_b200 import synth

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _decode(compute, case, k_pool, v_pool, tables):
    import torch
    out = torch.full((case.batch, case.num_heads, case.head_dim), float("nan"), device=DEV)
    compute.batched_paged_attention_decode(case.q, k_pool, v_pool, tables, torch.from_numpy(case.seq_lens).to(DEV), out,
                                           case.batch, case.num_heads, case.num_kv_heads, case.head_dim, synth.PAGE,
                                           case.max_blocks, 1.0 / np.sqrt(case.head_dim), num_blocks=case.num_blocks)
    compute.sync()
    return out


def _oracle_rows(case, b):
    """CPU result of sequence b alone, from its own pages copied off the device."""
    import torch
    from oracle import pyoracle
    n = int(case.seq_lens[b])
    pages = torch.from_numpy(case.tables[b, :(n + synth.PAGE - 1) // synth.PAGE].astype(np.int64)).to(DEV)
    rows = (pages[:, None] * synth.PAGE + torch.arange(synth.PAGE, device=DEV)[None]).reshape(-1)
    k = case.k_pool[rows].cpu().numpy().view(np.uint16)
    v = case.v_pool[rows].cpu().numpy().view(np.uint16)
    table = np.arange(len(pages), dtype=np.int32)[None]
    ref, bad = pyoracle.paged_decode_batch(case.q[b:b + 1].cpu().numpy(), k, v, table, case.seq_lens[b:b + 1], synth.PAGE)
    assert bad == 0
    return ref[0]


def _check_config(compute, name, batch, sample):
    import torch
    cfg = dict(synth.CONFIGS[name])
    cfg["batch"] = batch
    case = synth.paged_case(cfg["seed"], cfg["batch"], cfg["len_lo"], cfg["len_hi"], cfg["num_heads"], cfg["num_kv_heads"],
                            cfg["head_dim"], dist=cfg["dist"], device=DEV)
    tables = torch.from_numpy(case.tables).to(DEV)
    out = _decode(compute, case, case.k_pool, case.v_pool, tables)
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    for b in sample:
        assert_attention_close(got[b], _oracle_rows(case, b), f"{name}, sequence {b} ({int(case.seq_lens[b])} tokens)")
    # same inputs, same bits
    assert torch.equal(out, _decode(compute, case, case.k_pool, case.v_pool, tables))
    # the pages move, the tables follow: same bits
    gen = torch.Generator(device=DEV)
    gen.manual_seed(99)
    perm = torch.randperm(case.num_blocks, device=DEV, generator=gen)
    shape = (case.num_blocks, synth.PAGE, case.num_kv_heads, case.head_dim)
    k2 = torch.empty_like(case.k_pool)
    v2 = torch.empty_like(case.v_pool)
    k2.view(shape)[perm] = case.k_pool.view(shape)
    v2.view(shape)[perm] = case.v_pool.view(shape)
    t2 = torch.where(tables >= 0, perm[tables.clamp(min=0).long()].int(), tables)
    assert torch.equal(out, _decode(compute, case, k2, v2, t2))


def test_paged_decode_benchmark_configuration(compute):
    """64 sequences, lengths uniform in [1024, 32768], Hq 32, Hkv 8: about 4.4 GB of K/V."""
    _check_config(compute, "paged_decode_b64", 64, sample=(0, 21, 42, 63))


def test_long_context_shard(compute):
    """One GPU's share of the sharded long-context configuration: 32 of the 256 sequences,
    log-uniform in [4096, 131072], Hq 64, Hkv 8 (about 4.8 GB); plus one sequence at the maximum length."""
    import torch
    _check_config(compute, "paged_decode_long_b256", 32, sample=(0, 17, 31))
    cfg = synth.CONFIGS["paged_decode_long_b256"]
    case = synth.paged_case(7, 2, 0, 0, cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"],
                            seq_lens=np.array([131072, 1], np.int32), device=DEV)
    out = _decode(compute, case, case.k_pool, case.v_pool, torch.from_numpy(case.tables).to(DEV)).cpu().numpy()
    for b in (0, 1):
        assert_attention_close(out[b], _oracle_rows(case, b), f"maximum length, sequence {b}")


def test_long_prefill_and_long_tree_prefix(compute):
    """Many K/V steps per work item (every ring slot and barrier phase wraps dozens of times): the last
    128 query rows of an 8192-token prefill against the CPU checker, and a tree over a 40 000-token
    paged prefix."""
    import torch
    from oracle import pyoracle
    import test_prefill as TP
    import test_tree_verify as TT
    hq, hkv, d, seq = 8, 2, 128, 8192
    q, k, v = TP._case(77, seq, seq, seq, hq, hkv)
    got = TP._run(compute, q, k, v, seq, 0, True, False)
    assert np.isfinite(got).all()
    tail = slice(seq - 128, seq)
    qq = q.astype(np.float16).astype(np.float32)[tail]
    ref = pyoracle.attention(qq[None], pyoracle.cache_to_fp32(k.view(np.uint16), seq), pyoracle.cache_to_fp32(v.view(np.uint16), seq),
                             start_pos=seq - 128)[0]
    assert_attention_close(got[tail], ref, "prefill 8192, last query block")
    assert_attention_close(got[0], np.repeat(v[:, 0].astype(np.float32), hq // hkv, axis=0), "row 0 equals V[0]")

    n, prefix = 64, 40000
    case = synth.paged_case(5, 1, 0, 0, hq, hkv, d, seq_lens=np.array([prefix], np.int32), device=DEV)
    qt, kt, vt, parents = TT._tree_inputs(6, 1, n, hq, hkv)
    out = torch.zeros((1, hq, n, d), device=DEV)
    compute.attention_tree(torch.from_numpy(qt).to(DEV), case.k_pool, case.v_pool, torch.from_numpy(kt).to(DEV),
                           torch.from_numpy(vt).to(DEV), torch.from_numpy(parents).to(DEV), out, hq, hkv, n, prefix, d,
                           1.0 / np.sqrt(d), batch_size=1, block_tables=torch.from_numpy(case.tables).to(DEV),
                           max_blocks_per_seq=case.max_blocks, num_blocks=case.num_blocks)
    compute.sync()
    rows = (torch.from_numpy(case.tables[0].astype(np.int64)).to(DEV)[:, None] * synth.PAGE
            + torch.arange(synth.PAGE, device=DEV)[None]).reshape(-1)[:prefix]
    kr = case.k_pool[rows].cpu().numpy().astype(np.float32)
    vr = case.v_pool[rows].cpu().numpy().astype(np.float32)
    ref = TT._oracle_one(qt[0], kr, vr, kt[0], vt[0], parents[0])
    assert_attention_close(out.cpu().numpy()[0], ref, "tree over a 40000-token prefix")
