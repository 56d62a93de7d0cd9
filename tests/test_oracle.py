"""Pins the CPU checker (oracle/) before anything trusts it: against the reference's own
compiled objects and its own attention statements (golden files written by
tests/golden/make_golden.py, and live against oracle/_ref when that library is present), and
against the one attention known-answer test the reference holds (tests/test_vulkan.cpp:353-482)."""
from pathlib import Path

import numpy as np
import pytest

from oracle import pyoracle
from granite_b200 import synth

GOLD = Path(__file__).resolve().parent / "golden"


def test_fp16_widening_matches_reference_for_every_code():
    g = np.load(GOLD / "ref_fp16.npz")
    mine = pyoracle.f16_bits_to_f32(np.arange(65536, dtype=np.uint16)).view(np.uint32)
    assert np.array_equal(mine, g["widened_bits"])


def test_fp16_truncating_narrowing_matches_reference():
    g = np.load(GOLD / "ref_fp16.npz")
    floats = g["floats"].view(np.float32)
    mine = np.array([pyoracle.fp32_to_fp16(float(f)) for f in floats], np.uint16)
    assert np.array_equal(mine, g["narrowed"])
    # truncation, not rounding: 0.33337402 sits just below the next fp16 step
    assert pyoracle.fp32_to_fp16(0.3333740234375 - 1e-7) == pyoracle.fp32_to_fp16(0.333251953125)
    # flush of subnormal results and clamp to infinity (math_ops.cpp:51-52)
    assert pyoracle.fp32_to_fp16(5.9e-8) == 0
    assert pyoracle.fp32_to_fp16(70000.0) == 0x7C00
    assert pyoracle.fp32_to_fp16(float("nan")) == 0x7C00


def test_known_answer_2x3x4():
    g = np.load(GOLD / "kat_sdpa_2x3x4.npz")
    got = pyoracle.sdpa_kt(g["q"], g["kt"], g["v"], float(g["scale"][0]))
    assert np.abs(got - g["expected"]).max() <= 1e-4  # the reference test's own bound
    # the LLM-path loop gives the same numbers on the same problem (K given row-major)
    k = np.ascontiguousarray(g["kt"].T)[:, None, :]
    v = g["v"][:, None, :]
    q = g["q"][None, :, None, :]
    got2 = pyoracle.attention(q, k, v, start_pos=10, scale=float(g["scale"][0]), threads=1)[0, :, 0, :]
    assert np.abs(got2 - g["expected"]).max() <= 1e-4


def _loop_cases(g, suffix="_cfg"):
    names = [k[: -len(suffix)] for k in g.files if k.endswith(suffix)]
    return [n for n in names if not n.startswith(("widen", "mask"))]


def test_attention_loop_is_bit_identical_to_the_reference_statements():
    """The restated loops against outputs of the reference's own statements (transformer.mm:1779-1840,
    compiled from the checkout by oracle/ref_loops.cpp): causal masks with start_pos 0 and > 0, GQA 4:1
    and 8:1, a batch of two, head_dim 128.  Bit for bit, with one thread and with several."""
    g = np.load(GOLD / "ref_attention_loops.npz")
    cases = [n for n in _loop_cases(g) if f"{n}_k16" in g.files]
    assert len(cases) >= 5
    for name in cases:
        b, sq, t, start, hq, hkv, d = (int(x) for x in g[f"{name}_cfg"])
        k = pyoracle.f16_bits_to_f32(g[f"{name}_k16"])
        v = pyoracle.f16_bits_to_f32(g[f"{name}_v16"])
        for threads in (1, 3):
            got = pyoracle.attention(g[f"{name}_q"], k, v, start_pos=start, scale=float(g[f"{name}_scale"][0]), threads=threads)
            assert np.array_equal(got.view(np.uint32), g[f"{name}_out"]), name
        # scale 0 means 1/sqrt(head_dim) computed the reference's way (transformer.mm:1705)
        got = pyoracle.attention(g[f"{name}_q"], k, v, start_pos=start, threads=2)
        assert np.array_equal(got.view(np.uint32), g[f"{name}_out"]), name


def test_cache_widening_is_bit_identical_to_the_reference_statements():
    g = np.load(GOLD / "ref_attention_loops.npz")
    hkv, max_seq, d, total = (int(x) for x in g["widen_cfg"])
    assert np.array_equal(pyoracle.cache_to_fp32(g["widen_ck"], total).view(np.uint32), g["widen_k"])
    assert np.array_equal(pyoracle.cache_to_fp32(g["widen_cv"], total).view(np.uint32), g["widen_v"])


def test_tree_attention_and_mask_are_bit_identical_to_the_reference_statements():
    """transformer.mm:2044-2126 with the mask of :822-841: a 64-node tree over a 100-token prefix (GQA 4:1),
    a tree without a prefix, a batch of two with GQA 8:1."""
    g = np.load(GOLD / "ref_attention_loops.npz")
    cases = [n for n in _loop_cases(g) if f"{n}_parents" in g.files]
    assert len(cases) >= 3
    for name in cases:
        b, n, prefix, hq, hkv, d = (int(x) for x in g[f"{name}_cfg"])
        parents = g[f"{name}_parents"]
        mask = pyoracle.tree_mask(parents)
        assert np.array_equal(np.packbits(mask, axis=1), g[f"{name}_mask"]), name
        kp = pyoracle.f16_bits_to_f32(g[f"{name}_kp16"])
        vp = pyoracle.f16_bits_to_f32(g[f"{name}_vp16"])
        for threads in (1, 3):
            got = pyoracle.attention_tree(g[f"{name}_q"], kp, vp, g[f"{name}_kt"], g[f"{name}_vt"], parents,
                                          scale=float(g[f"{name}_scale"][0]), threads=threads)
            assert np.array_equal(got.view(np.uint32), g[f"{name}_out"]), name
    for i in range(4):
        assert np.array_equal(np.packbits(pyoracle.tree_mask(g[f"mask{i}_parents"]), axis=1), g[f"mask{i}"])


@pytest.mark.skipif(not pyoracle.ref_available(), reason="oracle/_ref not built (needs the reference checkout)")
def test_live_reference_statements_agree_on_fresh_seeded_cases():
    """Where the compiled reference statements are present: fresh random shapes, bit for bit."""
    ref = pyoracle.Ref()
    rng = np.random.default_rng(1779)
    for _ in range(12):
        hkv = int(rng.choice([1, 2, 3, 4]))
        hq = hkv * int(rng.choice([1, 2, 4, 8]))
        d = int(rng.choice([8, 32, 64, 128]))
        sq = int(rng.integers(1, 20))
        past = int(rng.integers(0, 60))
        extra = int(rng.integers(0, 3))  # keys cached beyond the last query's position
        t = past + sq + extra
        q = rng.standard_normal((1, sq, hq, d), dtype=np.float32)
        k = rng.standard_normal((t, hkv, d), dtype=np.float32).astype(np.float16).astype(np.float32)
        v = rng.standard_normal((t, hkv, d), dtype=np.float32).astype(np.float16).astype(np.float32)
        scale = float(np.float32(1.0) / np.sqrt(np.float32(d)))
        want = ref.attention_loop(q, k, v, past, scale)
        assert np.array_equal(pyoracle.attention(q, k, v, start_pos=past, scale=scale).view(np.uint32), want.view(np.uint32))
        n = int(rng.integers(1, 65))
        parents = synth.tree_parents(int(rng.integers(0, 1 << 30)), n)
        tq = rng.standard_normal((1, n, hq, d), dtype=np.float32)
        kt = rng.standard_normal((1, n, hkv, d), dtype=np.float32)
        vt = rng.standard_normal((1, n, hkv, d), dtype=np.float32)
        want = ref.attention_tree_loop(tq, k, v, kt, vt, parents, scale)
        got = pyoracle.attention_tree(tq, k, v, kt, vt, parents, scale=scale)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        assert np.array_equal(pyoracle.tree_mask(parents), ref.tree_mask(parents))
    # the paged decode of the checker is the same loop over rows gathered through the table
    case = synth.paged_case(seed=5, batch=3, len_lo=1, len_hi=200, num_heads=8, num_kv_heads=2, head_dim=64)
    tables = np.where(case.tables < 0, 0, case.tables)
    got, bad = pyoracle.paged_decode_batch(case.q, case.k_pool.view(np.uint16), case.v_pool.view(np.uint16), tables,
                                           case.seq_lens, synth.PAGE)
    assert bad == 0
    for b in range(case.batch):
        n = int(case.seq_lens[b])
        kr, _ = pyoracle.paged_gather(case.k_pool.view(np.uint16), tables[b], n, synth.PAGE)
        vr, _ = pyoracle.paged_gather(case.v_pool.view(np.uint16), tables[b], n, synth.PAGE)
        want = ref.attention_loop(case.q[b][None, None], pyoracle.f16_bits_to_f32(kr), pyoracle.f16_bits_to_f32(vr), n - 1,
                                  float(np.float32(1.0) / np.sqrt(np.float32(64))))
        assert np.array_equal(got[b].view(np.uint32), want[0, 0].view(np.uint32))


def test_oracle_small_cases_are_stable():
    g = np.load(GOLD / "oracle_small_cases.npz")
    seq = int(g["dec_seq"][0])
    k_all = pyoracle.cache_to_fp32(g["dec_k"], seq)
    v_all = pyoracle.cache_to_fp32(g["dec_v"], seq)
    for threads in (1, 4):
        assert np.array_equal(pyoracle.attention(g["dec_q"], k_all, v_all, start_pos=seq - 1, threads=threads), g["dec_out"])
        assert np.array_equal(pyoracle.attention(g["pre_q"], g["pre_k"], g["pre_v"], start_pos=0, threads=threads), g["pre_out"])
        assert np.array_equal(pyoracle.attention_tree(g["tree_q"], g["tree_kp"], g["tree_vp"], g["tree_kt"], g["tree_vt"],
                                                      g["tree_parents"], threads=threads), g["tree_out"])
    assert np.array_equal(pyoracle.tree_mask(g["tree_parents"]), g["tree_mask"])


def test_attention_against_float64_softmax():
    rng = np.random.default_rng(3)
    s, hq, hkv, d = 23, 4, 2, 32
    q = rng.standard_normal((1, s, hq, d)).astype(np.float32)
    k = rng.standard_normal((s, hkv, d)).astype(np.float32)
    v = rng.standard_normal((s, hkv, d)).astype(np.float32)
    got = pyoracle.attention(q, k, v, start_pos=0)
    for h in range(hq):
        sc = (q[0, :, h].astype(np.float64) @ k[:, h // 2].astype(np.float64).T) / np.sqrt(d)
        sc[np.triu_indices(s, 1)] = -np.inf
        p = np.exp(sc - sc.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        assert np.abs(p @ v[:, h // 2].astype(np.float64) - got[0, :, h]).max() < 1e-5


def test_causal_rule_uses_start_pos():
    """k_pos > start_pos + q_pos is masked (transformer.mm:1805-1806)."""
    rng = np.random.default_rng(4)
    q = rng.standard_normal((1, 2, 2, 8)).astype(np.float32)
    k = rng.standard_normal((6, 1, 8)).astype(np.float32)
    v = rng.standard_normal((6, 1, 8)).astype(np.float32)
    got = pyoracle.attention(q, k, v, start_pos=3)
    # query 0 sees keys 0..3, query 1 sees 0..4
    a = pyoracle.attention(q[:, :1], k[:4], v[:4], start_pos=3)
    b = pyoracle.attention(q[:, 1:], k[:5], v[:5], start_pos=4)
    assert np.array_equal(got[:, :1], a) and np.array_equal(got[:, 1:], b)


def test_paged_gather_follows_addressing_rule():
    case = synth.paged_case(seed=21, batch=3, len_lo=1, len_hi=90, num_heads=4, num_kv_heads=2, head_dim=8)
    pool = case.k_pool.view(np.uint16)
    for b in range(case.batch):
        n = int(case.seq_lens[b])
        rows, bad = pyoracle.paged_gather(pool, case.tables[b], n, synth.PAGE)
        assert bad == 0
        for pos in (0, n // 2, n - 1):
            phys = case.tables[b, pos // 16] * 16 + pos % 16  # metal_compute.h:857-861
            assert np.array_equal(rows[pos], pool[phys])
    _, bad = pyoracle.paged_gather(pool, np.array([case.num_blocks], np.int32), 3, synth.PAGE)
    assert bad == 3


def test_tree_mask_matches_definition_and_reference_tree():
    g = np.load(GOLD / "ref_spec_tree.npz")
    for i in range(4):
        parents = g[f"parents{i}"]
        assert np.array_equal(g[f"parents_out{i}"], parents)  # get_parent_indices keeps insertion order
        m = pyoracle.tree_mask(parents)
        depths = g[f"depths{i}"]
        n = len(parents)
        for a in range(n):
            anc = {a}
            c = parents[a]
            while c >= 0:
                anc.add(int(c))
                c = parents[c]
            assert set(np.flatnonzero(m[a])) == anc
            assert m[a].sum() == depths[a] + 1  # self + one ancestor per level
        assert pyoracle.tree_validate(parents)
    assert not pyoracle.tree_validate(np.array([-1, 2, 7], np.int32))
    assert not pyoracle.tree_validate(np.array([-2], np.int32))


def test_synthetic_tree_respects_limits():
    p = synth.tree_parents(1004, 64, max_children=4, max_depth=8)
    assert p[0] == -1 and (p[1:] < np.arange(1, 64)).all() and (p[1:] >= 0).all()
    assert np.bincount(p[1:], minlength=64).max() <= 4
    assert pyoracle.tree_mask(p).sum(1).max() - 1 <= 8


def test_rope_tables_and_rotation_match_reference():
    """RoPECache::initialize / apply of the compiled reference (src/llm/rope.cpp:5-92), bit for bit."""
    g = np.load(GOLD / "ref_rope.npz")
    for i in range(3):
        max_seq, d = (int(x) for x in g[f"t{i}_cfg"])
        cos, sin = pyoracle.rope_table(max_seq, d, float(g[f"t{i}_theta"][0]))
        rows = g[f"t{i}_rows"] if f"t{i}_rows" in g else np.arange(max_seq)
        assert np.array_equal(cos[rows].view(np.uint32), g[f"t{i}_cos"])
        assert np.array_equal(sin[rows].view(np.uint32), g[f"t{i}_sin"])
    for i in range(2):
        seq, hq, hk, d, start, max_seq = (int(x) for x in g[f"a{i}_cfg"])
        cos, sin = pyoracle.rope_table(max_seq, d)
        q = g[f"a{i}_q"].view(np.float32)
        k = g[f"a{i}_k"].view(np.float32)
        assert np.array_equal(pyoracle.rope_apply(q, start, cos, sin).view(np.uint32), g[f"a{i}_q_out"])
        assert np.array_equal(pyoracle.rope_apply(k, start, cos, sin).view(np.uint32), g[f"a{i}_k_out"])
    assert int(g["range_error_code"][0]) == 16  # InvalidArgument, rope.cpp:34-38
    with pytest.raises(ValueError):
        pyoracle.rope_apply(np.zeros((3, 1, 16), np.float32), 46, *pyoracle.rope_table(48, 16))


def test_rope_paged_append_is_rotation_then_truncation_then_scatter():
    rng = np.random.default_rng(5)
    batch, new_len, hq, hkv, d, bs, nblocks, max_blocks = 3, 2, 4, 2, 16, 4, 12, 4
    cos, sin = pyoracle.rope_table(16, d)
    q = rng.standard_normal((batch, new_len, hq, d), dtype=np.float32)
    k = rng.standard_normal((batch, new_len, hkv, d), dtype=np.float32)
    v = rng.standard_normal((batch, new_len, hkv, d), dtype=np.float32)
    tables = rng.permutation(nblocks).astype(np.int32).reshape(batch, max_blocks)
    positions = np.array([0, 3, 9], np.int32)
    kp = np.zeros((nblocks * bs, hkv, d), np.uint16)
    vp = np.zeros_like(kp)
    qr, bad = pyoracle.rope_paged_append(q, k, v, cos, sin, kp, vp, tables, positions, bs)
    assert bad == 0
    written = np.zeros(nblocks * bs, bool)
    for b in range(batch):
        for s in range(new_len):
            pos = int(positions[b]) + s
            row = tables[b, pos // bs] * bs + pos % bs
            written[row] = True
            kr = pyoracle.rope_apply(k[b, s:s + 1], pos, cos, sin)[0]
            assert np.array_equal(qr[b, s], pyoracle.rope_apply(q[b, s:s + 1], pos, cos, sin)[0])
            assert [pyoracle.fp32_to_fp16(float(x)) for x in kr.reshape(-1)] == kp[row].reshape(-1).tolist()
            assert [pyoracle.fp32_to_fp16(float(x)) for x in v[b, s].reshape(-1)] == vp[row].reshape(-1).tolist()
    assert not kp[~written].any() and not vp[~written].any()
    # a position outside the table, or a table entry outside the pool, skips the token and is counted
    tables_bad = tables.copy()
    tables_bad[1, 0] = nblocks
    _, bad = pyoracle.rope_paged_append(q, k, v, cos, sin, kp, vp, tables_bad, np.array([0, 3, 15], np.int32), bs)
    assert bad == 1 + 1  # sequence 1's first token (bad entry), sequence 2's second token (position 16)


@pytest.mark.skipif(not pyoracle.ref_available(), reason="oracle/_ref not built (needs the reference checkout)")
def test_live_reference_objects_agree_with_goldens():
    ref = pyoracle.Ref()
    g = np.load(GOLD / "ref_paged_pool.npz")
    for i in range(3):
        ms, mt, bs, mb = (int(x) for x in g[f"cfg{i}"])
        r = ref.paged_pool_script(ms, mt, bs, g[f"ops{i}"], mb)
        assert np.array_equal(r["results"], g[f"results{i}"])
        assert np.array_equal(r["tables"], g[f"tables{i}"])
    for h in (0, 1, 0x3FF, 0x400, 0x7BFF, 0x7C00, 0x7E00, 0x8001, 0xFC00):
        assert np.float32(ref.fp16_to_fp32(h)).tobytes() == np.float32(pyoracle.fp16_to_fp32(h)).tobytes()
