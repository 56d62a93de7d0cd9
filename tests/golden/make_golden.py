"""Regenerates the golden fixtures in this directory.  Run where the reference checkout exists:

    python tests/golden/make_golden.py

Sources of truth, per file:
  ref_fp16.npz            reference fp16_to_fp32 / fp32_to_fp16 (src/llm/math_ops.cpp:18-54) through
                          oracle/_ref (the reference's own compiled sources)
  ref_paged_pool.npz      reference PagedKVPool / PagedKVCache / BlockManager replaying a seeded
                          script of operations (src/llm/paged_kv_cache.cpp)
  ref_kvcache_append.npz  reference KVCache::append layout (src/llm/kv_cache.cpp:52-107)
  ref_spec_tree.npz       reference SpeculationTree parents / depths / BFS order
                          (src/llm/speculation_tree.cpp:13-84)
  ref_attention_loops.npz the reference's OWN attention statements - the blocks of src/llm/transformer.mm
                          at :1779-1840 (attention), :1753-1765 (cache widening), :2044-2126 (tree
                          attention) and :822-841 (tree mask), cut out of the checkout at build time
                          and compiled into oracle/_ref (oracle/ref_loops.cpp) - run on seeded inputs
                          with causal masks (start_pos 0 and > 0), GQA 4:1 and 8:1, a batch of two and
                          a 64-node tree over a prefix.  Inputs and outputs are both stored.
  kat_sdpa_2x3x4.npz      the one attention known-answer test the reference holds
                          (tests/test_vulkan.cpp:353-482): inputs and expected values recomputed
                          here in numpy float32 in the test's own order, independently of oracle/
  oracle_small_cases.npz  small seeded decode / causal prefill / tree cases evaluated by oracle/
                          (guards the checker itself against drift; not a reference output)
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from oracle import pyoracle  # noqa: E402
from granite_b200 import synth  # noqa: E402


def ref_fp16(ref):
    codes = np.arange(65536, dtype=np.uint16)
    widened = ref.fp16_to_fp32_bits(codes)
    rng = np.random.default_rng(42)
    floats = np.concatenate([
        rng.standard_normal(4000).astype(np.float32),
        (rng.standard_normal(2000) * 1e-6).astype(np.float32),
        (rng.standard_normal(2000) * 1e5).astype(np.float32),
        np.array([0.0, -0.0, 1.0, -1.0, 65504.0, 65520.0, 1e-8, 6.1e-5, 5.9e-8, np.inf, -np.inf, np.nan,
                  0.333251953125, 0.3333740234375], np.float32),
    ])
    narrowed = np.array([ref.fp32_to_fp16(float(f)) for f in floats], np.uint16)
    np.savez_compressed(HERE / "ref_fp16.npz", widened_bits=widened, floats=floats.view(np.uint32), narrowed=narrowed)


def paged_script(seed, n_ops, max_sequences, max_total_tokens, block_size):
    """A seeded walk over the page-manager operations, biased towards exhaustion and reuse."""
    rng = np.random.default_rng(seed)
    ops = []
    live = []
    for _ in range(n_ops):
        r = rng.random()
        if r < 0.15 or not live:
            ops.append((0, 0, 0))
            live.append(len(live))  # optimistic; replays are deterministic anyway
        elif r < 0.60:
            ops.append((1, int(rng.integers(0, max_sequences)), int(rng.integers(1, 3 * block_size))))
        elif r < 0.75:
            ops.append((2, int(rng.integers(0, max_sequences)), int(rng.integers(0, 4 * block_size))))
        elif r < 0.85:
            ops.append((3, int(rng.integers(-1, max_sequences + 1)), 0))
        elif r < 0.90:
            ops.append((4, 0, 0))
        elif r < 0.95:
            ops.append((5, int(rng.integers(-2, max_total_tokens // block_size + 2)), 0))
        else:
            ops.append((6 if rng.random() < 0.5 else 7, int(rng.integers(0, max_sequences)), int(rng.integers(0, 5 * block_size))))
    return np.array(ops, np.int32)


def ref_paged_pool(ref):
    out = {}
    for i, (seed, n_ops, ms, mt, bs) in enumerate([(1, 400, 4, 256, 16), (2, 600, 8, 100, 16), (3, 300, 3, 64, 4)]):
        ops = paged_script(seed, n_ops, ms, mt, bs)
        max_blocks = (mt + bs - 1) // bs
        r = ref.paged_pool_script(ms, mt, bs, ops, max_blocks)
        out[f"cfg{i}"] = np.array([ms, mt, bs, max_blocks], np.int32)
        out[f"ops{i}"] = ops
        for k in ("results", "seq_lens", "table_lens", "tables"):
            out[f"{k}{i}"] = r[k]
        out[f"free{i}"] = np.array([r["num_free"], r["num_total"]], np.int32)
    np.savez_compressed(HERE / "ref_paged_pool.npz", **out)


def ref_kvcache(ref):
    rng = np.random.default_rng(7)
    hkv, d, max_seq = 3, 8, 20
    steps = np.array([5, 1, 1, 7, 2], np.int32)
    ks = [rng.integers(0, 65536, size=(hkv, int(n), d)).astype(np.uint16) for n in steps]
    vs = [rng.integers(0, 65536, size=(hkv, int(n), d)).astype(np.uint16) for n in steps]
    k_out, v_out, final_len = ref.kvcache_append(hkv, d, max_seq, steps,
                                                 np.concatenate([k.reshape(-1) for k in ks]),
                                                 np.concatenate([v.reshape(-1) for v in vs]))
    np.savez_compressed(HERE / "ref_kvcache_append.npz", shape=np.array([hkv, d, max_seq], np.int32), steps=steps,
                        k_chunks=np.concatenate([k.reshape(-1) for k in ks]),
                        v_chunks=np.concatenate([v.reshape(-1) for v in vs]),
                        k_out=k_out, v_out=v_out, final_len=np.array([final_len], np.int32))


def ref_rope(ref):
    """RoPECache tables and apply() outputs from the compiled reference (src/llm/rope.cpp)."""
    rng = np.random.default_rng(19)
    out = {}
    # table samples: full small table, and rows of the large ones (first, odd, last positions)
    cos, sin = ref.rope_table(48, 16, 10000.0)
    out["t0_cfg"] = np.array([48, 16], np.int32)
    out["t0_theta"] = np.array([10000.0], np.float32)
    out["t0_cos"], out["t0_sin"] = cos.view(np.uint32), sin.view(np.uint32)
    for i, (max_seq, d, theta) in enumerate([(4096, 128, 10000.0), (2048, 64, 500000.0)], start=1):
        cos, sin = ref.rope_table(max_seq, d, theta)
        rows = np.array([0, 1, 2, 3, 17, 255, 1000, max_seq - 1], np.int32)
        out[f"t{i}_cfg"] = np.array([max_seq, d], np.int32)
        out[f"t{i}_theta"] = np.array([theta], np.float32)
        out[f"t{i}_rows"] = rows
        out[f"t{i}_cos"], out[f"t{i}_sin"] = cos[rows].view(np.uint32), sin[rows].view(np.uint32)
    # apply(): q [seq, Hq, D], k [seq, Hk, D] at a start position
    for i, (seq, hq, hk, d, start, max_seq) in enumerate([(3, 4, 2, 16, 5, 48), (2, 32, 8, 128, 4000, 4096)]):
        q = rng.standard_normal((seq, hq, d), dtype=np.float32)
        k = rng.standard_normal((seq, hk, d), dtype=np.float32)
        qr, kr, rc = ref.rope_apply(q, k, start, max_seq)
        assert rc == 0
        out[f"a{i}_cfg"] = np.array([seq, hq, hk, d, start, max_seq], np.int32)
        out[f"a{i}_q"], out[f"a{i}_k"] = q.view(np.uint32), k.view(np.uint32)
        out[f"a{i}_q_out"], out[f"a{i}_k_out"] = qr.view(np.uint32), kr.view(np.uint32)
    out["range_error_code"] = np.array([ref.rope_apply(np.zeros((3, 1, 16), np.float32), np.zeros((3, 1, 16), np.float32), 46, 48)[2]], np.int32)
    np.savez_compressed(HERE / "ref_rope.npz", **out)


def ref_spec_tree(ref):
    out = {}
    for i, (seed, n) in enumerate([(1004, 64), (5, 16), (6, 1), (8, 33)]):
        parents = synth.tree_parents(seed, n)
        r = ref.speculation_tree(parents)
        out[f"parents{i}"] = parents
        out[f"parents_out{i}"] = r["parents"]
        out[f"depths{i}"] = r["depths"]
        out[f"bfs{i}"] = r["bfs"]
        out[f"max_depth{i}"] = np.array([r["max_depth"]], np.int32)
    # accepted-path search (speculation_tree.cpp:85-143) on small-vocabulary trees
    rng = np.random.default_rng(11)
    for i in range(6):
        n = int(rng.integers(1, 40))
        parents = synth.tree_parents(200 + i, n)
        tokens = rng.integers(0, 4, size=n).astype(np.int32)
        targets = rng.integers(0, 4, size=int(rng.integers(1, 10))).astype(np.int32)
        targets[0] = tokens[0] if i % 3 else targets[0]
        out[f"ap_parents{i}"] = parents
        out[f"ap_tokens{i}"] = tokens
        out[f"ap_targets{i}"] = targets
        out[f"ap_path{i}"] = ref.find_accepted_path(parents, tokens, targets)
    np.savez_compressed(HERE / "ref_spec_tree.npz", **out)


# (name, batch, seq_q, total_seq, start_pos, Hq, Hkv, D): what TransformerModel::attention is asked for
ATTENTION_LOOP_CASES = [
    ("prefill_gqa4", 1, 33, 33, 0, 8, 2, 32),          # causal from position 0, GQA 4:1
    ("chunk_gqa8", 1, 5, 29, 24, 8, 1, 16),            # start_pos > 0, GQA 8:1: query i sees keys <= 24 + i
    ("decode_d128", 1, 1, 77, 76, 8, 2, 128),          # one query token over a cache, head_dim 128
    ("batch2_mha", 2, 3, 7, 4, 4, 4, 8),               # batch index in the query/context addressing
    ("future_keys", 1, 2, 12, 3, 4, 2, 16),            # keys past start_pos + q stay masked although cached
]
# (name, batch, N nodes, prefix, Hq, Hkv, D, tree seed)
TREE_LOOP_CASES = [
    ("tree64_prefix100", 1, 64, 100, 8, 2, 32, 1004),  # the benchmark's tree shape over a prefix
    ("tree16_no_prefix", 1, 16, 0, 4, 4, 16, 5),
    ("tree33_gqa8_batch2", 2, 33, 9, 8, 1, 16, 8),
]


def ref_attention_loops(ref):
    """Inputs are drawn like the cache holds them: K/V values that are exact in fp16 (stored as fp16
    bits), fp32 queries; tree K/V are fp32 as the reference computes them (transformer.mm:1950-1975)."""
    rng = np.random.default_rng(2044)
    out = {}
    for name, b, sq, t, start, hq, hkv, d in ATTENTION_LOOP_CASES:
        q = rng.standard_normal((b, sq, hq, d), dtype=np.float32)
        k16 = rng.standard_normal((t, hkv, d), dtype=np.float32).astype(np.float16)
        v16 = rng.standard_normal((t, hkv, d), dtype=np.float32).astype(np.float16)
        scale = np.float32(1.0) / np.sqrt(np.float32(d))
        ctx = ref.attention_loop(q, k16.astype(np.float32), v16.astype(np.float32), start, float(scale))
        out[f"{name}_cfg"] = np.array([b, sq, t, start, hq, hkv, d], np.int32)
        out[f"{name}_scale"] = np.array([scale], np.float32)
        out[f"{name}_q"], out[f"{name}_k16"], out[f"{name}_v16"] = q, k16.view(np.uint16), v16.view(np.uint16)
        out[f"{name}_out"] = ctx.view(np.uint32)
    # the widening of a cache that is longer than the live length
    hkv, max_seq, d, total = 3, 40, 16, 27
    ck = rng.integers(0, 65536, size=(hkv, max_seq, d)).astype(np.uint16)
    cv = rng.integers(0, 65536, size=(hkv, max_seq, d)).astype(np.uint16)
    kw, vw = ref.attention_cache_widen(ck, cv, total)
    out.update(widen_cfg=np.array([hkv, max_seq, d, total], np.int32), widen_ck=ck, widen_cv=cv,
               widen_k=kw.view(np.uint32), widen_v=vw.view(np.uint32))
    for name, b, n, prefix, hq, hkv, d, seed in TREE_LOOP_CASES:
        parents = synth.tree_parents(seed, n)
        q = rng.standard_normal((b, n, hq, d), dtype=np.float32)
        kp16 = rng.standard_normal((prefix, hkv, d), dtype=np.float32).astype(np.float16)
        vp16 = rng.standard_normal((prefix, hkv, d), dtype=np.float32).astype(np.float16)
        kt = rng.standard_normal((b, n, hkv, d), dtype=np.float32)
        vt = rng.standard_normal((b, n, hkv, d), dtype=np.float32)
        scale = np.float32(1.0) / np.sqrt(np.float32(d))
        ctx = ref.attention_tree_loop(q, kp16.astype(np.float32), vp16.astype(np.float32), kt, vt, parents, float(scale))
        out[f"{name}_cfg"] = np.array([b, n, prefix, hq, hkv, d], np.int32)
        out[f"{name}_scale"] = np.array([scale], np.float32)
        out[f"{name}_parents"] = parents
        out[f"{name}_q"], out[f"{name}_kp16"], out[f"{name}_vp16"] = q, kp16.view(np.uint16), vp16.view(np.uint16)
        out[f"{name}_kt"], out[f"{name}_vt"] = kt, vt
        out[f"{name}_mask"] = np.packbits(ref.tree_mask(parents), axis=1)
        out[f"{name}_out"] = ctx.view(np.uint32)
    # masks alone: a chain, a star, several roots, one node
    for i, parents in enumerate([np.arange(-1, 19), np.array([-1] + [0] * 11), np.array([-1, -1, 0, 1, 2, 3, -1, 6]),
                                 np.array([-1])]):
        parents = parents.astype(np.int32)
        out[f"mask{i}_parents"] = parents
        out[f"mask{i}"] = np.packbits(ref.tree_mask(parents), axis=1)
    np.savez_compressed(HERE / "ref_attention_loops.npz", **out)


def kat_sdpa():
    """tests/test_vulkan.cpp:366-474, recomputed in the test's own order with float32 steps."""
    f = np.float32
    sq, skv, d = 2, 3, 4
    q = np.array([f(i + 1) for i in range(sq * d)], f).reshape(sq, d)
    kt = np.array([f(i + 1) * f(0.5) for i in range(d * skv)], f).reshape(d, skv)
    v = np.array([f(i + 1) * f(0.25) for i in range(skv * d)], f).reshape(skv, d)
    scale = 1.0 / np.sqrt(float(d))
    expected = np.zeros((sq, d), f)
    for i in range(sq):
        scores = np.zeros(skv, f)
        for j in range(skv):
            s = f(0)
            for dd in range(d):
                s = f(s + f(f(i * d + dd + 1) * f(f(dd * skv + j + 1) * f(0.5))))
            scores[j] = f(s * f(scale))
        mx = scores.max()
        probs = np.zeros(skv, f)
        se = f(0)
        for j in range(skv):
            probs[j] = np.exp(f(scores[j] - mx), dtype=f)
            se = f(se + probs[j])
        inv = f(f(1) / se)
        probs = (probs * inv).astype(f)
        for dd in range(d):
            s = f(0)
            for j in range(skv):
                s = f(s + f(probs[j] * f(f(j * d + dd + 1) * f(0.25))))
            expected[i, dd] = s
    np.savez_compressed(HERE / "kat_sdpa_2x3x4.npz", q=q, kt=kt, v=v, scale=np.array([scale], np.float64),
                        expected=expected, tol=np.array([1e-4]))


def oracle_small_cases():
    out = {}
    rng = np.random.default_rng(99)
    # decode over a contiguous cache
    hq, hkv, d, seq, max_seq = 8, 2, 16, 37, 48
    q = rng.standard_normal((1, 1, hq, d)).astype(np.float32)
    kc = rng.standard_normal((hkv, max_seq, d)).astype(np.float16)
    vc = rng.standard_normal((hkv, max_seq, d)).astype(np.float16)
    k_all = pyoracle.cache_to_fp32(kc.view(np.uint16), seq)
    v_all = pyoracle.cache_to_fp32(vc.view(np.uint16), seq)
    out.update(dec_q=q, dec_k=kc.view(np.uint16), dec_v=vc.view(np.uint16), dec_seq=np.array([seq]),
               dec_out=pyoracle.attention(q, k_all, v_all, start_pos=seq - 1, threads=1))
    # causal prefill
    s = 19
    q = rng.standard_normal((1, s, hq, d)).astype(np.float32)
    k = rng.standard_normal((s, hkv, d)).astype(np.float32)
    v = rng.standard_normal((s, hkv, d)).astype(np.float32)
    out.update(pre_q=q, pre_k=k, pre_v=v, pre_out=pyoracle.attention(q, k, v, start_pos=0, threads=1))
    # tree
    n, prefix = 12, 21
    parents = synth.tree_parents(3, n)
    q = rng.standard_normal((1, n, hq, d)).astype(np.float32)
    kp = rng.standard_normal((prefix, hkv, d)).astype(np.float32)
    vp = rng.standard_normal((prefix, hkv, d)).astype(np.float32)
    kt = rng.standard_normal((1, n, hkv, d)).astype(np.float32)
    vt = rng.standard_normal((1, n, hkv, d)).astype(np.float32)
    out.update(tree_parents=parents, tree_q=q, tree_kp=kp, tree_vp=vp, tree_kt=kt, tree_vt=vt,
               tree_mask=pyoracle.tree_mask(parents),
               tree_out=pyoracle.attention_tree(q, kp, vp, kt, vt, parents, threads=1))
    np.savez_compressed(HERE / "oracle_small_cases.npz", **out)


if __name__ == "__main__":
    ref = pyoracle.Ref()
    ref_fp16(ref)
    ref_paged_pool(ref)
    ref_kvcache(ref)
    ref_spec_tree(ref)
    ref_rope(ref)
    ref_attention_loops(ref)
    kat_sdpa()
    oracle_small_cases()
    for p in sorted(HERE.glob("*.npz")):
        print(p.name, p.stat().st_size)
