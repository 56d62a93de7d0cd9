"""The C++ faces (CudaBackend, CudaAttentionOp, KVCache, PagedKVPool + CudaCompute) on a GPU, driven
through their extern "C" test drivers, plus the K/V append kernels through the C ABI."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

from conftest import assert_attention_close

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")


@pytest.fixture(scope="module", params=["standin", "reference_headers"])
def host_lib(request):
    """The test drivers of the C++ host faces: over the product library's classes, and - where it was
    built from the Granite checkout - the same class bodies compiled against Granite's real headers."""
    from host_drivers import build as drivers
    if request.param == "reference_headers" and not drivers.dropin_available():
        pytest.skip("oracle/_ref/libgranite_dropin.so not built (needs the Granite checkout)")
    lib = drivers.load(request.param)
    lib.granite_host_last_error.restype = C.c_char_p
    lib.granite_host_backend_selftest.argtypes = [C.c_int]
    lib.granite_host_operator_attention.argtypes = [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                    C.c_int, C.c_int, C.c_int, C.c_int, C.c_double, C.c_int64]
    lib.granite_host_kvcache_append.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, _i32p, C.c_int, _u16p, _u16p,
                                                _u16p, _u16p, _i32p, _i32p]
    lib.granite_host_paged_flow.argtypes = [C.c_int, C.c_int, _i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                            _f32p, _f32p, _f32p, _f32p, _i32p, C.c_int, _u16p, _u16p, C.c_int]
    lib.granite_host_rope_apply.argtypes = [C.c_int, _f32p, _f32p] + [C.c_int] * 6 + [C.c_float]
    lib.granite_host_decode_batch_flow.argtypes = [C.c_int, C.c_int, _i32p] + [C.c_int] * 10 + [_f32p] * 7 + \
        [_i32p, _i32p, _u16p, _u16p]
    lib.granite_host_decode_batch_regrow.argtypes = [C.c_int, C.c_int, C.c_int, _i32p, _i32p, _i32p]
    return lib


def test_backend_buffer_semantics(host_lib):
    lib = host_lib
    rc = lib.granite_host_backend_selftest(0)
    assert rc == 0, (rc, lib.granite_host_last_error())


def test_operator_known_answer_2x3x4(host_lib):
    """The reference's one attention test (tests/test_vulkan.cpp:353-482), same flow, CUDA backend."""
    lib = host_lib
    g = np.load(GOLD / "kat_sdpa_2x3x4.npz")
    q, kt, v = (np.ascontiguousarray(g[k], np.float32) for k in ("q", "kt", "v"))
    out = np.zeros_like(q)
    rc = lib.granite_host_operator_attention(0, 0, q.ctypes.data, kt.ctypes.data, v.ctypes.data, out.ctypes.data,
                                             2, 3, 4, 1, float(g["scale"][0]), 0)
    assert rc == 0, (rc, lib.granite_host_last_error())
    assert np.abs(out - g["expected"]).max() <= 1e-4  # the reference test's bound


@pytest.mark.parametrize("dtype,sq,skv,d,start_pos", [(0, 7, 33, 16, 0), (0, 50, 300, 128, 0), (1, 5, 9, 64, 0),
                                                      (1, 6, 40, 32, 11), (1, 200, 700, 128, 500), (1, 130, 130, 64, 0),
                                                      (1, 300, 300, 128, 0)])
def test_operator_layouts(host_lib, dtype, sq, skv, d, start_pos):
    """fp32: K pre-transposed, no mask (Vulkan contract); fp16: K row-major with the causal limit
    q + start_pos + 1 (Metal contract); default scale 1/sqrt(D)."""
    from oracle import pyoracle
    lib = host_lib
    rng = np.random.default_rng(sq * 100 + skv)
    q = rng.standard_normal((sq, d), np.float32)
    k = rng.standard_normal((skv, d), np.float32)
    v = rng.standard_normal((skv, d), np.float32)
    if dtype == 0:
        kt = np.ascontiguousarray(k.T)
        out = np.zeros((sq, d), np.float32)
        rc = lib.granite_host_operator_attention(0, 0, q.ctypes.data, kt.ctypes.data, v.ctypes.data, out.ctypes.data,
                                                 sq, skv, d, 0, 0.0, 0)
        ref = pyoracle.sdpa_kt(q, kt, v, 1.0 / np.sqrt(d))
        got = out
    else:
        qh, kh, vh = q.astype(np.float16), k.astype(np.float16), v.astype(np.float16)
        out = np.zeros((sq, d), np.float16)
        rc = lib.granite_host_operator_attention(0, 1, qh.ctypes.data, kh.ctypes.data, vh.ctypes.data,
                                                 out.ctypes.data, sq, skv, d, 0, 0.0, start_pos)
        ref = pyoracle.sdpa_kt(qh.astype(np.float32), np.ascontiguousarray(kh.astype(np.float32).T),
                               vh.astype(np.float32), 1.0 / np.sqrt(d), causal_start_pos=start_pos)
        got = out.astype(np.float32)
    assert rc == 0, (rc, lib.granite_host_last_error())
    assert_attention_close(got, ref, f"operator dtype={dtype}")


def test_kvcache_append_layout_matches_reference(host_lib):
    """Device KVCache against the bytes the reference KVCache produced (src/llm/kv_cache.cpp:52-107)."""
    lib = host_lib
    g = np.load(GOLD / "ref_kvcache_append.npz")
    hkv, d, max_seq = (int(x) for x in g["shape"])
    steps = np.ascontiguousarray(g["steps"], np.int32)
    k_out = np.zeros((hkv, max_seq, d), np.uint16)
    v_out = np.zeros_like(k_out)
    fl, oc = np.zeros(1, np.int32), np.zeros(1, np.int32)
    rc = lib.granite_host_kvcache_append(0, hkv, d, max_seq, steps, len(steps), np.ascontiguousarray(g["k_chunks"]),
                                         np.ascontiguousarray(g["v_chunks"]), k_out.reshape(-1), v_out.reshape(-1),
                                         fl, oc)
    assert rc == 0, (rc, lib.granite_host_last_error())
    assert np.array_equal(k_out, g["k_out"]) and np.array_equal(v_out, g["v_out"])
    assert int(fl[0]) == int(g["final_len"][0])
    assert int(oc[0]) == 16  # InvalidArgument: "KV cache overflow"


@pytest.mark.parametrize("lens,hq,hkv,step", [([40, 7, 129, 16], 32, 8, 24), ([300], 8, 2, 300), ([5, 5, 5], 16, 4, 1)])
def test_page_manager_in_hbm_end_to_end(host_lib, lens, hq, hkv, step):
    """PagedKVPool on the CUDA backend: ragged growth through BlockManager, fp32 K/V appended into
    the HBM pool by paged_kv_cache_append, tables mirrored to the device, one batched decode.
    Checks: every row read back through the block table is bit-identical to the reference's
    truncating fp32->fp16 of what was appended; the decode output matches the CPU attention."""
    from oracle import pyoracle
    lib = host_lib
    d, bs = 128, 16
    lens_a = np.array(lens, np.int32)
    batch = len(lens)
    num_blocks = int(((lens_a + bs - 1) // bs).sum()) + 3
    max_blocks = int(((lens_a + bs - 1) // bs).max())
    rng = np.random.default_rng(sum(lens))
    k_src = [rng.standard_normal((hkv, L, d), np.float32) for L in lens]
    v_src = [rng.standard_normal((hkv, L, d), np.float32) for L in lens]
    q = rng.standard_normal((batch, hq, d), np.float32)
    out = np.zeros((batch, hq, d), np.float32)
    tables = np.zeros((batch, max_blocks), np.int32)
    k_pool = np.zeros((num_blocks * bs, hkv, d), np.uint16)
    v_pool = np.zeros_like(k_pool)
    rc = lib.granite_host_paged_flow(0, batch, lens_a, hq, hkv, d, bs, num_blocks,
                                     np.concatenate([a.reshape(-1) for a in k_src]),
                                     np.concatenate([a.reshape(-1) for a in v_src]), q.reshape(-1), out.reshape(-1),
                                     tables.reshape(-1), max_blocks, k_pool.reshape(-1), v_pool.reshape(-1), step)
    assert rc == 0, (rc, lib.granite_host_last_error())
    trunc = np.vectorize(pyoracle.fp32_to_fp16, otypes=[np.uint16])
    used = set()
    for b, L in enumerate(lens):
        nb = (L + bs - 1) // bs
        assert (tables[b, :nb] >= 0).all() and (tables[b, nb:] == -1).all()
        used.update(int(x) for x in tables[b, :nb])
        rows, bad = pyoracle.paged_gather(k_pool, tables[b].clip(0), L, bs)
        vrows, _ = pyoracle.paged_gather(v_pool, tables[b].clip(0), L, bs)
        assert bad == 0
        assert np.array_equal(rows, trunc(k_src[b]).transpose(1, 0, 2)), f"K rows of sequence {b}"
        assert np.array_equal(vrows, trunc(v_src[b]).transpose(1, 0, 2)), f"V rows of sequence {b}"
    assert len(used) == int(((lens_a + bs - 1) // bs).sum())  # no page shared between sequences
    ref, bad = pyoracle.paged_decode_batch(q, k_pool, v_pool, tables.clip(0), lens_a, bs)
    assert bad == 0
    assert_attention_close(out, ref, "decode through the HBM page manager")


def test_kv_cache_append_kernel_is_bit_exact(compute):
    """kv_cache_append through the C ABI: [new_len, H, D] fp32 -> [H, max_seq, D] fp16 with the
    reference CPU's truncating cast, including values that flush to zero or clamp to infinity."""
    import torch
    from oracle import pyoracle
    dev = "cuda:0"
    h, d, max_seq, cur, new = 3, 64, 40, 9, 17
    rng = np.random.default_rng(8)
    nk = rng.standard_normal((new, h, d), np.float32)
    nv = rng.standard_normal((new, h, d), np.float32)
    nk.reshape(-1)[:6] = [1e-8, -1e-8, 70000.0, -70000.0, 0.333374, 6.0e-5]
    ck = torch.zeros((h, max_seq, d), dtype=torch.float16, device=dev)
    cv = torch.zeros_like(ck)
    compute.kv_cache_append(ck, cv, torch.from_numpy(nk).to(dev), torch.from_numpy(nv).to(dev), h, d, cur, new, max_seq)
    compute.sync()
    trunc = np.vectorize(pyoracle.fp32_to_fp16, otypes=[np.uint16])
    want_k = np.zeros((h, max_seq, d), np.uint16)
    want_v = np.zeros_like(want_k)
    want_k[:, cur:cur + new] = trunc(nk).transpose(1, 0, 2)
    want_v[:, cur:cur + new] = trunc(nv).transpose(1, 0, 2)
    assert np.array_equal(ck.cpu().numpy().view(np.uint16), want_k)
    assert np.array_equal(cv.cpu().numpy().view(np.uint16), want_v)
    import granite_b200 as g
    with pytest.raises(g.GraniteCudaError) as ei:
        compute.kv_cache_append(ck, cv, ck, cv, h, d, 30, 17, max_seq)
    assert ei.value.code == g.ErrorCode.InvalidArgument


def test_batched_paged_append_then_decode(compute):
    """A decode step of a batch: one new token per sequence appended at positions[b], then attended."""
    import torch
    from oracle import pyoracle
    from granite_b200 import synth
    dev = "cuda:0"
    case = synth.paged_case(seed=31, batch=5, len_lo=1, len_hi=90, num_heads=16, num_kv_heads=4, spare_blocks=0)
    lens = case.seq_lens.copy()
    k = torch.from_numpy(case.k_pool).to(dev)
    v = torch.from_numpy(case.v_pool).to(dev)
    tables = torch.from_numpy(case.tables).to(dev)
    rng = np.random.default_rng(2)
    nk = rng.standard_normal((case.batch, 4, 128), np.float32)
    nv = rng.standard_normal((case.batch, 4, 128), np.float32)
    pos = (lens - 1).astype(np.int32)  # overwrite each sequence's last token
    compute.paged_kv_cache_append(torch.from_numpy(nk).to(dev), torch.from_numpy(nv).to(dev), k, v, tables, 4, 128, 0,
                                  0, 16, num_blocks=case.num_blocks, table_len=case.max_blocks,
                                  positions=torch.from_numpy(pos).to(dev), batch_size=case.batch)
    out = torch.zeros((case.batch, 16, 128), device=dev)
    compute.batched_paged_attention_decode(torch.from_numpy(case.q).to(dev), k, v, tables, torch.from_numpy(lens).to(dev),
                                           out, case.batch, 16, 4, 128, 16, case.max_blocks, 1 / np.sqrt(128.0),
                                           num_blocks=case.num_blocks)
    compute.sync()
    trunc = np.vectorize(pyoracle.fp32_to_fp16, otypes=[np.uint16])
    kp, vp = case.k_pool.view(np.uint16).copy(), case.v_pool.view(np.uint16).copy()
    for b in range(case.batch):
        row = case.tables[b, pos[b] // 16] * 16 + pos[b] % 16
        kp[row], vp[row] = trunc(nk[b]), trunc(nv[b])
    assert np.array_equal(k.cpu().numpy().view(np.uint16), kp)
    ref, _ = pyoracle.paged_decode_batch(case.q, kp, vp, case.tables.clip(0), lens, 16)
    assert_attention_close(out.cpu().numpy(), ref, "append + decode")


def test_rope_cache_apply_through_backend_tensors(host_lib):
    """RoPECache::apply (src/llm/rope.cpp:24-92) on CUDA-backend tensors against the reference's outputs."""
    lib = host_lib
    g = np.load(GOLD / "ref_rope.npz")
    for i in range(2):
        seq, hq, hk, d, start, max_seq = (int(x) for x in g[f"a{i}_cfg"])
        q = g[f"a{i}_q"].view(np.float32).copy()
        k = g[f"a{i}_k"].view(np.float32).copy()
        rc = lib.granite_host_rope_apply(0, q.reshape(-1), k.reshape(-1), seq, hq, hk, d, start, max_seq, 10000.0)
        assert rc == 0, (rc, lib.granite_host_last_error())
        assert np.array_equal(q.view(np.uint32), g[f"a{i}_q_out"])
        assert np.array_equal(k.view(np.uint32), g[f"a{i}_k_out"])
    q = np.zeros((3, 1, 16), np.float32)
    rc = lib.granite_host_rope_apply(0, q.reshape(-1), q.copy().reshape(-1), 3, 1, 1, 16, 46, 48, 10000.0)
    assert rc == int(g["range_error_code"][0])  # InvalidArgument, as the reference answers
    assert b"RoPE position out of range: 46 + 3 > 48" in lib.granite_host_last_error()


@pytest.mark.parametrize("lens0,n_steps,remove_slot,remove_at", [([5, 0, 31, 16, 100], 40, 2, 7), ([300] * 3, 20, -1, 0),
                                                                ([1], 33, -1, 0)])
def test_batched_decode_loop_replays_on_the_cpu_checker(host_lib, lens0, n_steps, remove_slot, remove_at):
    """PagedKVPool + RoPECache + PagedDecodeBatch over several decode steps, one request leaving on
    the way: every step's rotated queries and cache bytes bit-exact, every output within tolerance."""
    from oracle import pyoracle
    lib = host_lib
    batch, hq, hkv, d, bs = len(lens0), 32, 8, 128, 16
    max_seq = 512
    max_blocks = max_seq // bs
    num_blocks = sum((n + n_steps + bs - 1) // bs for n in lens0) + 2
    rng = np.random.default_rng(batch * 7 + n_steps)
    lens0 = np.array(lens0, np.int32)
    prompt_k = rng.standard_normal((max(int(lens0.sum()), 1), hkv, d), dtype=np.float32)
    prompt_v = rng.standard_normal(prompt_k.shape, dtype=np.float32)
    step_q = rng.standard_normal((n_steps, batch, hq, d), dtype=np.float32)
    step_k = rng.standard_normal((n_steps, batch, hkv, d), dtype=np.float32)
    step_v = rng.standard_normal((n_steps, batch, hkv, d), dtype=np.float32)
    out = np.full((n_steps, batch, hq, d), np.nan, np.float32)
    q_rot = np.full_like(out, np.nan)
    tables = np.zeros((n_steps, batch, max_blocks), np.int32)
    lens = np.zeros((n_steps, batch), np.int32)
    k_pool = np.zeros((num_blocks * bs, hkv, d), np.uint16)
    v_pool = np.zeros_like(k_pool)
    rc = lib.granite_host_decode_batch_flow(0, batch, lens0, n_steps, remove_slot, remove_at, hq, hkv, d, bs, num_blocks,
                                            max_blocks, max_seq, prompt_k.reshape(-1), prompt_v.reshape(-1),
                                            step_q.reshape(-1), step_k.reshape(-1), step_v.reshape(-1), out.reshape(-1),
                                            q_rot.reshape(-1), tables.reshape(-1), lens.reshape(-1), k_pool.reshape(-1),
                                            v_pool.reshape(-1))
    assert rc == 0, (rc, lib.granite_host_last_error())

    # replay on the CPU checker with the block tables the page manager handed out
    cos, sin = pyoracle.rope_table(max_seq, d)
    ck = np.zeros_like(k_pool)
    cv = np.zeros_like(v_pool)
    off = 0
    for b in range(batch):
        n = int(lens0[b])
        if n:
            tab = np.where(tables[0, b] < 0, 0, tables[0, b])[None]
            _, bad = pyoracle.rope_paged_append(None, prompt_k[off:off + n][None], prompt_v[off:off + n][None], cos, sin,
                                                ck, cv, tab, np.zeros(1, np.int32), bs)
            assert bad == 0
        off += n
    for step in range(n_steps):
        active = [b for b in range(batch) if lens[step, b] >= 0]
        expect_active = [b for b in range(batch) if not (b == remove_slot and step >= remove_at)]
        assert active == expect_active
        for b in active:
            assert lens[step, b] == lens0[b] + step + 1
            tab = np.where(tables[step, b] < 0, 0, tables[step, b])[None]
            qr, bad = pyoracle.rope_paged_append(step_q[step, b][None, None], step_k[step, b][None, None],
                                                 step_v[step, b][None, None], cos, sin, ck, cv, tab,
                                                 np.array([lens[step, b] - 1], np.int32), bs)
            assert bad == 0
            assert np.array_equal(qr.reshape(hq, d).view(np.uint32), q_rot[step, b].view(np.uint32))
            ref, bad = pyoracle.paged_decode_batch(qr.reshape(1, hq, d), ck, cv, tab, lens[step, b:b + 1], bs)
            assert bad == 0
            assert_attention_close(out[step, b][None], ref, f"step {step} slot {b}")
    # pages the departed request gave back were handed out again and overwritten; everything
    # that is live at the end must hold the checker's bytes
    live = np.zeros(num_blocks * bs, bool)
    for b in range(batch):
        if lens[-1, b] >= 0:
            for pos in range(int(lens[-1, b])):
                live[tables[-1, b, pos // bs] * bs + pos % bs] = True
    assert np.array_equal(k_pool[live], ck[live]) and np.array_equal(v_pool[live], cv[live])


def test_device_block_table_follows_a_table_that_shrank_and_regrew(host_lib):
    """A sequence truncated across a block boundary (as after a tree commit) whose freed block went to
    another request and which then regrew over a different block: the device row must not keep the
    freed block's number."""
    lib = host_lib
    bs, max_blocks = 16, 6
    dev_rows = np.full((2, max_blocks), -7, np.int32)
    host_rows = np.full((2, max_blocks), -7, np.int32)
    lens = np.zeros(4, np.int32)
    rc = lib.granite_host_decode_batch_regrow(0, bs, max_blocks, dev_rows.reshape(-1), host_rows.reshape(-1), lens)
    assert rc == 0, (rc, lib.granite_host_last_error())
    assert np.array_equal(lens[:2], lens[2:])
    for b in range(2):
        n = int((host_rows[b] >= 0).sum())
        assert n == (lens[2 + b] + bs - 1) // bs
        assert np.array_equal(dev_rows[b, :n], host_rows[b, :n]), (b, dev_rows[b], host_rows[b])
    assert len(set(host_rows[host_rows >= 0].tolist())) == int((host_rows >= 0).sum())  # no block owned twice
