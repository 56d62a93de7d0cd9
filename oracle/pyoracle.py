"""ctypes face of liboracle.so (this directory's C restatement of Granite's CPU attention) and,
when it was built, of _ref/libgranite_ref.so (the reference's own sources).

TEST INFRASTRUCTURE ONLY: checker for tests/, the smoke check and the CPU-baseline timing.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_LIB = _DIR / "liboracle.so"
_REF = _DIR / "_ref" / "libgranite_ref.so"


def reference_checkout() -> Path | None:
    """The Granite checkout the reference half is built from: $GRANITE_REF_DIR, else a directory
    named `reference` beside this repository; None when neither holds Granite's sources."""
    cand = os.environ.get("GRANITE_REF_DIR")
    path = Path(cand) if cand else _DIR.parent.parent / "reference"
    return path if (path / "src" / "llm" / "transformer.mm").exists() else None


def build(quiet: bool = True) -> None:
    """Compiles liboracle.so (and _ref/ when the reference checkout is present)."""
    cmd = ["make", "-C", str(_DIR)]
    ref = reference_checkout()
    if ref is not None:
        cmd.append(f"GRANITE_REF_DIR={ref}")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + res.stdout + res.stderr)
    if not quiet:
        print(res.stdout)


def _load():
    if not _LIB.exists():
        build()
    return C.CDLL(str(_LIB))


_lib = _load()
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")

_lib.gro_fp16_to_fp32.restype = C.c_float
_lib.gro_fp16_to_fp32.argtypes = [C.c_uint16]
_lib.gro_fp32_to_fp16.restype = C.c_uint16
_lib.gro_fp32_to_fp16.argtypes = [C.c_float]
_lib.gro_cache_to_fp32.argtypes = [_u16p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int]
_lib.gro_paged_gather_f16.restype = C.c_int
_lib.gro_paged_gather_f16.argtypes = [_u16p, _i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _u16p]
_lib.gro_f16_to_f32_array.argtypes = [_u16p, _f32p, C.c_size_t]
_lib.gro_attention.argtypes = [_f32p, _f32p, _f32p, _f32p] + [C.c_int] * 7 + [C.c_float, C.c_int]
_lib.gro_tree_mask.argtypes = [_i32p, C.c_int, _u8p]
_lib.gro_tree_validate.restype = C.c_int
_lib.gro_tree_validate.argtypes = [_i32p, C.c_int]
_lib.gro_attention_tree.argtypes = [_f32p] * 5 + [_u8p, _f32p] + [C.c_int] * 6 + [C.c_float, C.c_int]
_lib.gro_paged_decode_batch.restype = C.c_int
_lib.gro_paged_decode_batch.argtypes = [_f32p, _u16p, _u16p, _i32p, _i32p, _f32p] + [C.c_int] * 7 + [C.c_float, C.c_int, C.c_int]
_lib.gro_sdpa_kt.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int]
_lib.gro_rope_table.argtypes = [C.c_int, C.c_int, C.c_float, _f32p, _f32p]
_lib.gro_rope_apply.restype = C.c_int
_lib.gro_rope_apply.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p, _f32p, C.c_int]
_lib.gro_rope_paged_append.restype = C.c_int
_lib.gro_rope_paged_append.argtypes = [C.c_void_p, _f32p, _f32p, _f32p, _f32p, C.c_int, _u16p, _u16p, _i32p, _i32p] + [C.c_int] * 8
_lib.gro_tree_commit.restype = C.c_int
_lib.gro_tree_commit.argtypes = [_u16p, _u16p, _u16p, _u16p, _i32p, _i32p, _i32p, _i32p] + [C.c_int] * 8


def num_threads() -> int:
    """std::thread::hardware_concurrency(), the reference's policy (src/llm/math_ops.cpp:56-58)."""
    return os.cpu_count() or 1


def fp16_to_fp32(h: int) -> float:
    return float(_lib.gro_fp16_to_fp32(h))


def fp32_to_fp16(f: float) -> int:
    return int(_lib.gro_fp32_to_fp16(f))


def f16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16)
    out = np.empty(a.shape, np.float32)
    _lib.gro_f16_to_f32_array(a.reshape(-1), out.reshape(-1), a.size)
    return out


def cache_to_fp32(cache_bits: np.ndarray, total_seq: int) -> np.ndarray:
    """[Hkv, max_seq, D] fp16 bits -> [total_seq, Hkv, D] fp32 (transformer.mm:1753-1763)."""
    hkv, max_seq, d = cache_bits.shape
    out = np.empty((total_seq, hkv, d), np.float32)
    _lib.gro_cache_to_fp32(np.ascontiguousarray(cache_bits, np.uint16), out, hkv, max_seq, total_seq, d)
    return out


def paged_gather(pool_bits: np.ndarray, table: np.ndarray, seq_len: int, block_size: int):
    """pool [num_blocks*bs, Hkv, D] fp16 bits -> ([seq_len, Hkv, D] bits, bad entries)."""
    rows, hkv, d = pool_bits.shape
    out = np.empty((seq_len, hkv, d), np.uint16)
    bad = _lib.gro_paged_gather_f16(np.ascontiguousarray(pool_bits, np.uint16),
                                    np.ascontiguousarray(table, np.int32), seq_len, block_size,
                                    rows // block_size, hkv, d, out)
    return out, bad


def attention(q, k_all, v_all, start_pos: int, scale: float = 0.0, threads: int | None = None):
    """q [B,Sq,Hq,D]; k_all, v_all [T,Hkv,D] fp32 -> ctx [B,Sq,Hq,D] (transformer.mm:1779-1840)."""
    q = np.ascontiguousarray(q, np.float32)
    k_all = np.ascontiguousarray(k_all, np.float32)
    v_all = np.ascontiguousarray(v_all, np.float32)
    b, sq, hq, d = q.shape
    t, hkv, _ = k_all.shape
    ctx = np.empty_like(q)
    _lib.gro_attention(q, k_all, v_all, ctx, b, sq, t, hq, hkv, d, start_pos, scale,
                       threads or num_threads())
    return ctx


def tree_mask(parents) -> np.ndarray:
    parents = np.ascontiguousarray(parents, np.int32)
    n = parents.size
    m = np.zeros((n, n), np.uint8)
    _lib.gro_tree_mask(parents, n, m)
    return m


def tree_validate(parents) -> bool:
    parents = np.ascontiguousarray(parents, np.int32)
    return _lib.gro_tree_validate(parents, parents.size) == 0


def attention_tree(q, k_cached, v_cached, k_tree, v_tree, parents, scale: float = 0.0,
                   threads: int | None = None):
    """q [B,N,Hq,D]; k_cached/v_cached [L,Hkv,D]; k_tree/v_tree [B,N,Hkv,D]; all fp32."""
    q = np.ascontiguousarray(q, np.float32)
    b, n, hq, d = q.shape
    k_tree = np.ascontiguousarray(k_tree, np.float32)
    v_tree = np.ascontiguousarray(v_tree, np.float32)
    hkv = k_tree.shape[2]
    k_cached = np.ascontiguousarray(k_cached, np.float32).reshape(-1, hkv, d)
    v_cached = np.ascontiguousarray(v_cached, np.float32).reshape(-1, hkv, d)
    mask = tree_mask(parents)
    ctx = np.empty_like(q)
    _lib.gro_attention_tree(q, k_cached, v_cached, k_tree, v_tree, mask, ctx, b, n,
                            k_cached.shape[0], hq, hkv, d, scale, threads or num_threads())
    return ctx


def paged_decode_batch(q, k_pool, v_pool, tables, seq_lens, block_size: int, scale: float = 0.0,
                       threads: int | None = None, stride: int = 1):
    """q [B,Hq,D] fp32; pools [rows,Hkv,D] fp16 bits; tables [B,max_blocks]; -> (out, bad)."""
    q = np.ascontiguousarray(q, np.float32)
    b, hq, d = q.shape
    rows, hkv, _ = k_pool.shape
    tables = np.ascontiguousarray(tables, np.int32).reshape(b, -1)
    out = np.zeros_like(q)
    bad = _lib.gro_paged_decode_batch(q, np.ascontiguousarray(k_pool, np.uint16),
                                      np.ascontiguousarray(v_pool, np.uint16), tables,
                                      np.ascontiguousarray(seq_lens, np.int32), out, b, hq, hkv, d,
                                      block_size, tables.shape[1], rows // block_size, scale,
                                      threads or num_threads(), stride)
    return out, bad


def sdpa_kt(q, kt, v, scale: float, causal_start_pos: int = -1):
    """Operator-level attention with K pre-transposed [D,T] (vulkan_operators.cpp:345-434)."""
    q = np.ascontiguousarray(q, np.float32)
    kt = np.ascontiguousarray(kt, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    out = np.empty_like(q)
    _lib.gro_sdpa_kt(q, kt, v, out, q.shape[0], kt.shape[1], q.shape[1], scale, causal_start_pos)
    return out


def rope_table(max_seq: int, head_dim: int, theta: float = 10000.0):
    """cos, sin [max_seq, head_dim/2] as RoPECache::initialize builds them (src/llm/rope.cpp:5-22)."""
    cos = np.empty((max_seq, head_dim // 2), np.float32)
    sin = np.empty_like(cos)
    _lib.gro_rope_table(max_seq, head_dim, theta, cos, sin)
    return cos, sin


def rope_apply(x: np.ndarray, start_pos: int, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """x [seq, heads, D] -> rotated copy (src/llm/rope.cpp:52-86)."""
    out = np.ascontiguousarray(x, np.float32).copy()
    seq, heads, d = out.shape
    rc = _lib.gro_rope_apply(out, seq, heads, d, start_pos, np.ascontiguousarray(cos, np.float32),
                             np.ascontiguousarray(sin, np.float32), cos.shape[0])
    if rc:
        raise ValueError("RoPE position out of range")
    return out


def rope_paged_append(q, k, v, cos, sin, k_pool, v_pool, tables, positions, block_size: int):
    """q [B, new_len, Hq, D] (or None), k/v [B, new_len, Hkv, D] fp32; pools [num_blocks*bs, Hkv, D]
    fp16 bits, updated in place.  Returns (rotated q, tokens that could not be written)."""
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    batch, new_len, hkv, d = k.shape
    qr = None if q is None else np.ascontiguousarray(q, np.float32).copy()
    hq = 0 if qr is None else qr.shape[2]
    tables = np.ascontiguousarray(tables, np.int32)
    assert k_pool.dtype == np.uint16 and k_pool.flags.c_contiguous and v_pool.flags.c_contiguous
    bad = _lib.gro_rope_paged_append(None if qr is None else qr.ctypes.data_as(C.c_void_p), k, v,
                                     np.ascontiguousarray(cos, np.float32), np.ascontiguousarray(sin, np.float32),
                                     cos.shape[0], k_pool, v_pool, tables, np.ascontiguousarray(positions, np.int32),
                                     batch, new_len, hq, hkv, d, block_size, tables.shape[1],
                                     k_pool.shape[0] // block_size)
    return qr, bad


def tree_commit(k_tree, v_tree, k_pool, v_pool, tables, cache_lens, accepted, num_accepted, block_size: int) -> int:
    """Tree K/V [B, Hkv, N, D] fp16 bits: accepted rows -> the paged pools (in place). Returns rows skipped."""
    batch, hkv, n, d = k_tree.shape
    tables = np.ascontiguousarray(tables, np.int32)
    accepted = np.ascontiguousarray(accepted, np.int32)
    return _lib.gro_tree_commit(np.ascontiguousarray(k_tree, np.uint16), np.ascontiguousarray(v_tree, np.uint16),
                                k_pool, v_pool, tables, np.ascontiguousarray(cache_lens, np.int32), accepted,
                                np.ascontiguousarray(num_accepted, np.int32), batch, n, accepted.shape[1], hkv, d,
                                block_size, tables.shape[1], k_pool.shape[0] // block_size)


# ------------------------------------------------------------------ the reference's own objects
def ref_available() -> bool:
    return _REF.exists()


class Ref:
    """C-ABI glue over the reference's unmodified sources (see ref_harness.cpp)."""

    def __init__(self):
        if not _REF.exists():
            raise FileNotFoundError(f"{_REF} was not built (needs the reference checkout)")
        r = C.CDLL(str(_REF))
        r.ref_fp16_to_fp32.restype = C.c_float
        r.ref_fp16_to_fp32.argtypes = [C.c_uint16]
        r.ref_fp32_to_fp16.restype = C.c_uint16
        r.ref_fp32_to_fp16.argtypes = [C.c_float]
        r.ref_fp16_to_fp32_bits.argtypes = [_u16p, np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS"), C.c_size_t]
        r.ref_num_threads.restype = C.c_int
        r.ref_paged_pool_script.restype = C.c_int
        r.ref_paged_pool_script.argtypes = [C.c_int, C.c_int, C.c_int, _i32p, C.c_int, _i32p, _i32p,
                                            _i32p, _i32p, C.c_int, _i32p, _i32p]
        r.ref_kvcache_append.restype = C.c_int
        r.ref_kvcache_append.argtypes = [C.c_int, C.c_int, C.c_int, _i32p, C.c_int, _u16p, _u16p,
                                         _u16p, _u16p, _i32p]
        r.ref_speculation_tree.restype = C.c_int
        r.ref_speculation_tree.argtypes = [_i32p, C.c_int, _i32p, _i32p, _i32p, _i32p, _i32p]
        r.ref_find_accepted_path.restype = C.c_int
        r.ref_find_accepted_path.argtypes = [_i32p, _i32p, C.c_int, _i32p, C.c_int, _i32p, _i32p]
        r.ref_rope_table.restype = C.c_int
        r.ref_rope_table.argtypes = [C.c_int, C.c_int, C.c_float, _f32p, _f32p]
        r.ref_rope_apply.restype = C.c_int
        r.ref_rope_apply.argtypes = [_f32p, _f32p] + [C.c_int] * 6 + [C.c_float]
        # the reference's own attention statements (ref_loops.cpp)
        r.ref_attention_loop.restype = None
        r.ref_attention_loop.argtypes = [_f32p, _f32p, _f32p, _f32p] + [C.c_int] * 7 + [C.c_float]
        r.ref_attention_cache_widen.restype = None
        r.ref_attention_cache_widen.argtypes = [_u16p, _u16p, _f32p, _f32p] + [C.c_int] * 4
        r.ref_tree_mask.restype = None
        r.ref_tree_mask.argtypes = [_i32p, C.c_int, _u8p]
        r.ref_attention_tree_loop.restype = None
        r.ref_attention_tree_loop.argtypes = [_f32p] * 5 + [_i32p, _f32p] + [C.c_int] * 6 + [C.c_float]
        self._r = r

    def attention_loop(self, q, k_all, v_all, start_pos: int, scale: float):
        """The statements of TransformerModel::attention (transformer.mm:1779-1840) on q [B,Sq,Hq,D],
        k_all / v_all [T,Hkv,D] fp32 -> context [B,Sq,Hq,D]."""
        q = np.ascontiguousarray(q, np.float32)
        k_all = np.ascontiguousarray(k_all, np.float32)
        v_all = np.ascontiguousarray(v_all, np.float32)
        b, sq, hq, d = q.shape
        t, hkv, _ = k_all.shape
        out = np.empty_like(q)
        self._r.ref_attention_loop(q, k_all, v_all, out, b, sq, t, hq, hkv, d, start_pos, scale)
        return out

    def attention_cache_widen(self, ck, cv, total_seq: int):
        """transformer.mm:1753-1765: [Hkv, max_seq, D] fp16 bits -> two [total_seq, Hkv, D] fp32."""
        ck = np.ascontiguousarray(ck, np.uint16)
        cv = np.ascontiguousarray(cv, np.uint16)
        hkv, max_seq, d = ck.shape
        k = np.empty((total_seq, hkv, d), np.float32)
        v = np.empty_like(k)
        self._r.ref_attention_cache_widen(ck, cv, k, v, hkv, max_seq, total_seq, d)
        return k, v

    def tree_mask(self, parents) -> np.ndarray:
        """transformer.mm:822-841 on a parent array -> [N, N] bytes."""
        parents = np.ascontiguousarray(parents, np.int32)
        m = np.zeros((parents.size, parents.size), np.uint8)
        self._r.ref_tree_mask(parents, parents.size, m)
        return m

    def attention_tree_loop(self, q, k_cached, v_cached, k_tree, v_tree, parents, scale: float):
        """The statements of TransformerModel::attention_tree (transformer.mm:2044-2126), mask from
        :822-841.  q [B,N,Hq,D]; k_cached / v_cached [L,Hkv,D]; k_tree / v_tree [B,N,Hkv,D]; fp32."""
        q = np.ascontiguousarray(q, np.float32)
        b, n, hq, d = q.shape
        k_tree = np.ascontiguousarray(k_tree, np.float32)
        v_tree = np.ascontiguousarray(v_tree, np.float32)
        hkv = k_tree.shape[2]
        k_cached = np.ascontiguousarray(k_cached, np.float32).reshape(-1, hkv, d)
        v_cached = np.ascontiguousarray(v_cached, np.float32).reshape(-1, hkv, d)
        out = np.empty_like(q)
        self._r.ref_attention_tree_loop(q, k_cached, v_cached, k_tree, v_tree, np.ascontiguousarray(parents, np.int32),
                                        out, b, n, k_cached.shape[0], hq, hkv, d, scale)
        return out

    def rope_table(self, max_seq: int, head_dim: int, theta: float = 10000.0):
        cos = np.empty((max_seq, head_dim // 2), np.float32)
        sin = np.empty_like(cos)
        self._r.ref_rope_table(max_seq, head_dim, theta, cos, sin)
        return cos, sin

    def rope_apply(self, q, k, start_pos: int, max_seq: int, theta: float = 10000.0):
        """q [seq, Hq, D], k [seq, Hk, D] -> rotated copies through RoPECache::apply."""
        q = np.ascontiguousarray(q, np.float32).copy()
        k = np.ascontiguousarray(k, np.float32).copy()
        rc = self._r.ref_rope_apply(q, k, q.shape[0], q.shape[1], k.shape[1], q.shape[2], start_pos, max_seq, theta)
        return q, k, rc

    def fp16_to_fp32(self, h: int) -> float:
        return float(self._r.ref_fp16_to_fp32(h))

    def fp32_to_fp16(self, f: float) -> int:
        return int(self._r.ref_fp32_to_fp16(f))

    def fp16_to_fp32_bits(self, codes: np.ndarray) -> np.ndarray:
        codes = np.ascontiguousarray(codes, np.uint16)
        out = np.empty(codes.shape, np.uint32)
        self._r.ref_fp16_to_fp32_bits(codes.reshape(-1), out.reshape(-1), codes.size)
        return out

    def num_threads(self) -> int:
        return int(self._r.ref_num_threads())

    def paged_pool_script(self, max_sequences, max_total_tokens, block_size, ops, max_blocks):
        ops = np.ascontiguousarray(ops, np.int32).reshape(-1, 3)
        res = np.zeros(len(ops), np.int32)
        seq_lens = np.zeros(max_sequences, np.int32)
        tlens = np.zeros(max_sequences, np.int32)
        tables = np.zeros((max_sequences, max_blocks), np.int32)
        nfree = np.zeros(1, np.int32)
        ntotal = np.zeros(1, np.int32)
        rc = self._r.ref_paged_pool_script(max_sequences, max_total_tokens, block_size, ops.reshape(-1),
                                           len(ops), res, seq_lens, tlens, tables.reshape(-1),
                                           max_blocks, nfree, ntotal)
        if rc != 0:
            raise RuntimeError("reference PagedKVPool failed to initialise")
        return dict(results=res, seq_lens=seq_lens, table_lens=tlens, tables=tables,
                    num_free=int(nfree[0]), num_total=int(ntotal[0]))

    def kvcache_append(self, hkv, d, max_seq, step_lens, k_chunks, v_chunks):
        step_lens = np.ascontiguousarray(step_lens, np.int32)
        k_out = np.zeros((hkv, max_seq, d), np.uint16)
        v_out = np.zeros((hkv, max_seq, d), np.uint16)
        fl = np.zeros(1, np.int32)
        rc = self._r.ref_kvcache_append(hkv, d, max_seq, step_lens, len(step_lens),
                                        np.ascontiguousarray(k_chunks, np.uint16).reshape(-1),
                                        np.ascontiguousarray(v_chunks, np.uint16).reshape(-1),
                                        k_out.reshape(-1), v_out.reshape(-1), fl)
        if rc != 0:
            raise RuntimeError(f"reference KVCache append failed ({rc})")
        return k_out, v_out, int(fl[0])

    def speculation_tree(self, parents):
        parents = np.ascontiguousarray(parents, np.int32)
        n = parents.size
        po = np.zeros(n, np.int32)
        dep = np.zeros(n, np.int32)
        bfs = np.zeros(n, np.int32)
        nb = np.zeros(1, np.int32)
        md = np.zeros(1, np.int32)
        self._r.ref_speculation_tree(parents, n, po, dep, bfs, nb, md)
        return dict(parents=po, depths=dep, bfs=bfs[: int(nb[0])], max_depth=int(md[0]))

    def find_accepted_path(self, parents, tokens, targets):
        parents = np.ascontiguousarray(parents, np.int32)
        tokens = np.ascontiguousarray(tokens, np.int32)
        targets = np.ascontiguousarray(targets, np.int32)
        out = np.zeros(len(targets) + 1, np.int32)
        n = np.zeros(1, np.int32)
        self._r.ref_find_accepted_path(parents, tokens, len(parents), targets, len(targets), out, n)
        return out[: int(n[0])]
