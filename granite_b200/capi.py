"""ctypes binding of include/granite_cuda.h.

Mirrors the attention group of Granite's compute class (include/granite/metal_compute.h:749-920)
with the same method names and argument order, taking raw device pointers (ints) in place of
``MTL::Buffer*``.  Every call goes through the C ABI of libgranite_cuda.so; there is no Python or
CPU implementation behind it.
"""
from __future__ import annotations

import ctypes as C
import enum
from pathlib import Path

_PKG = Path(__file__).resolve().parent


def library_path() -> Path:
    return _PKG / "libgranite_cuda.so"


def _load() -> C.CDLL:
    path = library_path()
    if not path.exists():
        raise ImportError(
            f"{path} is missing: build it with `python -m granite_b200.build` "
            "(nvcc, sm_100a). There is no fallback implementation.")
    return C.CDLL(str(path))


lib = _load()


class ErrorCode(enum.IntEnum):
    """granite::ErrorCode values (include/granite/error.h:16-57)."""
    Success = 0
    FileNotFound = 1
    InvalidFormat = 2
    IOError = 3
    OutOfMemory = 4
    AllocationFailed = 5
    BufferTooSmall = 6
    BackendNotSupported = 7
    BackendNotInitialized = 8
    OperatorNotImplemented = 9
    ShaderCompilationFailed = 10
    ExecutionFailed = 11
    Timeout = 12
    InvalidShape = 13
    ShapeMismatch = 14
    DTypeMismatch = 15
    InvalidArgument = 16
    NullPointer = 17
    InvalidGraph = 18
    CycleDetected = 19
    InvalidState = 20
    UnsupportedModel = 21
    CorruptedWeights = 22
    MissingOperator = 23
    InternalError = 24
    NotImplemented = 25


class GraniteCudaError(RuntimeError):
    def __init__(self, code: int, message: str):
        self.code = ErrorCode(code)
        super().__init__(f"{self.code.name}: {message}")


class PagedDecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("block_tables", C.c_void_p), ("seq_lens", C.c_void_p), ("output", C.c_void_p),
        ("batch_size", C.c_uint32), ("num_heads", C.c_uint32), ("num_kv_heads", C.c_uint32),
        ("head_dim", C.c_uint32), ("block_size", C.c_uint32), ("max_blocks_per_seq", C.c_uint32),
        ("num_blocks", C.c_uint32), ("seq_len", C.c_uint32), ("scale", C.c_float),
    ]


class AttentionArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("output", C.c_void_p),
        ("num_heads", C.c_uint32), ("num_kv_heads", C.c_uint32), ("seq_q", C.c_uint32),
        ("seq_kv", C.c_uint32), ("head_dim", C.c_uint32), ("max_seq", C.c_uint32),
        ("q_dtype", C.c_uint32), ("out_dtype", C.c_uint32), ("scale", C.c_float),
        ("start_pos", C.c_uint32), ("batch_size", C.c_uint32),
    ]


class TreeAttentionArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("k_tree", C.c_void_p),
        ("v_tree", C.c_void_p), ("parent_indices", C.c_void_p), ("block_tables", C.c_void_p),
        ("cache_lens", C.c_void_p), ("output", C.c_void_p),
        ("batch_size", C.c_uint32), ("num_heads", C.c_uint32), ("num_kv_heads", C.c_uint32),
        ("num_nodes", C.c_uint32), ("cache_len", C.c_uint32), ("head_dim", C.c_uint32),
        ("cache_stride", C.c_uint32), ("block_size", C.c_uint32), ("max_blocks_per_seq", C.c_uint32),
        ("num_blocks", C.c_uint32), ("q_dtype", C.c_uint32), ("scale", C.c_float),
    ]


class KvAppendArgs(C.Structure):
    _fields_ = [("cache_k", C.c_void_p), ("cache_v", C.c_void_p), ("new_k", C.c_void_p), ("new_v", C.c_void_p),
                ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("current_len", C.c_uint32),
                ("new_len", C.c_uint32), ("max_seq_len", C.c_uint32)]


class PagedKvAppendArgs(C.Structure):
    _fields_ = [("new_k", C.c_void_p), ("new_v", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
                ("block_table", C.c_void_p), ("positions", C.c_void_p),
                ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("start_pos", C.c_uint32),
                ("new_len", C.c_uint32), ("block_size", C.c_uint32), ("num_blocks", C.c_uint32),
                ("table_len", C.c_uint32), ("batch_size", C.c_uint32)]


class RopeAppendArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("cos_table", C.c_void_p),
                ("sin_table", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
                ("block_tables", C.c_void_p), ("positions", C.c_void_p),
                ("batch_size", C.c_uint32), ("new_len", C.c_uint32), ("num_heads", C.c_uint32),
                ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("block_size", C.c_uint32),
                ("max_blocks_per_seq", C.c_uint32), ("num_blocks", C.c_uint32), ("table_len", C.c_uint32),
                ("start_pos", C.c_uint32)]


class TreeCommitArgs(C.Structure):
    _fields_ = [("k_tree", C.c_void_p), ("v_tree", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
                ("block_tables", C.c_void_p), ("cache_lens", C.c_void_p), ("accepted", C.c_void_p),
                ("num_accepted", C.c_void_p),
                ("batch_size", C.c_uint32), ("num_nodes", C.c_uint32), ("max_accepted", C.c_uint32),
                ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("block_size", C.c_uint32),
                ("max_blocks_per_seq", C.c_uint32), ("num_blocks", C.c_uint32)]


class PagedPrefillArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("block_table", C.c_void_p),
                ("output", C.c_void_p),
                ("num_heads", C.c_uint32), ("num_kv_heads", C.c_uint32), ("seq_q", C.c_uint32),
                ("start_pos", C.c_uint32), ("head_dim", C.c_uint32), ("block_size", C.c_uint32),
                ("max_blocks_per_seq", C.c_uint32), ("num_blocks", C.c_uint32), ("q_dtype", C.c_uint32),
                ("out_dtype", C.c_uint32), ("scale", C.c_float)]


class KernelTiming(C.Structure):
    _fields_ = [("name", C.c_char * 64), ("gpu_time_ms", C.c_double), ("dispatches", C.c_uint64)]


def _sig(name, restype, *argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = list(argtypes)
    return fn


_sig("granite_cuda_last_error_message", C.c_char_p)
_sig("granite_cuda_device_count", C.c_int)
_sig("granite_cuda_compute_create", C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_void_p))
_sig("granite_cuda_compute_destroy", None, C.c_void_p)
_sig("granite_cuda_compute_stream", C.c_void_p, C.c_void_p)
_sig("granite_cuda_compute_sm_count", C.c_int, C.c_void_p)
_sig("granite_cuda_sync", C.c_int, C.c_void_p)
_sig("granite_cuda_get_profiling_stats", None, C.c_void_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64))
_sig("granite_cuda_enable_kernel_timing", None, C.c_void_p, C.c_int)
_sig("granite_cuda_reset_kernel_timing", None, C.c_void_p)
_sig("granite_cuda_get_kernel_timing_stats", C.c_int, C.c_void_p, C.POINTER(KernelTiming), C.c_int)
_sig("granite_cuda_malloc", C.c_int, C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p))
_sig("granite_cuda_free", C.c_int, C.c_void_p, C.c_void_p)
_sig("granite_cuda_malloc_host", C.c_int, C.c_size_t, C.POINTER(C.c_void_p))
_sig("granite_cuda_free_host", C.c_int, C.c_void_p)
_sig("granite_cuda_write_buffer", C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t)
_sig("granite_cuda_read_buffer", C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t)
_sig("granite_cuda_copy_buffer", C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t)
_sig("granite_cuda_memset", C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_size_t)
_sig("granite_cuda_batched_paged_attention_decode", C.c_int, C.c_void_p, C.POINTER(PagedDecodeArgs))
_sig("granite_cuda_batched_paged_attention_decode_gather", C.c_int, C.c_void_p, C.POINTER(PagedDecodeArgs),
     C.POINTER(C.c_void_p), C.c_uint32, C.c_uint64)
_sig("granite_cuda_batched_paged_attention_decode_gather_heads", C.c_int, C.c_void_p, C.POINTER(PagedDecodeArgs),
     C.POINTER(C.c_void_p), C.c_uint32, C.c_uint64, C.c_uint32, C.c_uint32)
_sig("granite_cuda_multihead_attention", C.c_int, C.c_void_p, C.POINTER(AttentionArgs))
_sig("granite_cuda_kv_cache_append", C.c_int, C.c_void_p, C.POINTER(KvAppendArgs))
_sig("granite_cuda_paged_kv_cache_append", C.c_int, C.c_void_p, C.POINTER(PagedKvAppendArgs))
_sig("granite_cuda_attention_tree", C.c_int, C.c_void_p, C.POINTER(TreeAttentionArgs))
_sig("granite_cuda_build_tree_mask", C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32)
_sig("granite_cuda_rope_table_create", C.c_int, C.c_void_p, C.c_uint32, C.c_uint32, C.c_float,
     C.POINTER(C.c_void_p), C.POINTER(C.c_void_p))
_sig("granite_cuda_rope_multihead", C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32,
     C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint32)
_sig("granite_cuda_rope_paged_kv_cache_append", C.c_int, C.c_void_p, C.POINTER(RopeAppendArgs))
_sig("granite_cuda_tree_commit", C.c_int, C.c_void_p, C.POINTER(TreeCommitArgs))
_sig("granite_cuda_paged_prefill_attention", C.c_int, C.c_void_p, C.POINTER(PagedPrefillArgs))
_sig("granite_cuda_selftest_bounded_wait", C.c_int, C.c_void_p, C.c_uint64, C.c_void_p)
_sig("granite_cuda_push_rows", C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_uint32,
     C.c_uint64, C.c_uint64)
_sig("granite_cuda_batched_paged_attention_decode_static", C.c_int, C.POINTER(PagedDecodeArgs), C.c_void_p,
     C.c_void_p)


def last_error() -> str:
    return lib.granite_cuda_last_error_message().decode()


def check(code: int) -> None:
    if code != 0:
        raise GraniteCudaError(code, last_error())


def _ptr(x) -> int:
    """Device/host address of a torch tensor, numpy array, or a plain int address."""
    if x is None:
        return 0
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    raise TypeError(f"cannot take the address of {type(x)!r}")


class CudaCompute:
    """Python face of the compute object, method for method the attention group of MetalCompute.

    ``stream``: a ``cudaStream_t`` as int (e.g. ``torch.cuda.current_stream().cuda_stream``; 0 is
    taken as the default stream) or ``None`` to let the object create its own stream.
    """

    def __init__(self, device: int = 0, stream: int | None = None):
        self._h = C.c_void_p()
        if stream is None:
            raw = 0          # NULL: the object creates its own stream
        elif stream == 0:
            raw = 1          # cudaStreamLegacy: the handle of the default stream (0 itself means "own")
        else:
            raw = stream
        check(lib.granite_cuda_compute_create(device, C.c_void_p(raw), C.byref(self._h)))
        self.device = device

    def shutdown(self) -> None:
        if self._h:
            lib.granite_cuda_compute_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.shutdown()
        except Exception:
            pass

    @property
    def handle(self) -> C.c_void_p:
        return self._h

    @property
    def stream(self) -> int:
        return lib.granite_cuda_compute_stream(self._h) or 0

    @property
    def sm_count(self) -> int:
        return lib.granite_cuda_compute_sm_count(self._h)

    def sync(self) -> None:
        check(lib.granite_cuda_sync(self._h))

    def get_profiling_stats(self) -> tuple[int, int]:
        d, s = C.c_uint64(), C.c_uint64()
        lib.granite_cuda_get_profiling_stats(self._h, C.byref(d), C.byref(s))
        return d.value, s.value

    def enable_kernel_timing(self, enable: bool) -> None:
        lib.granite_cuda_enable_kernel_timing(self._h, int(enable))

    def reset_kernel_timing(self) -> None:
        lib.granite_cuda_reset_kernel_timing(self._h)

    def get_kernel_timing_stats(self) -> dict[str, tuple[float, int]]:
        """{kernel name: (total GPU ms, dispatches)}; drains the stream first."""
        buf = (KernelTiming * 32)()
        n = lib.granite_cuda_get_kernel_timing_stats(self._h, buf, 32)
        return {buf[i].name.decode(): (buf[i].gpu_time_ms, buf[i].dispatches) for i in range(min(n, 32))}

    # ---- raw buffers
    def create_buffer(self, size: int) -> int:
        p = C.c_void_p()
        check(lib.granite_cuda_malloc(self._h, size, C.byref(p)))
        return p.value

    def destroy_buffer(self, ptr: int) -> None:
        check(lib.granite_cuda_free(self._h, C.c_void_p(ptr)))

    def write_buffer(self, dev_ptr, host, nbytes: int) -> None:
        check(lib.granite_cuda_write_buffer(self._h, C.c_void_p(_ptr(dev_ptr)), C.c_void_p(_ptr(host)), nbytes))

    def read_buffer(self, host, dev_ptr, nbytes: int) -> None:
        check(lib.granite_cuda_read_buffer(self._h, C.c_void_p(_ptr(host)), C.c_void_p(_ptr(dev_ptr)), nbytes))

    # ---- attention group
    def batched_paged_attention_decode(self, Q, K_cache, V_cache, block_tables, seq_lens, output,
                                       batch_size, num_heads, num_kv_heads, head_dim, block_size,
                                       max_blocks_per_seq, scale, *, num_blocks, seq_len=0,
                                       gather_ptrs=None, gather_row_offset=0, gather_num_heads=0,
                                       gather_head_offset=0) -> None:
        a = PagedDecodeArgs(_ptr(Q), _ptr(K_cache), _ptr(V_cache), _ptr(block_tables), _ptr(seq_lens),
                            _ptr(output), batch_size, num_heads, num_kv_heads, head_dim, block_size,
                            max_blocks_per_seq, num_blocks, seq_len, scale)
        if gather_ptrs:
            # gather_ptrs: device addresses of [total sequences, num_heads, head_dim] fp32 buffers (this GPU's
            # or peer-mapped ones); every final row is also stored to row gather_row_offset + b of each
            arr = (C.c_void_p * len(gather_ptrs))(*[int(x) for x in gather_ptrs])
            if gather_num_heads:
                # KV heads sharded across GPUs: a destination row holds gather_num_heads query heads and this
                # call's num_heads of them start at gather_head_offset
                check(lib.granite_cuda_batched_paged_attention_decode_gather_heads(
                    self._h, C.byref(a), arr, len(gather_ptrs), int(gather_row_offset), int(gather_num_heads),
                    int(gather_head_offset)))
                return
            check(lib.granite_cuda_batched_paged_attention_decode_gather(self._h, C.byref(a), arr, len(gather_ptrs),
                                                                         int(gather_row_offset)))
            return
        check(lib.granite_cuda_batched_paged_attention_decode(self._h, C.byref(a)))

    def paged_attention_decode(self, Q, K_cache, V_cache, block_table, output, num_heads,
                               num_kv_heads, seq_len, head_dim, block_size, scale, *, num_blocks,
                               num_logical_blocks=None) -> None:
        nlb = num_logical_blocks or (seq_len + block_size - 1) // block_size
        self.batched_paged_attention_decode(Q, K_cache, V_cache, block_table, None, output, 1,
                                            num_heads, num_kv_heads, head_dim, block_size, max(nlb, 1),
                                            scale, num_blocks=num_blocks, seq_len=seq_len)

    def multihead_attention(self, Q, K, V, output, num_heads, num_kv_heads, seq_q, seq_kv, head_dim,
                            scale, max_seq=0, *, q_dtype=0, out_dtype=0, start_pos=0, batch_size=1) -> None:
        a = AttentionArgs(_ptr(Q), _ptr(K), _ptr(V), _ptr(output), num_heads, num_kv_heads, seq_q,
                          seq_kv, head_dim, max_seq, q_dtype, out_dtype, scale, start_pos, batch_size)
        check(lib.granite_cuda_multihead_attention(self._h, C.byref(a)))

    def attention_tree(self, Q, K_cache, V_cache, K_tree, V_tree, parent_indices, output, num_heads,
                       num_kv_heads, num_nodes, cache_len, head_dim, scale, *, batch_size=1,
                       block_tables=None, cache_lens=None, cache_stride=0, block_size=16,
                       max_blocks_per_seq=0, num_blocks=0, q_dtype=0) -> None:
        a = TreeAttentionArgs(_ptr(Q), _ptr(K_cache), _ptr(V_cache), _ptr(K_tree), _ptr(V_tree),
                              _ptr(parent_indices), _ptr(block_tables), _ptr(cache_lens), _ptr(output),
                              batch_size, num_heads, num_kv_heads, num_nodes, cache_len, head_dim,
                              cache_stride, block_size, max_blocks_per_seq, num_blocks, q_dtype, scale)
        check(lib.granite_cuda_attention_tree(self._h, C.byref(a)))

    def kv_cache_append(self, cache_k, cache_v, new_k, new_v, num_kv_heads, head_dim, current_len,
                        new_len, max_seq_len) -> None:
        a = KvAppendArgs(_ptr(cache_k), _ptr(cache_v), _ptr(new_k), _ptr(new_v), num_kv_heads, head_dim,
                         current_len, new_len, max_seq_len)
        check(lib.granite_cuda_kv_cache_append(self._h, C.byref(a)))

    def paged_kv_cache_append(self, new_k, new_v, K_cache, V_cache, block_table, num_kv_heads, head_dim,
                              start_pos, new_len, block_size, *, num_blocks, table_len, positions=None,
                              batch_size=0) -> None:
        a = PagedKvAppendArgs(_ptr(new_k), _ptr(new_v), _ptr(K_cache), _ptr(V_cache), _ptr(block_table),
                              _ptr(positions), num_kv_heads, head_dim, start_pos, new_len, block_size,
                              num_blocks, table_len, batch_size)
        check(lib.granite_cuda_paged_kv_cache_append(self._h, C.byref(a)))

    def rope_table_create(self, max_seq_len: int, head_dim: int, theta: float = 10000.0) -> tuple[int, int]:
        """Device addresses of the cos and sin tables [max_seq_len, head_dim/2] (free with destroy_buffer)."""
        cos, sin = C.c_void_p(), C.c_void_p()
        check(lib.granite_cuda_rope_table_create(self._h, max_seq_len, head_dim, theta, C.byref(cos), C.byref(sin)))
        return cos.value, sin.value

    def rope_multihead(self, q, k, num_heads_q, num_heads_k, seq_len, head_dim, start_pos, cos_table, sin_table,
                       table_len) -> None:
        check(lib.granite_cuda_rope_multihead(self._h, C.c_void_p(_ptr(q)), C.c_void_p(_ptr(k)), num_heads_q,
                                              num_heads_k, seq_len, head_dim, start_pos,
                                              C.c_void_p(_ptr(cos_table)), C.c_void_p(_ptr(sin_table)), table_len))

    def rope_paged_kv_cache_append(self, q, k, v, cos_table, sin_table, K_cache, V_cache, block_tables, positions,
                                   batch_size, new_len, num_heads, num_kv_heads, head_dim, block_size,
                                   max_blocks_per_seq, num_blocks, table_len, start_pos=0) -> None:
        a = RopeAppendArgs(_ptr(q), _ptr(k), _ptr(v), _ptr(cos_table), _ptr(sin_table), _ptr(K_cache),
                           _ptr(V_cache), _ptr(block_tables), _ptr(positions), batch_size, new_len, num_heads,
                           num_kv_heads, head_dim, block_size, max_blocks_per_seq, num_blocks, table_len, start_pos)
        check(lib.granite_cuda_rope_paged_kv_cache_append(self._h, C.byref(a)))

    def tree_commit(self, K_tree, V_tree, K_cache, V_cache, block_tables, cache_lens, accepted, num_accepted,
                    batch_size, num_nodes, max_accepted, num_kv_heads, head_dim, block_size, max_blocks_per_seq,
                    num_blocks) -> None:
        a = TreeCommitArgs(_ptr(K_tree), _ptr(V_tree), _ptr(K_cache), _ptr(V_cache), _ptr(block_tables),
                           _ptr(cache_lens), _ptr(accepted), _ptr(num_accepted), batch_size, num_nodes,
                           max_accepted, num_kv_heads, head_dim, block_size, max_blocks_per_seq, num_blocks)
        check(lib.granite_cuda_tree_commit(self._h, C.byref(a)))

    def paged_prefill_attention(self, Q, K_cache, V_cache, block_table, output, num_heads, num_kv_heads, seq_q,
                                start_pos, head_dim, block_size, max_blocks_per_seq, num_blocks, scale,
                                q_dtype=0, out_dtype=0) -> None:
        a = PagedPrefillArgs(_ptr(Q), _ptr(K_cache), _ptr(V_cache), _ptr(block_table), _ptr(output), num_heads,
                             num_kv_heads, seq_q, start_pos, head_dim, block_size, max_blocks_per_seq, num_blocks,
                             q_dtype, out_dtype, scale)
        check(lib.granite_cuda_paged_prefill_attention(self._h, C.byref(a)))

    def selftest_bounded_wait(self, limit_cycles: int, released_early) -> None:
        check(lib.granite_cuda_selftest_bounded_wait(self._h, limit_cycles, C.c_void_p(_ptr(released_early))))

    def push_rows(self, src, dst_ptrs, dst_offset_bytes: int, nbytes: int, stream: int | None = None) -> None:
        """Stores `nbytes` bytes of `src` at every address in `dst_ptrs` (+ offset): local or peer-mapped buffers."""
        arr = (C.c_void_p * len(dst_ptrs))(*[_ptr(d) for d in dst_ptrs])
        check(lib.granite_cuda_push_rows(self._h, C.c_void_p(stream or 0), C.c_void_p(_ptr(src)), arr, len(dst_ptrs),
                                         dst_offset_bytes, nbytes))

    def build_tree_mask(self, parent_indices, masks, batch_size, num_nodes) -> None:
        check(lib.granite_cuda_build_tree_mask(self._h, C.c_void_p(_ptr(parent_indices)),
                                               C.c_void_p(_ptr(masks)), batch_size, num_nodes))


def batched_paged_attention_decode_static(Q, K_cache, V_cache, block_tables, seq_lens, output, batch_size,
                                          num_heads, num_kv_heads, head_dim, block_size, max_blocks_per_seq,
                                          scale, *, num_blocks, stream: int = 0, device_status=None,
                                          seq_len: int = 0) -> None:
    """The allocation-free paged decode: for hosts that own all device memory themselves or cannot
    tolerate cudaMalloc's device-wide synchronisation.  Needs no compute object; runs on the current
    device and on `stream`; scratch is a fixed array inside the library (batch <= 4096, heads <= 64).
    Calls that overlap on one GPU race on that array - serialise them."""
    a = PagedDecodeArgs(_ptr(Q), _ptr(K_cache), _ptr(V_cache), _ptr(block_tables), _ptr(seq_lens),
                        _ptr(output), batch_size, num_heads, num_kv_heads, head_dim, block_size,
                        max_blocks_per_seq, num_blocks, seq_len, scale)
    check(lib.granite_cuda_batched_paged_attention_decode_static(C.byref(a), C.c_void_p(stream),
                                                                 C.c_void_p(_ptr(device_status))))
