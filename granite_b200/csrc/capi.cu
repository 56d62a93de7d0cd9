// extern "C" entry points declared in include/granite_cuda.h: compute-object lifecycle, raw
// buffers, and the attention calls.  Errors are values (granite::ErrorCode numbers), never
// exceptions; there is no CPU fallback anywhere below this boundary.
#include <cmath>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "compute_internal.h"

namespace gb200 {

static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }
int fail(int code, const std::string& msg) {
    g_last_error = msg;
    return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is fetched at run time so that the library links (and loads) on
// machines without libcuda; it simply cannot compute there.
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return (EncodeTiledFn) nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

}  // namespace gb200

using namespace gb200;

int granite_cuda_compute::ensure_scratch(size_t bytes) {
    if (bytes <= scratch_bytes) return GRANITE_CUDA_SUCCESS;
    // growing: make sure nothing in flight still uses the old arena
    GB_CUDA_TRY(cudaStreamSynchronize(stream));
    if (scratch) cudaFree(scratch);
    scratch = nullptr;
    scratch_bytes = 0;
    size_t want = bytes + bytes / 4;
    cudaError_t e = cudaMalloc(&scratch, want);
    if (e != cudaSuccess) return fail(GRANITE_CUDA_OUT_OF_MEMORY, "scratch arena: cudaMalloc failed");
    scratch_bytes = want;
    return GRANITE_CUDA_SUCCESS;
}

int granite_cuda_compute::ensure_page_counters(size_t count) {
    if (count <= pages_done_count) return GRANITE_CUDA_SUCCESS;
    GB_CUDA_TRY(cudaStreamSynchronize(stream));  // growing: nothing in flight may still count in the old array
    if (d_pages_done) cudaFree(d_pages_done);
    d_pages_done = nullptr;
    pages_done_count = 0;
    const size_t want = count + count / 4 + 1024;
    if (cudaMalloc(&d_pages_done, want * sizeof(int)) != cudaSuccess)
        return fail(GRANITE_CUDA_OUT_OF_MEMORY, "decode page counters: cudaMalloc failed");
    GB_CUDA_TRY(cudaMemsetAsync(d_pages_done, 0, want * sizeof(int), stream));
    pages_done_count = want;
    return GRANITE_CUDA_SUCCESS;
}

const CUtensorMap* granite_cuda_compute::encode_map(const TensorMapKey& key) {
    const uint64_t tick = ++tensor_map_tick;
    auto it = tensor_maps.find(key);
    if (it != tensor_maps.end()) {
        it->second.last_use = tick;
        return &it->second.map;
    }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return nullptr;
    }
    if ((reinterpret_cast<uintptr_t>(key.base) & 15) != 0 || (key.stride1 & 15) != 0 || (key.stride2 & 15) != 0 ||
        (key.stride3 & 15) != 0) {
        set_error("tensor map: base address and strides must be 16-byte aligned");
        return nullptr;
    }
    CUtensorMap map;
    cuuint64_t dims[4] = {key.dim0, key.dim1, key.dim2, key.dim3};
    cuuint64_t strides[3] = {key.stride1, key.stride2, key.stride3};
    cuuint32_t box[4] = {key.box0, key.box1, key.box2, key.box3};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUtensorMapSwizzle sw = key.swizzle == 128  ? CU_TENSOR_MAP_SWIZZLE_128B
                            : key.swizzle == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                            : key.swizzle == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)key.rank, const_cast<void*>(key.base), dims,
                     strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r));
        return nullptr;
    }
    // Bounded cache.  A launcher holds the pointers of up to six maps while it fetches the next
    // one, so eviction never touches the kKeepRecent most recently used entries; erasing other
    // nodes of a std::map leaves pointers to the remaining ones valid.
    if (tensor_maps.size() >= kMaxTensorMaps) {
        for (auto e = tensor_maps.begin(); e != tensor_maps.end();)
            e = (e->second.last_use + kKeepRecent < tick) ? tensor_maps.erase(e) : std::next(e);
    }
    auto ins = tensor_maps.emplace(key, CachedTensorMap{map, tick});
    return &ins.first->second.map;
}

const CUtensorMap* granite_cuda_compute::tensor_map_2d(const void* base, uint64_t dim0, uint64_t dim1,
                                                       uint64_t stride1_bytes, uint32_t box0,
                                                       uint32_t box1, int swizzle_bytes) {
    return encode_map(TensorMapKey{base, dim0, dim1, 0, stride1_bytes, 0, box0, box1, 0, swizzle_bytes, 2});
}

const CUtensorMap* granite_cuda_compute::tensor_map_3d(const void* base, uint64_t dim0, uint64_t dim1,
                                                       uint64_t dim2, uint64_t stride1_bytes,
                                                       uint64_t stride2_bytes, uint32_t box0, uint32_t box1,
                                                       uint32_t box2, int swizzle_bytes) {
    return encode_map(TensorMapKey{base, dim0, dim1, dim2, stride1_bytes, stride2_bytes, box0, box1, box2,
                                   swizzle_bytes, 3});
}

const CUtensorMap* granite_cuda_compute::tensor_map_pages(const void* base, uint32_t head_dim, uint64_t rows,
                                                          uint64_t row_stride_bytes, uint64_t heads,
                                                          uint64_t head_stride_bytes, uint32_t rows_per_box,
                                                          uint32_t tile_heads) {
    TensorMapKey key{base, 64, rows, head_dim / 64, row_stride_bytes, 128, 64, rows_per_box, head_dim / 64, 128, 4};
    key.dim3 = heads;
    key.stride3 = head_stride_bytes;
    key.box3 = tile_heads;
    return encode_map(key);
}

const CUtensorMap* granite_cuda_compute::tensor_map_page_groups(const void* base, uint64_t width, uint64_t rows,
                                                                uint32_t head_dim) {
    TensorMapKey key{base, width, 8, head_dim / 64, width * 2, 128, 64, 8, head_dim / 64, 128, 4};
    key.dim3 = rows / 8;
    key.stride3 = width * 2 * 8;
    key.box3 = 2;
    return encode_map(key);
}

cudaEvent_t granite_cuda_compute::take_event() {
    if (!event_pool.empty()) {
        cudaEvent_t e = event_pool.back();
        event_pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

void granite_cuda_compute::resolve_timings() {
    for (auto& t : pending_timings) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, t.begin, t.end) == cudaSuccess) {
            auto& st = kernel_stats[t.name];
            st.ms += ms;
            st.dispatches++;
        } else {
            cudaGetLastError();
        }
        event_pool.push_back(t.begin);
        event_pool.push_back(t.end);
    }
    pending_timings.clear();
}

extern "C" {

const char* granite_cuda_last_error_message(void) { return g_last_error.c_str(); }

int granite_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int granite_cuda_compute_create(int device, void* stream, granite_cuda_compute_t** out) {
    if (!out) return fail(GRANITE_CUDA_NULL_POINTER, "compute_create: out is null");
    *out = nullptr;
    int n = granite_cuda_device_count();
    if (n <= 0) return fail(GRANITE_CUDA_BACKEND_NOT_INITIALIZED, "no CUDA device is visible; this backend has no CPU fallback");
    if (device < 0 || device >= n) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "compute_create: device index out of range");
    GB_CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    GB_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(GRANITE_CUDA_BACKEND_NOT_SUPPORTED,
                    std::string("this library is built for sm_100a only; device is ") + prop.name);
    auto* c = new (std::nothrow) granite_cuda_compute();
    if (!c) return fail(GRANITE_CUDA_OUT_OF_MEMORY, "compute_create: host allocation failed");
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    c->smem_optin = (int)prop.sharedMemPerBlockOptin;
    if (stream) {
        c->stream = static_cast<cudaStream_t>(stream);
    } else {
        if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) {
            delete c;
            return fail(GRANITE_CUDA_EXECUTION_FAILED, "compute_create: cudaStreamCreate failed");
        }
        c->owns_stream = true;
    }
    if (cudaMalloc(&c->d_status, kStatusBlockBytes) != cudaSuccess ||
        cudaMallocHost(&c->h_status, sizeof(int)) != cudaSuccess ||
        cudaMemsetAsync(c->d_status, 0, kStatusBlockBytes, c->stream) != cudaSuccess) {
        granite_cuda_compute_destroy(c);
        return fail(GRANITE_CUDA_OUT_OF_MEMORY, "compute_create: status word allocation failed");
    }
    *c->h_status = 0;
    c->d_direct_done = reinterpret_cast<unsigned*>(c->d_status + 64);
    *out = c;
    return GRANITE_CUDA_SUCCESS;
}

void granite_cuda_compute_destroy(granite_cuda_compute_t* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    c->resolve_timings();
    for (cudaEvent_t e : c->event_pool) cudaEventDestroy(e);
    if (c->scratch) cudaFree(c->scratch);
    if (c->d_status) cudaFree(c->d_status);
    if (c->d_pages_done) cudaFree(c->d_pages_done);
    if (c->h_status) cudaFreeHost(c->h_status);
    if (c->owns_stream && c->stream) cudaStreamDestroy(c->stream);
    delete c;
}

void* granite_cuda_compute_stream(granite_cuda_compute_t* c) { return c ? c->stream : nullptr; }
int granite_cuda_compute_sm_count(granite_cuda_compute_t* c) { return c ? c->sm_count : 0; }

int granite_cuda_sync(granite_cuda_compute_t* c) {
    if (!c) return fail(GRANITE_CUDA_NULL_POINTER, "sync: compute object is null");
    c->syncs++;
    GB_CUDA_TRY(cudaMemcpyAsync(c->h_status, c->d_status, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
    GB_CUDA_TRY(cudaStreamSynchronize(c->stream));
    c->resolve_timings();
    int st = *c->h_status;
    if (st == 0) return GRANITE_CUDA_SUCCESS;
    // (a launch that gave up may have left arrival counters of the one-launch decode half counted)
    GB_CUDA_TRY(cudaMemsetAsync(c->d_status, 0, kStatusBlockBytes, c->stream));
    if (c->d_pages_done) GB_CUDA_TRY(cudaMemsetAsync(c->d_pages_done, 0, c->pages_done_count * sizeof(int), c->stream));
    if (st & kStatusTimeout) return fail(GRANITE_CUDA_TIMEOUT, "a device-side wait ran out (status " + std::to_string(st) + ")");
    if (st & kStatusBadTable) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "a block-table entry was outside the pool");
    if (st & kStatusBadSeqLen) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "a sequence length was negative or exceeded its block table");
    if (st & kStatusBadParent) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "a tree parent index was out of range");
    if (st & kStatusLayout) return fail(GRANITE_CUDA_INTERNAL_ERROR, "a kernel's shared-memory layout did not fit its window");
    return fail(GRANITE_CUDA_EXECUTION_FAILED, "device status " + std::to_string(st));
}

void granite_cuda_get_profiling_stats(granite_cuda_compute_t* c, uint64_t* dispatches, uint64_t* syncs) {
    if (dispatches) *dispatches = c ? c->dispatches : 0;
    if (syncs) *syncs = c ? c->syncs : 0;
}

void granite_cuda_enable_kernel_timing(granite_cuda_compute_t* c, int enable) {
    if (c) c->kernel_timing = enable != 0;
}

void granite_cuda_reset_kernel_timing(granite_cuda_compute_t* c) {
    if (!c) return;
    cudaStreamSynchronize(c->stream);
    c->resolve_timings();
    c->kernel_stats.clear();
}

int granite_cuda_get_kernel_timing_stats(granite_cuda_compute_t* c, GraniteCudaKernelTiming* out, int capacity) {
    if (!c) return 0;
    cudaStreamSynchronize(c->stream);
    c->resolve_timings();
    int n = 0;
    for (auto& kv : c->kernel_stats) {
        if (out && n < capacity) {
            std::strncpy(out[n].name, kv.first.c_str(), sizeof(out[n].name) - 1);
            out[n].name[sizeof(out[n].name) - 1] = 0;
            out[n].gpu_time_ms = kv.second.ms;
            out[n].dispatches = kv.second.dispatches;
        }
        n++;
    }
    return n;
}

int granite_cuda_malloc(granite_cuda_compute_t* c, size_t bytes, void** dev_ptr) {
    if (!c || !dev_ptr) return fail(GRANITE_CUDA_NULL_POINTER, "malloc: null argument");
    *dev_ptr = nullptr;
    if (bytes == 0) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "malloc: zero bytes");
    cudaSetDevice(c->device);
    if (cudaMalloc(dev_ptr, bytes) != cudaSuccess) {
        cudaGetLastError();
        return fail(GRANITE_CUDA_OUT_OF_MEMORY, "cudaMalloc of " + std::to_string(bytes) + " bytes failed");
    }
    return GRANITE_CUDA_SUCCESS;
}

int granite_cuda_free(granite_cuda_compute_t* c, void* dev_ptr) {
    if (!c) return fail(GRANITE_CUDA_NULL_POINTER, "free: compute object is null");
    if (!dev_ptr) return GRANITE_CUDA_SUCCESS;
    // tensor maps that point into the buffer are dropped with it
    for (auto it = c->tensor_maps.begin(); it != c->tensor_maps.end();)
        it = (it->first.base == dev_ptr) ? c->tensor_maps.erase(it) : std::next(it);
    GB_CUDA_TRY(cudaStreamSynchronize(c->stream));
    GB_CUDA_TRY(cudaFree(dev_ptr));
    return GRANITE_CUDA_SUCCESS;
}

int granite_cuda_malloc_host(size_t bytes, void** host_ptr) {
    if (!host_ptr) return fail(GRANITE_CUDA_NULL_POINTER, "malloc_host: null argument");
    *host_ptr = nullptr;
    if (cudaMallocHost(host_ptr, bytes) != cudaSuccess) {
        cudaGetLastError();
        return fail(GRANITE_CUDA_OUT_OF_MEMORY, "cudaMallocHost failed");
    }
    return GRANITE_CUDA_SUCCESS;
}

int granite_cuda_free_host(void* host_ptr) {
    if (host_ptr) GB_CUDA_TRY(cudaFreeHost(host_ptr));
    return GRANITE_CUDA_SUCCESS;
}

int granite_cuda_write_buffer(granite_cuda_compute_t* c, void* dev_dst, const void* host_src, size_t bytes) {
    if (!c || !dev_dst || !host_src) return fail(GRANITE_CUDA_NULL_POINTER, "write_buffer: null argument");
    GB_CUDA_TRY(cudaMemcpyAsync(dev_dst, host_src, bytes, cudaMemcpyHostToDevice, c->stream));
    return GRANITE_CUDA_SUCCESS;
}

int granite_cuda_read_buffer(granite_cuda_compute_t* c, void* host_dst, const void* dev_src, size_t bytes) {
    if (!c || !host_dst || !dev_src) return fail(GRANITE_CUDA_NULL_POINTER, "read_buffer: null argument");
    GB_CUDA_TRY(cudaMemcpyAsync(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost, c->stream));
    return GRANITE_CUDA_SUCCESS;
}

int granite_cuda_copy_buffer(granite_cuda_compute_t* c, void* dev_dst, const void* dev_src, size_t bytes) {
    if (!c || !dev_dst || !dev_src) return fail(GRANITE_CUDA_NULL_POINTER, "copy_buffer: null argument");
    GB_CUDA_TRY(cudaMemcpyAsync(dev_dst, dev_src, bytes, cudaMemcpyDeviceToDevice, c->stream));
    return GRANITE_CUDA_SUCCESS;
}

int granite_cuda_memset(granite_cuda_compute_t* c, void* dev_dst, int byte, size_t bytes) {
    if (!c || !dev_dst) return fail(GRANITE_CUDA_NULL_POINTER, "memset: null argument");
    GB_CUDA_TRY(cudaMemsetAsync(dev_dst, byte, bytes, c->stream));
    return GRANITE_CUDA_SUCCESS;
}

int granite_cuda_batched_paged_attention_decode(granite_cuda_compute_t* c, const GraniteCudaPagedDecodeArgs* args) {
    if (!c || !args) return fail(GRANITE_CUDA_NULL_POINTER, "paged decode: null argument");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    return launch_paged_decode(c, *args, false, 0);
}

int granite_cuda_batched_paged_attention_decode_gather(granite_cuda_compute_t* c, const GraniteCudaPagedDecodeArgs* args,
                                                       void* const* dst_ptrs, uint32_t n_dst, uint64_t dst_row_offset) {
    if (!c || !args) return fail(GRANITE_CUDA_NULL_POINTER, "paged decode: null argument");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    const DecodeGather g{dst_ptrs, n_dst, dst_row_offset};
    return launch_paged_decode(c, *args, false, 0, &g);
}

int granite_cuda_batched_paged_attention_decode_gather_heads(granite_cuda_compute_t* c, const GraniteCudaPagedDecodeArgs* args,
                                                             void* const* dst_ptrs, uint32_t n_dst, uint64_t dst_row_offset,
                                                             uint32_t dst_num_heads, uint32_t dst_head_offset) {
    if (!c || !args) return fail(GRANITE_CUDA_NULL_POINTER, "paged decode: null argument");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    const DecodeGather g{dst_ptrs, n_dst, dst_row_offset, dst_num_heads, dst_head_offset};
    return launch_paged_decode(c, *args, false, 0, &g);
}

int granite_cuda_multihead_attention(granite_cuda_compute_t* c, const GraniteCudaAttentionArgs* a) {
    if (!c || !a) return fail(GRANITE_CUDA_NULL_POINTER, "multihead_attention: null argument");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    const uint32_t max_seq = a->max_seq ? a->max_seq : a->seq_kv;
    if (a->seq_q == 1) {
        if (a->q_dtype != 0 || a->out_dtype != 0)
            return fail(GRANITE_CUDA_INVALID_ARGUMENT, "decode takes fp32 Q and writes fp32");
        if (a->seq_kv > max_seq) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "seq_kv exceeds max_seq");
        GraniteCudaPagedDecodeArgs d{};
        d.q = static_cast<const float*>(a->q);
        d.k_cache = a->k;
        d.v_cache = a->v;
        d.output = static_cast<float*>(a->output);
        d.batch_size = a->batch_size ? a->batch_size : 1;
        d.num_heads = a->num_heads;
        d.num_kv_heads = a->num_kv_heads;
        d.head_dim = a->head_dim;
        d.block_size = 16;
        d.seq_len = a->seq_kv;
        d.scale = a->scale;
        return launch_paged_decode(c, d, true, max_seq);
    }
    return launch_prefill(c, *a);
}

int granite_cuda_sdpa(granite_cuda_compute_t* c, const GraniteCudaSdpaArgs* args) {
    if (!c || !args) return fail(GRANITE_CUDA_NULL_POINTER, "sdpa: null argument");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    return launch_sdpa_operator(c, *args);
}

int granite_cuda_kv_cache_append(granite_cuda_compute_t* c, const GraniteCudaKvAppendArgs* args) {
    if (!c || !args) return fail(GRANITE_CUDA_NULL_POINTER, "kv_cache_append: null argument");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    return launch_kv_cache_append(c, *args);
}

int granite_cuda_paged_kv_cache_append(granite_cuda_compute_t* c, const GraniteCudaPagedKvAppendArgs* args) {
    if (!c || !args) return fail(GRANITE_CUDA_NULL_POINTER, "paged_kv_cache_append: null argument");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    return launch_paged_kv_cache_append(c, *args);
}

int granite_cuda_rope_table_create(granite_cuda_compute_t* c, uint32_t max_seq_len, uint32_t head_dim, float theta,
                                   float** cos_table, float** sin_table) {
    if (!c || !cos_table || !sin_table) return fail(GRANITE_CUDA_NULL_POINTER, "rope_table_create: null argument");
    if (max_seq_len == 0 || head_dim < 2 || head_dim % 2 != 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "rope_table_create: head_dim must be even and max_seq_len positive");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    // Host arithmetic on purpose: the tables must carry the bits of the CPU path's own
    // float pow / cos / sin (src/llm/rope.cpp:13-20), which device intrinsics do not promise.
    const size_t half_dim = head_dim / 2, n = (size_t)max_seq_len * half_dim;
    std::vector<float> inv_freq(half_dim), cos_h(n), sin_h(n);
    for (size_t i = 0; i < half_dim; i++)
        inv_freq[i] = 1.0f / std::pow(theta, static_cast<float>(2 * i) / static_cast<int>(head_dim));
    for (size_t pos = 0; pos < max_seq_len; pos++)
        for (size_t i = 0; i < half_dim; i++) {
            const float angle = static_cast<float>(pos) * inv_freq[i];
            cos_h[pos * half_dim + i] = std::cos(angle);
            sin_h[pos * half_dim + i] = std::sin(angle);
        }
    float *cos_d = nullptr, *sin_d = nullptr;
    cudaError_t e = cudaMalloc(&cos_d, n * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&sin_d, n * sizeof(float));
    if (e == cudaSuccess) e = cudaMemcpyAsync(cos_d, cos_h.data(), n * sizeof(float), cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(sin_d, sin_h.data(), n * sizeof(float), cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);  // the host vectors go away on return
    if (e != cudaSuccess) {
        cudaFree(cos_d);
        cudaFree(sin_d);
        cudaGetLastError();
        return fail(e == cudaErrorMemoryAllocation ? GRANITE_CUDA_OUT_OF_MEMORY : GRANITE_CUDA_INTERNAL_ERROR,
                    std::string("rope_table_create: ") + cudaGetErrorString(e));
    }
    *cos_table = cos_d;
    *sin_table = sin_d;
    return GRANITE_CUDA_SUCCESS;
}

int granite_cuda_rope_multihead(granite_cuda_compute_t* c, float* q, float* k, uint32_t num_heads_q, uint32_t num_heads_k,
                                uint32_t seq_len, uint32_t head_dim, uint32_t start_pos, const float* cos_table,
                                const float* sin_table, uint32_t table_len) {
    if (!c) return fail(GRANITE_CUDA_NULL_POINTER, "rope_multihead: null argument");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    return launch_rope_multihead(c, q, k, num_heads_q, num_heads_k, seq_len, head_dim, start_pos, cos_table, sin_table, table_len);
}

int granite_cuda_rope_paged_kv_cache_append(granite_cuda_compute_t* c, const GraniteCudaRopeAppendArgs* args) {
    if (!c || !args) return fail(GRANITE_CUDA_NULL_POINTER, "rope_paged_kv_cache_append: null argument");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    return launch_rope_paged_append(c, *args);
}

int granite_cuda_tree_commit(granite_cuda_compute_t* c, const GraniteCudaTreeCommitArgs* args) {
    if (!c || !args) return fail(GRANITE_CUDA_NULL_POINTER, "tree_commit: null argument");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    return launch_tree_commit(c, *args);
}

int granite_cuda_paged_prefill_attention(granite_cuda_compute_t* c, const GraniteCudaPagedPrefillArgs* args) {
    if (!c || !args) return fail(GRANITE_CUDA_NULL_POINTER, "paged_prefill_attention: null argument");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    return launch_paged_prefill(c, *args);
}

int granite_cuda_selftest_bounded_wait(granite_cuda_compute_t* c, uint64_t limit_cycles, int32_t* released_early) {
    if (!c) return fail(GRANITE_CUDA_NULL_POINTER, "selftest: null argument");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    return launch_bounded_wait_selftest(c, limit_cycles, released_early);
}

int granite_cuda_push_rows(granite_cuda_compute_t* c, void* stream, const void* src, void* const* dst_ptrs,
                           uint32_t n_dst, uint64_t dst_offset_bytes, uint64_t bytes) {
    if (!c) return fail(GRANITE_CUDA_NULL_POINTER, "push_rows: null argument");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    return launch_push_rows(c, static_cast<cudaStream_t>(stream), src, dst_ptrs, n_dst, dst_offset_bytes, bytes);
}

int granite_cuda_attention_tree(granite_cuda_compute_t* c, const GraniteCudaTreeAttentionArgs* args) {
    if (!c || !args) return fail(GRANITE_CUDA_NULL_POINTER, "attention_tree: null argument");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    return launch_tree_verify(c, *args);
}

int granite_cuda_build_tree_mask(granite_cuda_compute_t* c, const int32_t* parent_indices, uint64_t* masks,
                                 uint32_t batch_size, uint32_t num_nodes) {
    if (!c) return fail(GRANITE_CUDA_NULL_POINTER, "build_tree_mask: compute object is null");
    GB_CUDA_TRY(cudaSetDevice(c->device));
    return launch_tree_mask(c, parent_indices, masks, batch_size, num_nodes);
}

}  // extern "C"
