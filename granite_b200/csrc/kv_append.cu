// K/V cache writes: scatter freshly projected K/V rows into the contiguous cache or, through the
// block table, into the paged pool, narrowing fp32 to fp16 on the way.
//
// Replaces kv_cache_append_f16 and paged_kv_cache_append
// (src/backend/metal/kernels/metal_shaders_attention.h:102-132, :2142-2176; wrappers
// MetalCompute::kv_cache_append / paged_kv_cache_append, include/granite/metal_compute.h:787-797,
// :887-898).  Source layouts are the kernels' own: [new_len, H, D] for the contiguous cache,
// [H, new_len, D] for the paged pool.  The narrowing follows the CPU path the results are checked
// against - truncation of the mantissa, flush of results below the normal range to signed zero,
// clamp to infinity (src/llm/math_ops.cpp:45-54, used at src/llm/transformer.mm:1681-1691) - so
// the cache bytes are bit-identical to what Granite's CPU attention would read.  (The Metal
// kernels round to nearest instead; the two differ in the last bit.)
#include "compute_internal.h"

namespace gb200 {

__device__ __forceinline__ unsigned short f32_to_f16_trunc(float f) {
    const unsigned int bits = __float_as_uint(f);
    const unsigned int sign = (bits >> 16) & 0x8000u;
    const int exp = (int)((bits >> 23) & 0xFFu) - 127 + 15;
    const unsigned int mant = (bits >> 13) & 0x3FFu;
    if (exp <= 0) return (unsigned short)sign;
    if (exp >= 31) return (unsigned short)(sign | 0x7C00u);
    return (unsigned short)(sign | ((unsigned int)exp << 10) | mant);
}

// grid-stride over new_len * H * D elements, d fastest (coalesced reads and writes of D runs)
__global__ void kv_cache_append_kernel(const float* __restrict__ new_k, const float* __restrict__ new_v,
                                       unsigned short* __restrict__ cache_k, unsigned short* __restrict__ cache_v,
                                       int num_heads, int head_dim, int current_len, int new_len, int max_seq) {
    const size_t total = (size_t)new_len * num_heads * head_dim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(i % head_dim);
        const int h = (int)((i / head_dim) % num_heads);
        const int s = (int)(i / ((size_t)head_dim * num_heads));
        const size_t dst = ((size_t)h * max_seq + current_len + s) * head_dim + d;  // [H, max_seq, D]
        cache_k[dst] = f32_to_f16_trunc(new_k[i]);                                  // src [new_len, H, D]
        cache_v[dst] = f32_to_f16_trunc(new_v[i]);
    }
}

__global__ void paged_kv_cache_append_kernel(const float* __restrict__ new_k, const float* __restrict__ new_v,
                                             unsigned short* __restrict__ pool_k, unsigned short* __restrict__ pool_v,
                                             const int* __restrict__ block_table, int num_kv_heads, int head_dim,
                                             int start_pos, int new_len, int block_size, int num_blocks,
                                             int table_len, int* status) {
    const size_t total = (size_t)new_len * num_kv_heads * head_dim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(i % head_dim);
        const int h = (int)((i / head_dim) % num_kv_heads);
        const int s = (int)(i / ((size_t)head_dim * num_kv_heads));
        const int pos = start_pos + s;
        const int logical = pos / block_size;
        if (logical >= table_len) {
            atomicOr(status, kStatusBadSeqLen);
            continue;
        }
        const int phys = block_table[logical];
        if (phys < 0 || phys >= num_blocks) {
            atomicOr(status, kStatusBadTable);
            continue;
        }
        const size_t src = ((size_t)h * new_len + s) * head_dim + d;                                  // [H, new_len, D]
        const size_t dst = (((size_t)phys * block_size + pos % block_size) * num_kv_heads + h) * head_dim + d;
        pool_k[dst] = f32_to_f16_trunc(new_k[src]);
        pool_v[dst] = f32_to_f16_trunc(new_v[src]);
    }
}

// One new token per sequence (a decode step of a batch): new_k/new_v [B, H, D]; token b goes to
// position positions[b] of sequence b through its row of block_tables.
__global__ void batched_paged_kv_append_kernel(const float* __restrict__ new_k, const float* __restrict__ new_v,
                                               unsigned short* __restrict__ pool_k, unsigned short* __restrict__ pool_v,
                                               const int* __restrict__ block_tables, const int* __restrict__ positions,
                                               int batch, int num_kv_heads, int head_dim, int block_size,
                                               int max_blocks, int num_blocks, int* status) {
    const size_t total = (size_t)batch * num_kv_heads * head_dim;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(i % head_dim);
        const int h = (int)((i / head_dim) % num_kv_heads);
        const int b = (int)(i / ((size_t)head_dim * num_kv_heads));
        const int pos = positions[b];
        const int logical = pos / block_size;
        if (pos < 0 || logical >= max_blocks) {
            atomicOr(status, kStatusBadSeqLen);
            continue;
        }
        const int phys = block_tables[(size_t)b * max_blocks + logical];
        if (phys < 0 || phys >= num_blocks) {
            atomicOr(status, kStatusBadTable);
            continue;
        }
        const size_t dst = (((size_t)phys * block_size + pos % block_size) * num_kv_heads + h) * head_dim + d;
        pool_k[dst] = f32_to_f16_trunc(new_k[i]);
        pool_v[dst] = f32_to_f16_trunc(new_v[i]);
    }
}

static unsigned grid_for(size_t total, int sm_count) {
    size_t blocks = (total + 255) / 256;
    const size_t cap = (size_t)sm_count * 8;
    return (unsigned)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

int launch_kv_cache_append(granite_cuda_compute* c, const GraniteCudaKvAppendArgs& a) {
    if (!a.cache_k || !a.cache_v || !a.new_k || !a.new_v) return fail(GRANITE_CUDA_NULL_POINTER, "kv_cache_append: null buffer");
    if (a.new_len == 0) return GRANITE_CUDA_SUCCESS;
    if (a.num_kv_heads == 0 || a.head_dim == 0) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "kv_cache_append: empty shape");
    if ((uint64_t)a.current_len + a.new_len > a.max_seq_len)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "kv_cache_append: KV cache overflow");  // kv_cache.cpp:60-64
    const size_t total = (size_t)a.new_len * a.num_kv_heads * a.head_dim;
    LaunchScope t(c, "kv_cache_append");
    kv_cache_append_kernel<<<grid_for(total, c->sm_count), 256, 0, c->stream>>>(
        static_cast<const float*>(a.new_k), static_cast<const float*>(a.new_v),
        static_cast<unsigned short*>(a.cache_k), static_cast<unsigned short*>(a.cache_v), (int)a.num_kv_heads,
        (int)a.head_dim, (int)a.current_len, (int)a.new_len, (int)a.max_seq_len);
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

int launch_paged_kv_cache_append(granite_cuda_compute* c, const GraniteCudaPagedKvAppendArgs& a) {
    if (!a.k_cache || !a.v_cache || !a.new_k || !a.new_v || !a.block_table)
        return fail(GRANITE_CUDA_NULL_POINTER, "paged_kv_cache_append: null buffer");
    if (a.block_size == 0 || a.num_blocks == 0 || a.num_kv_heads == 0 || a.head_dim == 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "paged_kv_cache_append: empty shape");
    if (a.positions) {
        if (a.batch_size == 0) return GRANITE_CUDA_SUCCESS;
        const size_t total = (size_t)a.batch_size * a.num_kv_heads * a.head_dim;
        LaunchScope t(c, "batched_paged_kv_append");
        batched_paged_kv_append_kernel<<<grid_for(total, c->sm_count), 256, 0, c->stream>>>(
            static_cast<const float*>(a.new_k), static_cast<const float*>(a.new_v),
            static_cast<unsigned short*>(a.k_cache), static_cast<unsigned short*>(a.v_cache), a.block_table, a.positions,
            (int)a.batch_size, (int)a.num_kv_heads, (int)a.head_dim, (int)a.block_size, (int)a.table_len,
            (int)a.num_blocks, c->d_status);
    } else {
        if (a.new_len == 0) return GRANITE_CUDA_SUCCESS;
        const size_t total = (size_t)a.new_len * a.num_kv_heads * a.head_dim;
        LaunchScope t(c, "paged_kv_cache_append");
        paged_kv_cache_append_kernel<<<grid_for(total, c->sm_count), 256, 0, c->stream>>>(
            static_cast<const float*>(a.new_k), static_cast<const float*>(a.new_v),
            static_cast<unsigned short*>(a.k_cache), static_cast<unsigned short*>(a.v_cache), a.block_table,
            (int)a.num_kv_heads, (int)a.head_dim, (int)a.start_pos, (int)a.new_len, (int)a.block_size,
            (int)a.num_blocks, (int)a.table_len, c->d_status);
    }
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

}  // namespace gb200
