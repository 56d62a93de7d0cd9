// RoPE, the fused RoPE + paged K/V write, and the tree commit copy: the cache-writing steps on
// either side of the attention kernels.  All three are small byte-bound kernels (a decode step of
// 64 sequences moves under 2 MB); the point of the fusion is one launch and no round trip of the
// rotated K through HBM instead of three launches
// (rope_multihead -> paged_kv_cache_append, src/llm/transformer.mm:2975-2986).
//
// Arithmetic follows the CPU path results are checked against (src/llm/rope.cpp:52-86): tables of
// cos/sin per (position, pair) built on the host, adjacent pairs (2i, 2i+1), both products of each
// output rounded separately (__fmul_rn / __fsub_rn / __fadd_rn keep the compiler from fusing them),
// then the truncating fp32 -> fp16 cast of src/llm/math_ops.cpp:45-54 for what goes into the cache.
#include "compute_internal.h"
#include "ptx.cuh"

namespace gb200 {

namespace {

__device__ __forceinline__ unsigned short trunc_f16(float f) {
    const unsigned int bits = __float_as_uint(f);
    const unsigned int sign = (bits >> 16) & 0x8000u;
    const int exp = (int)((bits >> 23) & 0xFFu) - 127 + 15;
    const unsigned int mant = (bits >> 13) & 0x3FFu;
    if (exp <= 0) return (unsigned short)sign;
    if (exp >= 31) return (unsigned short)(sign | 0x7C00u);
    return (unsigned short)(sign | ((unsigned int)exp << 10) | mant);
}

// two adjacent pairs (elements 4u .. 4u+3 of a head) rotated with their two table entries
__device__ __forceinline__ float4 rotate4(float4 x, float2 c, float2 s) {
    float4 r;
    r.x = __fsub_rn(__fmul_rn(x.x, c.x), __fmul_rn(x.y, s.x));
    r.y = __fadd_rn(__fmul_rn(x.x, s.x), __fmul_rn(x.y, c.x));
    r.z = __fsub_rn(__fmul_rn(x.z, c.y), __fmul_rn(x.w, s.y));
    r.w = __fadd_rn(__fmul_rn(x.z, s.y), __fmul_rn(x.w, c.y));
    return r;
}

__device__ __forceinline__ uint2 narrow4(float4 x) {
    uint2 r;
    r.x = (unsigned)trunc_f16(x.x) | ((unsigned)trunc_f16(x.y) << 16);
    r.y = (unsigned)trunc_f16(x.z) | ((unsigned)trunc_f16(x.w) << 16);
    return r;
}

struct RopeAppendParams {
    float* q;
    const float* k;
    const float* v;
    float* k_inplace;  // rotate-only form: k is written back instead of being stored in the cache
    const float* cos_t;
    const float* sin_t;
    unsigned short* k_pool;
    unsigned short* v_pool;
    const int* tables;
    const int* positions;
    int batch, new_len, hq, hkv, head_dim, block_size, max_blocks, num_blocks, table_len, start_pos;
    int* status;
};

// One thread per group of four consecutive elements of one head of one token; the heads of a
// token are laid out as [Hq query heads | Hkv key heads | Hkv value heads] in the work index, so
// neighbouring threads read and write neighbouring 16-byte pieces.
__global__ void rope_paged_append_kernel(RopeAppendParams p) {
    const int quads = p.head_dim / 4;
    const int heads_per_token = (p.q ? p.hq : 0) + p.hkv + (p.v ? p.hkv : 0);
    const size_t total = (size_t)p.batch * p.new_len * heads_per_token * quads;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int u = (int)(i % quads);
        int hh = (int)((i / quads) % heads_per_token);
        const size_t token = i / ((size_t)quads * heads_per_token);  // b * new_len + s
        const int b = (int)(token / p.new_len), s = (int)(token % p.new_len);
        const int pos = (p.positions ? p.positions[b] : p.start_pos) + s;
        if (pos < 0 || pos >= p.table_len) {
            if (u == 0 && hh == 0) atomicOr(p.status, kStatusBadSeqLen);
            continue;
        }
        size_t cache_row = 0;
        if (p.k_pool) {
            const int logical = pos / p.block_size;
            if (logical >= p.max_blocks) {
                if (u == 0 && hh == 0) atomicOr(p.status, kStatusBadSeqLen);
                continue;
            }
            const int phys = p.tables[(size_t)b * p.max_blocks + logical];
            if (phys < 0 || phys >= p.num_blocks) {
                if (u == 0 && hh == 0) atomicOr(p.status, kStatusBadTable);
                continue;
            }
            cache_row = (size_t)phys * p.block_size + pos % p.block_size;
        }
        const size_t trig = (size_t)pos * (p.head_dim / 2) + 2 * u;
        if (p.q && hh < p.hq) {
            float4* x = reinterpret_cast<float4*>(p.q + (token * p.hq + hh) * p.head_dim) + u;
            *x = rotate4(*x, *reinterpret_cast<const float2*>(p.cos_t + trig), *reinterpret_cast<const float2*>(p.sin_t + trig));
            continue;
        }
        if (p.q) hh -= p.hq;
        if (hh < p.hkv) {
            const float4 x = *(reinterpret_cast<const float4*>(p.k + (token * p.hkv + hh) * p.head_dim) + u);
            const float4 r = rotate4(x, *reinterpret_cast<const float2*>(p.cos_t + trig), *reinterpret_cast<const float2*>(p.sin_t + trig));
            if (p.k_pool)
                *(reinterpret_cast<uint2*>(p.k_pool + (cache_row * p.hkv + hh) * p.head_dim) + u) = narrow4(r);
            else
                *(reinterpret_cast<float4*>(p.k_inplace + (token * p.hkv + hh) * p.head_dim) + u) = r;
            continue;
        }
        hh -= p.hkv;
        const float4 x = *(reinterpret_cast<const float4*>(p.v + (token * p.hkv + hh) * p.head_dim) + u);
        *(reinterpret_cast<uint2*>(p.v_pool + (cache_row * p.hkv + hh) * p.head_dim) + u) = narrow4(x);
    }
}

struct TreeCommitParams {
    const uint4* k_tree;
    const uint4* v_tree;
    uint4* k_pool;
    uint4* v_pool;
    const int* tables;
    const int* cache_lens;
    const int* accepted;
    const int* num_accepted;
    int batch, num_nodes, max_accepted, hkv, row_vecs /* head_dim * 2 / 16 */, block_size, max_blocks, num_blocks;
    int* status;
};

// One thread per 16 bytes of one (sequence, accepted slot, KV head) row.
__global__ void tree_commit_kernel(TreeCommitParams p) {
    const size_t total = (size_t)p.batch * p.max_accepted * p.hkv * p.row_vecs;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int u = (int)(i % p.row_vecs);
        const int h = (int)((i / p.row_vecs) % p.hkv);
        const int j = (int)((i / ((size_t)p.row_vecs * p.hkv)) % p.max_accepted);
        const int b = (int)(i / ((size_t)p.row_vecs * p.hkv * p.max_accepted));
        int n_acc = p.num_accepted[b];
        if (n_acc < 0 || n_acc > p.max_accepted) {
            if (u == 0 && h == 0 && j == 0) atomicOr(p.status, kStatusBadSeqLen);
            n_acc = 0;
        }
        if (j >= n_acc) continue;
        const int node = p.accepted[(size_t)b * p.max_accepted + j];
        if (node < 0 || node >= p.num_nodes) {
            if (u == 0 && h == 0) atomicOr(p.status, kStatusBadParent);
            continue;
        }
        const int pos = p.cache_lens[b] + j;
        const int logical = pos / p.block_size;
        if (pos < 0 || logical >= p.max_blocks) {
            if (u == 0 && h == 0) atomicOr(p.status, kStatusBadSeqLen);
            continue;
        }
        const int phys = p.tables[(size_t)b * p.max_blocks + logical];
        if (phys < 0 || phys >= p.num_blocks) {
            if (u == 0 && h == 0) atomicOr(p.status, kStatusBadTable);
            continue;
        }
        const size_t src = (((size_t)b * p.hkv + h) * p.num_nodes + node) * p.row_vecs + u;
        const size_t dst = (((size_t)phys * p.block_size + pos % p.block_size) * p.hkv + h) * p.row_vecs + u;
        p.k_pool[dst] = p.k_tree[src];
        p.v_pool[dst] = p.v_tree[src];
    }
}

constexpr int kMaxPushDst = 16;
struct PushParams {
    const uint4* src;
    uint4* dst[kMaxPushDst];
    int n_dst;
    size_t n_vec;
};

// Every 16-byte piece of the source is read once and stored to each destination (local or a peer
// GPU's memory mapped into this process): consecutive threads write consecutive pieces, so every
// store instruction of a warp is 512 contiguous bytes on the link.
__global__ void push_rows_kernel(PushParams p) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.n_vec; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 v = p.src[i];
        for (int r = 0; r < p.n_dst; r++) p.dst[r][i] = v;
    }
}

// The bounded wait every pipeline role uses, exercised on purpose: thread 0 waits on a barrier
// that nothing will ever arrive at and gives up after `limit_cycles`; a second waiter with the full
// limit must be released early by the abort flag the first one raises.  Ends by itself.
__global__ void bounded_wait_selftest_kernel(int* status, long long limit_cycles, int* released_early) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if ((threadIdx.x & 31) != 0) return;
    const long long t0 = clock64();
    const bool ok = mbar_wait(&bar, 0, &abort_flag, threadIdx.x == 0 ? limit_cycles : kWaitCycleLimit);
    if (threadIdx.x == 0) {
        if (!ok) atomicOr(status, kStatusTimeout);
    } else {
        *released_early = (!ok && clock64() - t0 < 4 * limit_cycles + 1000000) ? 1 : 0;
    }
}

unsigned grid_for(size_t total, int sm_count) {
    size_t blocks = (total + 255) / 256;
    const size_t cap = (size_t)sm_count * 8;
    return (unsigned)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

}  // namespace

int launch_rope_multihead(granite_cuda_compute* c, float* q, float* k, uint32_t hq, uint32_t hk, uint32_t seq_len,
                          uint32_t head_dim, uint32_t start_pos, const float* cos_t, const float* sin_t, uint32_t table_len) {
    if (!q || !cos_t || !sin_t) return fail(GRANITE_CUDA_NULL_POINTER, "rope_multihead: null buffer");
    if (seq_len == 0) return GRANITE_CUDA_SUCCESS;
    if (head_dim == 0 || head_dim % 4 != 0 || hq == 0) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "rope_multihead: head_dim must be a multiple of 4");
    if ((uint64_t)start_pos + seq_len > table_len)  // rope.cpp:34-38
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "rope_multihead: RoPE position out of range");
    RopeAppendParams p{};
    p.q = q;
    p.k = k;
    p.k_inplace = k;
    p.cos_t = cos_t;
    p.sin_t = sin_t;
    p.batch = 1;
    p.new_len = (int)seq_len;
    p.hq = (int)hq;
    p.hkv = k ? (int)hk : 0;
    p.head_dim = (int)head_dim;
    p.table_len = (int)table_len;
    p.start_pos = (int)start_pos;
    p.status = c->d_status;
    const size_t total = (size_t)seq_len * (hq + p.hkv) * (head_dim / 4);
    LaunchScope t(c, "rope_multihead");
    rope_paged_append_kernel<<<grid_for(total, c->sm_count), 256, 0, c->stream>>>(p);
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

int launch_rope_paged_append(granite_cuda_compute* c, const GraniteCudaRopeAppendArgs& a) {
    if (!a.k || !a.v || !a.cos_table || !a.sin_table || !a.k_cache || !a.v_cache || !a.block_tables)
        return fail(GRANITE_CUDA_NULL_POINTER, "rope_paged_kv_cache_append: null buffer");
    if (a.batch_size == 0 || a.new_len == 0) return GRANITE_CUDA_SUCCESS;
    if (a.head_dim == 0 || a.head_dim % 4 != 0 || a.num_kv_heads == 0 || a.block_size == 0 || a.num_blocks == 0 ||
        a.max_blocks_per_seq == 0 || (a.q && a.num_heads == 0))
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "rope_paged_kv_cache_append: empty shape or head_dim not a multiple of 4");
    RopeAppendParams p{};
    p.q = a.q;
    p.k = a.k;
    p.v = a.v;
    p.cos_t = a.cos_table;
    p.sin_t = a.sin_table;
    p.k_pool = static_cast<unsigned short*>(a.k_cache);
    p.v_pool = static_cast<unsigned short*>(a.v_cache);
    p.tables = a.block_tables;
    p.positions = a.positions;
    p.batch = (int)a.batch_size;
    p.new_len = (int)a.new_len;
    p.hq = (int)a.num_heads;
    p.hkv = (int)a.num_kv_heads;
    p.head_dim = (int)a.head_dim;
    p.block_size = (int)a.block_size;
    p.max_blocks = (int)a.max_blocks_per_seq;
    p.num_blocks = (int)a.num_blocks;
    p.table_len = (int)a.table_len;
    p.start_pos = (int)a.start_pos;
    p.status = c->d_status;
    const size_t total = (size_t)a.batch_size * a.new_len * ((a.q ? a.num_heads : 0) + 2 * a.num_kv_heads) * (a.head_dim / 4);
    LaunchScope t(c, "rope_paged_kv_append");
    rope_paged_append_kernel<<<grid_for(total, c->sm_count), 256, 0, c->stream>>>(p);
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

int launch_tree_commit(granite_cuda_compute* c, const GraniteCudaTreeCommitArgs& a) {
    if (!a.k_tree || !a.v_tree || !a.k_cache || !a.v_cache || !a.block_tables || !a.cache_lens || !a.accepted || !a.num_accepted)
        return fail(GRANITE_CUDA_NULL_POINTER, "tree_commit: null buffer");
    if (a.batch_size == 0 || a.max_accepted == 0) return GRANITE_CUDA_SUCCESS;
    if (a.head_dim == 0 || a.head_dim % 8 != 0 || a.num_kv_heads == 0 || a.block_size == 0 || a.num_blocks == 0 ||
        a.max_blocks_per_seq == 0 || a.num_nodes == 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "tree_commit: empty shape or head_dim not a multiple of 8");
    TreeCommitParams p{};
    p.k_tree = static_cast<const uint4*>(a.k_tree);
    p.v_tree = static_cast<const uint4*>(a.v_tree);
    p.k_pool = static_cast<uint4*>(a.k_cache);
    p.v_pool = static_cast<uint4*>(a.v_cache);
    p.tables = a.block_tables;
    p.cache_lens = a.cache_lens;
    p.accepted = a.accepted;
    p.num_accepted = a.num_accepted;
    p.batch = (int)a.batch_size;
    p.num_nodes = (int)a.num_nodes;
    p.max_accepted = (int)a.max_accepted;
    p.hkv = (int)a.num_kv_heads;
    p.row_vecs = (int)(a.head_dim * 2 / 16);
    p.block_size = (int)a.block_size;
    p.max_blocks = (int)a.max_blocks_per_seq;
    p.num_blocks = (int)a.num_blocks;
    p.status = c->d_status;
    const size_t total = (size_t)a.batch_size * a.max_accepted * a.num_kv_heads * p.row_vecs;
    LaunchScope t(c, "tree_commit");
    tree_commit_kernel<<<grid_for(total, c->sm_count), 256, 0, c->stream>>>(p);
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

int launch_bounded_wait_selftest(granite_cuda_compute* c, uint64_t limit_cycles, int* released_early_dev) {
    if (!released_early_dev) return fail(GRANITE_CUDA_NULL_POINTER, "selftest: null buffer");
    if (limit_cycles == 0 || limit_cycles > 200000000ull)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "selftest: limit must be in [1, 2e8] cycles (about 0.1 s)");
    LaunchScope t(c, "bounded_wait_selftest");
    bounded_wait_selftest_kernel<<<1, 64, 0, c->stream>>>(c->d_status, (long long)limit_cycles, released_early_dev);
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

int launch_push_rows(granite_cuda_compute* c, cudaStream_t stream, const void* src, void* const* dst_ptrs, uint32_t n_dst,
                     uint64_t dst_offset_bytes, uint64_t bytes) {
    if (!src || !dst_ptrs) return fail(GRANITE_CUDA_NULL_POINTER, "push_rows: null buffer");
    if (n_dst == 0 || bytes == 0) return GRANITE_CUDA_SUCCESS;
    if (n_dst > (uint32_t)kMaxPushDst) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "push_rows: at most 16 destinations");
    if ((reinterpret_cast<uintptr_t>(src) | dst_offset_bytes | bytes) & 15)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "push_rows: source, offset and size must be 16-byte aligned");
    PushParams p{};
    p.src = static_cast<const uint4*>(src);
    p.n_dst = (int)n_dst;
    p.n_vec = bytes / 16;
    for (uint32_t r = 0; r < n_dst; r++) {
        if (!dst_ptrs[r]) return fail(GRANITE_CUDA_NULL_POINTER, "push_rows: null destination");
        if (reinterpret_cast<uintptr_t>(dst_ptrs[r]) & 15)
            return fail(GRANITE_CUDA_INVALID_ARGUMENT, "push_rows: destinations must be 16-byte aligned");
        p.dst[r] = reinterpret_cast<uint4*>(static_cast<uint8_t*>(dst_ptrs[r]) + dst_offset_bytes);
    }
    // a small grid without shared memory: it fits on SMs beside a persistent attention CTA
    size_t blocks = (p.n_vec + 255) / 256;
    if (blocks > 64) blocks = 64;
    cudaStream_t st = stream ? stream : c->stream;
    if (st == c->stream) {
        LaunchScope t(c, "push_rows");
        push_rows_kernel<<<(unsigned)blocks, 256, 0, st>>>(p);
    } else {
        push_rows_kernel<<<(unsigned)blocks, 256, 0, st>>>(p);  // timed by the caller's own events
    }
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

}  // namespace gb200
