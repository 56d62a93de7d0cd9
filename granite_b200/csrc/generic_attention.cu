// Attention for the shapes the tuned kernels do not take: head_dim other than 128 and 64 (the two
// the reference's GPU path serves, src/backend/metal/metal_compute.mm:2550-2561), page sizes other
// than 16, KV-head counts the decode tiling does not cover.  One plain kernel for
// decode, causal prefill and tree verification over a contiguous or paged cache: fp32 arithmetic
// throughout, one block per (sequence, query row, query head), keys in chunks of 128 with an
// online softmax.  It keeps such models running on the GPU - there is no CPU fallback - at a
// fraction of the tuned kernels' speed; nothing on the benchmarked configurations goes through it.
//
// Arithmetic as in src/llm/transformer.mm:1779-1840 (scores = (q . k) * scale, causal rule
// k_pos > start_pos + q_pos) and :2044-2126 (tree: whole prefix, then the node itself and its
// ancestors, :823-840).
#include "compute_internal.h"
#include "ptx.cuh"

namespace gb200 {

namespace {

constexpr int kGenThreads = 128;
constexpr int kGenMaxDim = 256;

struct GenericParams {
    const void* q;          // fp32 or fp16
    void* out;              // fp32 or fp16
    const __half* k;        // cache: contiguous [batch, Hkv, kv_stride, D] or pool [num_blocks*bs, Hkv, D]
    const __half* v;
    const __half* k_tree;   // [batch, Hkv, N, D] or nullptr
    const __half* v_tree;
    const int* tables;      // [batch, max_blocks] or nullptr (contiguous)
    const int* kv_lens;     // [batch] or nullptr (kv_len for all)
    const int* parents;     // [batch, N] or nullptr
    int q_f16, out_f16, tree_layout;  // tree_layout: q/out [batch, Hq, rows, D], else [batch, rows, Hq, D]
    int batch, q_rows, hq, hkv, d;
    int kv_len, kv_stride, max_blocks, block_size, num_blocks, n_nodes;
    int causal_start;       // >= 0: query row r sees cache keys <= causal_start + r; -1: the whole cache
    float scale;
    int* status;
};

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = red[0];
    for (int w = 1; w < kGenThreads / 32; w++) m = fmaxf(m, red[w]);
    __syncthreads();
    return m;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float m = 0.f;
    for (int w = 0; w < kGenThreads / 32; w++) m += red[w];
    __syncthreads();
    return m;
}

__global__ void __launch_bounds__(kGenThreads) generic_attention_kernel(GenericParams p) {
    __shared__ float s_q[kGenMaxDim];
    __shared__ float s_p[kGenThreads];
    __shared__ const __half* s_vrow[kGenThreads];
    __shared__ float s_red[kGenThreads / 32];
    const int tid = threadIdx.x;
    const int h = blockIdx.y;
    const int b = blockIdx.x / p.q_rows, r = blockIdx.x % p.q_rows;
    const int kvh = h / (p.hq / p.hkv);
    const size_t qo = p.tree_layout ? (((size_t)b * p.hq + h) * p.q_rows + r) * p.d
                                    : (((size_t)b * p.q_rows + r) * p.hq + h) * p.d;
    for (int i = tid; i < p.d; i += kGenThreads)
        s_q[i] = p.q_f16 ? __half2float(static_cast<const __half*>(p.q)[qo + i]) : static_cast<const float*>(p.q)[qo + i];
    __syncthreads();

    int cache_len = p.kv_lens ? p.kv_lens[b] : p.kv_len;
    const int cap = p.tables ? p.max_blocks * p.block_size : p.kv_stride;
    if (cache_len < 0 || cache_len > cap) {
        if (tid == 0) atomicOr(p.status, kStatusBadSeqLen);
        cache_len = 0;
    }
    int visible = cache_len;  // cache keys [0, visible)
    if (p.causal_start >= 0) visible = min(cache_len, p.causal_start + r + 1);
    // tree part: the node's own key and its ancestors' (bit j of the word)
    unsigned long long anc = 0ull;
    if (p.parents) {
        const int* par = p.parents + (size_t)b * p.n_nodes;
        if (par[r] < -1 || par[r] >= p.n_nodes) {
            if (tid == 0) atomicOr(p.status, kStatusBadParent);
        }
        anc = 1ull << r;
        int cur = par[r];
        for (int hops = 0; cur >= 0 && cur < p.n_nodes && hops < p.n_nodes; hops++) {
            anc |= 1ull << cur;
            cur = par[cur];
        }
    }
    const int total = visible + (p.parents ? p.n_nodes : 0);

    float m_run = -INFINITY, l_run = 0.f;
    float acc[kGenMaxDim / kGenThreads] = {0.f, 0.f};  // output dims tid, tid + 128
    for (int base = 0; base < total; base += kGenThreads) {
        // phase 1: thread = key
        const int key = base + tid;
        const __half *krow = nullptr, *vrow = nullptr;
        if (key < visible) {
            size_t row;
            bool ok = true;
            if (p.tables) {
                const int phys = p.tables[(size_t)b * p.max_blocks + key / p.block_size];
                if (phys < 0 || phys >= p.num_blocks) {
                    atomicOr(p.status, kStatusBadTable);
                    ok = false;
                }
                row = ((size_t)(ok ? phys : 0) * p.block_size + key % p.block_size) * p.hkv + kvh;
            } else {
                row = ((size_t)b * p.hkv + kvh) * p.kv_stride + key;
            }
            if (ok) {
                krow = p.k + row * p.d;
                vrow = p.v + row * p.d;
            }
        } else if (key < total) {
            const int node = key - visible;
            if ((anc >> node) & 1ull) {
                const size_t row = ((size_t)b * p.hkv + kvh) * p.n_nodes + node;
                krow = p.k_tree + row * p.d;
                vrow = p.v_tree + row * p.d;
            }
        }
        float s = -INFINITY;
        if (krow) {
            float dot = 0.f;
            for (int i = 0; i < p.d; i += 8) {  // head_dim is a multiple of 8: 16-byte pieces
                const uint4 pk = *reinterpret_cast<const uint4*>(krow + i);
                const __half2* h2 = reinterpret_cast<const __half2*>(&pk);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 kf = __half22float2(h2[e]);
                    dot = fmaf(s_q[i + 2 * e], kf.x, dot);
                    dot = fmaf(s_q[i + 2 * e + 1], kf.y, dot);
                }
            }
            s = dot * p.scale;
        }
        const float m_chunk = block_max(s, s_red);
        const float m_new = fmaxf(m_run, m_chunk);
        const float pw = (krow && m_new > -INFINITY) ? __expf(s - m_new) : 0.f;
        s_p[tid] = pw;
        s_vrow[tid] = vrow;
        const float l_chunk = block_sum(pw, s_red);  // its barriers also publish s_p / s_vrow
        const float alpha = m_run > -INFINITY ? __expf(m_run - m_new) : 0.f;
        l_run = l_run * alpha + l_chunk;
        m_run = m_new;
        // phase 2: thread = output dim
        const int n_keys = min(kGenThreads, total - base);
#pragma unroll
        for (int u = 0; u < kGenMaxDim / kGenThreads; u++) {
            const int dim = tid + u * kGenThreads;
            if (dim >= p.d) continue;
            float a = acc[u] * alpha;
            for (int j = 0; j < n_keys; j++) {
                const __half* vr = s_vrow[j];
                if (vr) a = fmaf(s_p[j], __half2float(vr[dim]), a);
            }
            acc[u] = a;
        }
        __syncthreads();  // s_p / s_vrow are rewritten by the next chunk
    }
#pragma unroll
    for (int u = 0; u < kGenMaxDim / kGenThreads; u++) {
        const int dim = tid + u * kGenThreads;
        if (dim >= p.d) continue;
        const float o = l_run > 0.f ? acc[u] / l_run : 0.f;  // an empty sequence gives zeros
        if (p.out_f16) static_cast<__half*>(p.out)[qo + dim] = __float2half_rn(o);
        else static_cast<float*>(p.out)[qo + dim] = o;
    }
}

int launch(granite_cuda_compute* c, const GenericParams& p, const char* name) {
    if (p.d <= 0 || p.d > kGenMaxDim || p.d % 8 != 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, std::string(name) + ": head_dim must be a multiple of 8, at most 256");
    if (p.hkv <= 0 || p.hq % p.hkv != 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, std::string(name) + ": num_heads must be a multiple of num_kv_heads");
    if ((long long)p.batch * p.q_rows > 0x7fffffffLL || p.hq > 65535)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, std::string(name) + ": too many query rows or heads for one launch");
    if (p.batch == 0 || p.q_rows == 0) return GRANITE_CUDA_SUCCESS;
    LaunchScope t(c, name);
    generic_attention_kernel<<<dim3((unsigned)(p.batch * p.q_rows), (unsigned)p.hq), kGenThreads, 0, c->stream>>>(p);
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

}  // namespace

int launch_generic_decode(granite_cuda_compute* c, const GraniteCudaPagedDecodeArgs& a, bool contiguous, uint32_t max_seq) {
    if (!a.q || !a.k_cache || !a.v_cache || !a.output || (!contiguous && !a.block_tables))
        return fail(GRANITE_CUDA_NULL_POINTER, "decode: null buffer");
    if (!contiguous && (a.block_size == 0 || a.num_blocks == 0 || a.max_blocks_per_seq == 0))
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "paged decode: empty pool or table");
    GenericParams p{};
    p.q = a.q;
    p.out = a.output;
    p.k = static_cast<const __half*>(a.k_cache);
    p.v = static_cast<const __half*>(a.v_cache);
    p.tables = contiguous ? nullptr : a.block_tables;
    p.kv_lens = a.seq_lens;
    p.batch = (int)a.batch_size;
    p.q_rows = 1;
    p.hq = (int)a.num_heads;
    p.hkv = (int)a.num_kv_heads;
    p.d = (int)a.head_dim;
    p.kv_len = (int)a.seq_len;
    p.kv_stride = (int)max_seq;
    p.max_blocks = (int)a.max_blocks_per_seq;
    p.block_size = (int)a.block_size;
    p.num_blocks = (int)a.num_blocks;
    p.causal_start = -1;
    p.scale = a.scale;
    p.status = c->d_status;
    return launch(c, p, "generic_decode");
}

int launch_generic_prefill(granite_cuda_compute* c, const GraniteCudaAttentionArgs& a) {
    if (!a.q || !a.k || !a.v || !a.output) return fail(GRANITE_CUDA_NULL_POINTER, "prefill: null buffer");
    if (a.q_dtype > 1 || a.out_dtype > 1) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "prefill: dtype must be 0 (fp32) or 1 (fp16)");
    const uint32_t max_seq = a.max_seq ? a.max_seq : a.seq_kv;
    if (a.seq_kv == 0 || a.seq_kv > max_seq) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "prefill: seq_kv must be in [1, max_seq]");
    GenericParams p{};
    p.q = a.q;
    p.out = a.output;
    p.q_f16 = a.q_dtype == 1;
    p.out_f16 = a.out_dtype == 1;
    p.k = static_cast<const __half*>(a.k);
    p.v = static_cast<const __half*>(a.v);
    p.batch = a.batch_size ? (int)a.batch_size : 1;
    p.q_rows = (int)a.seq_q;
    p.hq = (int)a.num_heads;
    p.hkv = (int)a.num_kv_heads;
    p.d = (int)a.head_dim;
    p.kv_len = (int)a.seq_kv;
    p.kv_stride = (int)max_seq;
    p.causal_start = (int)a.start_pos;
    p.scale = a.scale;
    p.status = c->d_status;
    return launch(c, p, "generic_prefill");
}

int launch_generic_paged_prefill(granite_cuda_compute* c, const GraniteCudaPagedPrefillArgs& a) {
    if (!a.q || !a.k_cache || !a.v_cache || !a.block_table || !a.output)
        return fail(GRANITE_CUDA_NULL_POINTER, "paged_prefill_attention: null buffer");
    if (a.q_dtype > 1 || a.out_dtype > 1)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "paged_prefill_attention: dtype must be 0 (fp32) or 1 (fp16)");
    if (a.block_size == 0 || a.num_blocks == 0 || a.max_blocks_per_seq == 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "paged_prefill_attention: empty pool or table");
    if ((uint64_t)a.start_pos + a.seq_q > (uint64_t)a.max_blocks_per_seq * a.block_size)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "paged_prefill_attention: the chunk ends beyond the block table");
    GenericParams p{};
    p.q = a.q;
    p.out = a.output;
    p.q_f16 = a.q_dtype == 1;
    p.out_f16 = a.out_dtype == 1;
    p.k = static_cast<const __half*>(a.k_cache);
    p.v = static_cast<const __half*>(a.v_cache);
    p.tables = a.block_table;
    p.batch = 1;
    p.q_rows = (int)a.seq_q;
    p.hq = (int)a.num_heads;
    p.hkv = (int)a.num_kv_heads;
    p.d = (int)a.head_dim;
    p.kv_len = (int)(a.start_pos + a.seq_q);
    p.max_blocks = (int)a.max_blocks_per_seq;
    p.block_size = (int)a.block_size;
    p.num_blocks = (int)a.num_blocks;
    p.causal_start = (int)a.start_pos;
    p.scale = a.scale;
    p.status = c->d_status;
    return launch(c, p, "generic_paged_prefill");
}

int launch_generic_tree(granite_cuda_compute* c, const GraniteCudaTreeAttentionArgs& a) {
    if (!a.q || !a.k_tree || !a.v_tree || !a.parent_indices || !a.output)
        return fail(GRANITE_CUDA_NULL_POINTER, "attention_tree: null buffer");
    if (a.num_nodes == 0 || a.num_nodes > 64) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: num_nodes must be in [1, 64]");
    if (a.q_dtype > 1) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: q_dtype must be 0 (fp32) or 1 (fp16)");
    const bool paged = a.block_tables != nullptr;
    const bool has_cache = a.cache_lens != nullptr || a.cache_len > 0;
    if (has_cache && (!a.k_cache || !a.v_cache)) return fail(GRANITE_CUDA_NULL_POINTER, "attention_tree: null cache");
    if (paged && (a.block_size == 0 || a.num_blocks == 0 || a.max_blocks_per_seq == 0))
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: paged prefix needs a non-empty pool");
    const uint32_t cache_stride = a.cache_stride ? a.cache_stride : a.cache_len;
    if (!paged && has_cache && a.cache_len > cache_stride)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: cache_len exceeds cache_stride");
    GenericParams p{};
    p.q = a.q;
    p.out = a.output;
    p.q_f16 = a.q_dtype == 1;
    p.tree_layout = 1;
    p.k = static_cast<const __half*>(a.k_cache);
    p.v = static_cast<const __half*>(a.v_cache);
    p.k_tree = static_cast<const __half*>(a.k_tree);
    p.v_tree = static_cast<const __half*>(a.v_tree);
    p.tables = a.block_tables;
    p.kv_lens = a.cache_lens;
    p.parents = a.parent_indices;
    p.batch = (int)a.batch_size;
    p.q_rows = (int)a.num_nodes;
    p.n_nodes = (int)a.num_nodes;
    p.hq = (int)a.num_heads;
    p.hkv = (int)a.num_kv_heads;
    p.d = (int)a.head_dim;
    p.kv_len = (int)a.cache_len;
    p.kv_stride = (int)cache_stride;
    p.max_blocks = (int)a.max_blocks_per_seq;
    p.block_size = (int)a.block_size;
    p.num_blocks = (int)a.num_blocks;
    p.causal_start = -1;
    p.scale = a.scale;
    p.status = c->d_status;
    return launch(c, p, "generic_tree_verify");
}

}  // namespace gb200
