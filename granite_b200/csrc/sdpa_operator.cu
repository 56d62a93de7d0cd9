// Operator-level scaled-dot-product attention: out = softmax(scale * Q K^T) V for one head and
// any head_dim.  This is the small general form behind OpType::ScaledDotProductAttention
// (the operator registry path; the LLM path uses the decode / prefill / tree kernels):
//   - fp32, K given pre-transposed as [D, T], no mask: the Vulkan operator's contract
//     (src/operators/vulkan/vulkan_operators.cpp:345-434, known answer in
//     tests/test_vulkan.cpp:353-482);
//   - fp16, K as [T, D], keys limited to q_idx + start_pos + 1: the Metal operator's contract
//     (src/operators/metal/metal_operators.mm:619-690, :1226-1325).
// One block per query row; scores live in shared memory; fp32 arithmetic, three-pass softmax.
#include <cuda_fp16.h>

#include "compute_internal.h"

namespace gb200 {

template <typename T>
__device__ __forceinline__ float ld(const T* p, size_t i);
template <>
__device__ __forceinline__ float ld<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ld<__half>(const __half* p, size_t i) { return __half2float(p[i]); }
__device__ __forceinline__ void st(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void st(__half* p, size_t i, float v) { p[i] = __float2half_rn(v); }

template <typename T>
__global__ void sdpa_operator_kernel(const T* q, const T* k, const T* v, T* out, int seq_q, int seq_kv,
                                     int head_dim, float scale, int k_transposed, int causal, int start_pos) {
    extern __shared__ float scores[];
    __shared__ float red[32];
    const int qi = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    int kv = seq_kv;
    if (causal) kv = min(seq_kv, qi + start_pos + 1);
    for (int j = tid; j < kv; j += nt) {
        float dot = 0.f;
        for (int d = 0; d < head_dim; d++) {
            const float kk = k_transposed ? ld(k, (size_t)d * seq_kv + j) : ld(k, (size_t)j * head_dim + d);
            dot += ld(q, (size_t)qi * head_dim + d) * kk;
        }
        scores[j] = dot * scale;
    }
    __syncthreads();
    auto block_reduce = [&](float val, bool is_max) {
        for (int o = 16; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, val, o);
            val = is_max ? fmaxf(val, other) : val + other;
        }
        if ((tid & 31) == 0) red[tid >> 5] = val;
        __syncthreads();
        float r = is_max ? -INFINITY : 0.f;
        for (int w = 0; w < (nt + 31) / 32; w++) r = is_max ? fmaxf(r, red[w]) : r + red[w];
        __syncthreads();
        return r;
    };
    float mx = -INFINITY;
    for (int j = tid; j < kv; j += nt) mx = fmaxf(mx, scores[j]);
    mx = block_reduce(mx, true);
    float sum = 0.f;
    for (int j = tid; j < kv; j += nt) {
        const float e = expf(scores[j] - mx);
        scores[j] = e;
        sum += e;
    }
    sum = block_reduce(sum, false);
    const float inv = 1.0f / sum;
    for (int d = tid; d < head_dim; d += nt) {
        float acc = 0.f;
        for (int j = 0; j < kv; j++) acc += scores[j] * inv * ld(v, (size_t)j * head_dim + d);
        st(out, (size_t)qi * head_dim + d, acc);
    }
}

int launch_sdpa_operator(granite_cuda_compute* c, const GraniteCudaSdpaArgs& a) {
    if (!a.q || !a.k || !a.v || !a.output) return fail(GRANITE_CUDA_NULL_POINTER, "sdpa: null buffer");
    if (a.seq_q == 0 || a.seq_kv == 0 || a.head_dim == 0) return fail(GRANITE_CUDA_INVALID_SHAPE, "sdpa: empty shape");
    if (a.dtype > 1) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "sdpa: dtype must be 0 (fp32) or 1 (fp16)");
    // The Metal operator's layout (fp16, K row-major, keys limited to q + start_pos + 1) with a head_dim the
    // tensor-core kernel is tiled for IS causal prefill of one head: it runs there, on tcgen05, instead of on
    // the one-block-per-row kernel below.
    if (a.dtype == 1 && !a.k_transposed && a.causal && a.seq_q >= 2 && (a.head_dim == 128 || a.head_dim == 64)) {
        GraniteCudaAttentionArgs p{};
        p.q = a.q;
        p.k = a.k;
        p.v = a.v;
        p.output = a.output;
        p.num_heads = 1;
        p.num_kv_heads = 1;
        p.seq_q = a.seq_q;
        p.seq_kv = a.seq_kv;
        p.head_dim = a.head_dim;
        p.max_seq = a.seq_kv;
        p.q_dtype = 1;
        p.out_dtype = 1;
        p.scale = a.scale;
        p.start_pos = a.start_pos;
        p.batch_size = 1;
        return launch_prefill(c, p);
    }
    const size_t smem = (size_t)a.seq_kv * sizeof(float);
    if (smem > 200 * 1024) return fail(GRANITE_CUDA_INVALID_SHAPE, "sdpa operator: seq_kv above 51200 is not supported");
    LaunchScope t(c, "sdpa_operator");
    if (a.dtype == 0) {
        auto kern = sdpa_operator_kernel<float>;
        GB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<a.seq_q, 128, smem, c->stream>>>(static_cast<const float*>(a.q), static_cast<const float*>(a.k),
                                                static_cast<const float*>(a.v), static_cast<float*>(a.output),
                                                (int)a.seq_q, (int)a.seq_kv, (int)a.head_dim, a.scale,
                                                (int)a.k_transposed, (int)a.causal, (int)a.start_pos);
    } else {
        auto kern = sdpa_operator_kernel<__half>;
        GB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<a.seq_q, 128, smem, c->stream>>>(static_cast<const __half*>(a.q), static_cast<const __half*>(a.k),
                                                static_cast<const __half*>(a.v), static_cast<__half*>(a.output),
                                                (int)a.seq_q, (int)a.seq_kv, (int)a.head_dim, a.scale,
                                                (int)a.k_transposed, (int)a.causal, (int)a.start_pos);
    }
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

}  // namespace gb200
