// Causal flash-attention prefill on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Replaces flash_attention_prefill (src/backend/metal/kernels/metal_shaders_attention.h:1453,
// dispatched by MetalCompute::multihead_attention with seq_q > 1,
// src/backend/metal/metal_compute.mm:2333-2375); the arithmetic it must match is the CPU loop
// src/llm/transformer.mm:1779-1840 with the causal rule k_pos > start_pos + q_pos -> -inf.
//
// One CTA owns two 128-row query tiles that share every K/V tile: the two query heads of a GQA
// pair at the same query block.  Roles (384 threads):
//   warp 0      TMA producer: Q tiles once, then K_j / V_j into 2-deep rings (128-byte swizzle)
//   warp 1      one elected thread issues tcgen05.mma: S_t = Q_t K_j^T (both operands in shared
//               memory) and O_t += P_t V_j (P from TMEM, V from shared memory, MN-major);
//               order S0 S1 | PV0 S0' PV1 S1' | ... so one tile's softmax overlaps the other's MMAs
//   warps 4-7   softmax of tile 0, warps 8-11 softmax of tile 1: thread = query row; S is read
//               from TMEM with tcgen05.ld, P (fp16) is written back over S with tcgen05.st;
//               the running maximum is only raised when it grows by more than 2^8 (lazy rescale
//               of O in TMEM), which is exact because l and O always share the same reference
// TMEM (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each; P_t aliases the first 64 of S_t.
// Accumulation is fp32 throughout; P is rounded to fp16 only as the MMA input.
#include <cstdio>
#include <cstring>

#include "compute_internal.h"
#include "ptx.cuh"

namespace gb200 {

// Development aid: built with -DGB_FA_TRACE the first CTA records clock64() at the hand-over points
// of its roles (slot = role * 64 + step * 4 + event) and the launcher prints the timeline.
#ifdef GB_FA_TRACE
#define FA_TRACE(role, step, ev) \
    do { if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && (step) < 16) p.trace[(role) * 64 + (step) * 4 + (ev)] = clock64(); } while (0)
#else
#define FA_TRACE(role, step, ev) do {} while (0)
#endif

constexpr int kFaThreads = 384;
constexpr int kTile = 128;                    // query rows per tile, keys per KV tile, head_dim
constexpr int kTileBytes = kTile * kTile * 2;  // 32 KB: one [128 x 128] fp16 tile
constexpr int kChunkBytes = kTileBytes / 2;    // 16 KB: one 64-column (128-byte) swizzle block
constexpr float kLazyRescaleLog2 = 8.0f;

struct FaParams {
    void* out;           // [seq_q, Hq, 128] fp16 or fp32
    int out_fp16;
    int seq_q, seq_kv, max_seq;
    int num_heads, num_kv_heads, group, pairs;  // pairs = ceil(group / 2)
    int n_qblocks;
    int start_pos;
    float scale_log2;
    int* status;
    unsigned long long* trace;  // timeline hook, only used in GB_FA_TRACE builds
};

struct FaSmem {
    uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_ready[2], o_final[2];
    uint32_t tmem_base;
    int abort_flag;
};

// fp32 -> fp16 hi + fp16 lo (x ~= hi + lo to about 22 bits), so fp32 queries lose nothing.
__global__ void split_f32_to_f16_kernel(const float* __restrict__ src, __half* __restrict__ hi,
                                        __half* __restrict__ lo, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float x = src[i];
        const __half h = __float2half_rn(x);
        hi[i] = h;
        lo[i] = __float2half_rn(x - __half2float(h));
    }
}

// kSplitP: P enters the PV product as fp16 hi + fp16 lo (two MMAs per step) so that the softmax
//          weights keep ~22 bits, as the fp32 reference does.  kSplitQ: the query tile is given as
//          hi + lo fp16 arrays (fp32 queries); the CTA then owns one query tile, not two.
template <bool kSplitP, bool kSplitQ>
__global__ void __launch_bounds__(kFaThreads, 1)
prefill_fa_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap qlomap,
                  const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                  FaParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_smem = smem;                       // 2 tiles
    uint8_t* k_smem = smem + 2 * kTileBytes;      // 2 stages
    uint8_t* v_smem = smem + 4 * kTileBytes;      // 2 stages
    FaSmem* sh = reinterpret_cast<FaSmem*>(smem + 6 * kTileBytes);
    volatile int* abort_flag = &sh->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // work item: heaviest query blocks first
    int item = blockIdx.x;
    const int pair = item % p.pairs; item /= p.pairs;
    const int kvh = item % p.num_kv_heads; item /= p.num_kv_heads;
    const int qb = p.n_qblocks - 1 - item;
    const int q0 = qb * kTile;
    const int head0 = kSplitQ ? kvh * p.group + pair : kvh * p.group + 2 * pair;
    const bool valid1 = !kSplitQ && (2 * pair + 1 < p.group);
    const int rows_here = min(kTile, p.seq_q - q0);
    const int k_end = min(p.seq_kv, p.start_pos + q0 + rows_here);  // exclusive: last visible key + 1
    const int n_kv = (k_end + kTile - 1) / kTile;

    if (threadIdx.x == 0) {
        mbar_init(&sh->q_full, 1);
        for (int i = 0; i < 2; i++) {
            mbar_init(&sh->k_full[i], 1);
            mbar_init(&sh->k_empty[i], 1);
            mbar_init(&sh->v_full[i], 1);
            mbar_init(&sh->v_empty[i], 1);
            mbar_init(&sh->s_full[i], 1);
            mbar_init(&sh->p_ready[i], 128);
            mbar_init(&sh->o_final[i], 1);
        }
        sh->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(&sh->tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sh->tmem_base;

    if (warp < 4) {
    setmaxnreg_dec<56>();  // producer / MMA warpgroup gives registers up
    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&qmap);
            tma_prefetch_desc(&kmap);
            tma_prefetch_desc(&vmap);
            if (kSplitQ) {
                tma_prefetch_desc(&qlomap);
                mbar_arrive_expect_tx(&sh->q_full, 2 * kTileBytes);
                for (int c = 0; c < 2; c++) {
                    tma_load_2d(q_smem + c * kChunkBytes, &qmap, &sh->q_full, head0 * kTile + c * 64, q0);
                    tma_load_2d(q_smem + kTileBytes + c * kChunkBytes, &qlomap, &sh->q_full, head0 * kTile + c * 64, q0);
                }
            } else {
                mbar_arrive_expect_tx(&sh->q_full, (valid1 ? 2 : 1) * kTileBytes);
                for (int t = 0; t < (valid1 ? 2 : 1); t++)
                    for (int c = 0; c < 2; c++)
                        tma_load_2d(q_smem + t * kTileBytes + c * kChunkBytes, &qmap, &sh->q_full,
                                    (head0 + t) * kTile + c * 64, q0);
            }
            bool ok = true;
            for (int j = 0; j < n_kv && ok; j++) {
                const int s = j & 1;
                const uint32_t ph = ((j >> 1) & 1) ^ 1;
                const int y = kvh * p.max_seq + j * kTile;
                ok = mbar_wait(&sh->k_empty[s], ph, abort_flag);
                if (!ok) break;
                mbar_arrive_expect_tx(&sh->k_full[s], kTileBytes);
                for (int c = 0; c < 2; c++)
                    tma_load_2d(k_smem + s * kTileBytes + c * kChunkBytes, &kmap, &sh->k_full[s], c * 64, y);
                ok = mbar_wait(&sh->v_empty[s], ph, abort_flag);
                if (!ok) break;
                mbar_arrive_expect_tx(&sh->v_full[s], kTileBytes);
                for (int c = 0; c < 2; c++)
                    tma_load_2d(v_smem + s * kTileBytes + c * kChunkBytes, &vmap, &sh->v_full[s], c * 64, y);
            }
            if (!ok) atomicOr(p.status, kStatusTimeout);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_f16(kTile, kTile, false, false);
            constexpr uint32_t idesc_pv = umma_idesc_f16(kTile, kTile, false, true);
            const uint32_t q_addr = smem_u32(q_smem), k_addr = smem_u32(k_smem), v_addr = smem_u32(v_smem);
            // descriptor low words of every operand base; a k-step only adds a constant
            const uint32_t q_lo[2] = {desc_lo(q_addr, 16), desc_lo(q_addr + kTileBytes, 16)};
            const uint32_t k_lo[2] = {desc_lo(k_addr, 16), desc_lo(k_addr + kTileBytes, 16)};
            const uint32_t v_lo[2] = {desc_lo(v_addr, kChunkBytes), desc_lo(v_addr + kTileBytes, kChunkBytes)};
            auto issue_qk = [&](int t, int s) {
                // S_t = Q_t K^T: K-major operands, 8 steps of 16 along head_dim (32 bytes inside the
                // swizzled row, the second 64-wide block 16 KB further)
                const uint32_t d = tmem + t * kTile;
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    const uint32_t off = ((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4;
                    umma_ss_words(d, q_lo[t] + off, k_lo[s] + off, kDescHiSw128, idesc_qk, ks > 0 ? 1u : 0u);
                }
                if (kSplitQ) {  // + Q_lo K^T (the low halves sit in the second query slot)
#pragma unroll
                    for (int ks = 0; ks < 8; ks++) {
                        const uint32_t off = ((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4;
                        umma_ss_words(d, q_lo[1] + off, k_lo[s] + off, kDescHiSw128, idesc_qk, 1u);
                    }
                }
            };
            auto issue_pv = [&](int t, int s, bool acc) {
                // O_t += P_t V: P from TMEM (8 columns per 16 keys), V MN-major in shared memory
                // (16 keys = 2 KB further per step; the second 64-wide block of head_dim via LBO)
                const uint32_t d = tmem + 2 * kTile + t * kTile;
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    const uint32_t vl = v_lo[s] + ks * (2048 >> 4);
                    if (kSplitP) {
                        // each 64-column half of S_t was replaced by 32 columns of P_hi + 32 of P_lo
                        const uint32_t a_hi = tmem + t * kTile + (ks >> 2) * 64 + (ks & 3) * 8;
                        umma_ts_words(d, a_hi, vl, kDescHiSw128, idesc_pv, (acc || ks > 0) ? 1u : 0u);
                        umma_ts_words(d, a_hi + 32, vl, kDescHiSw128, idesc_pv, 1u);
                    } else {
                        umma_ts_words(d, tmem + t * kTile + ks * 8, vl, kDescHiSw128, idesc_pv, (acc || ks > 0) ? 1u : 0u);
                    }
                }
            };
            bool ok = mbar_wait(&sh->q_full, 0, abort_flag) && mbar_wait(&sh->k_full[0], 0, abort_flag);
            if (ok) {
                tc_fence_after_sync();
                issue_qk(0, 0);
                tc_commit(&sh->s_full[0]);
                if (valid1) {
                    issue_qk(1, 0);
                    tc_commit(&sh->s_full[1]);
                }
                tc_commit(&sh->k_empty[0]);
            }
            for (int j = 0; j < n_kv && ok; j++) {
                const int s = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                const bool more = j + 1 < n_kv;
                const int s2 = (j + 1) & 1;
                const uint32_t ph2 = ((j + 1) >> 1) & 1;
                FA_TRACE(0, j, 0);
                ok = mbar_wait(&sh->v_full[s], ph, abort_flag) && mbar_wait(&sh->p_ready[0], j & 1, abort_flag);
                if (!ok) break;
                FA_TRACE(0, j, 1);
                tc_fence_after_sync();
                issue_pv(0, s, j > 0);
                if (!more) tc_commit(&sh->o_final[0]);
                if (more) {
                    ok = mbar_wait(&sh->k_full[s2], ph2, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_qk(0, s2);
                    tc_commit(&sh->s_full[0]);
                }
                if (valid1) {
                    FA_TRACE(0, j, 2);
                    ok = mbar_wait(&sh->p_ready[1], j & 1, abort_flag);
                    if (!ok) break;
                    FA_TRACE(0, j, 3);
                    tc_fence_after_sync();
                    issue_pv(1, s, j > 0);
                    if (!more) tc_commit(&sh->o_final[1]);
                }
                tc_commit(&sh->v_empty[s]);
                if (more) {
                    if (valid1) {
                        issue_qk(1, s2);
                        tc_commit(&sh->s_full[1]);
                    }
                    tc_commit(&sh->k_empty[s2]);
                }
            }
            if (!ok) atomicOr(p.status, kStatusTimeout);
        }
    }
    } else {
        setmaxnreg_inc<224>();  // softmax warpgroups hold a whole S row in registers
        // ------------------------------------------------------------------ softmax + epilogue
        const int t = (warp - 4) >> 2;           // which query tile
        const int quarter = warp & 3;            // TMEM lane quarter this warp may touch
        const int row = quarter * 32 + lane;     // query row inside the tile
        if (t == 0 || valid1) {
            const uint32_t lane_base = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
            const uint32_t s_addr = lane_base + t * kTile;
            const uint32_t o_addr = lane_base + 2 * kTile + t * kTile;
            const int q_pos = q0 + row;
            const int last_visible = min(p.start_pos + q_pos, p.seq_kv - 1);  // key index
            float m_used = -INFINITY, l_run = 0.f;
            bool ok = true;
            for (int j = 0; j < n_kv; j++) {
                if (quarter == 0) FA_TRACE(1 + t, j, 0);
                ok = mbar_wait(&sh->s_full[t], j & 1, abort_flag);
                if (!ok) break;
                if (quarter == 0) FA_TRACE(1 + t, j, 1);
                tc_fence_after_sync();
                const int k0 = j * kTile;
                const bool need_mask = (k0 + kTile - 1 > p.start_pos + q0) || (k0 + kTile > p.seq_kv);
                const int limit = last_visible - k0;  // column c is visible iff c <= limit
                // S row (128 fp32) into registers: four loads in flight, one wait
                uint32_t x0[32], x1[32], x2[32], x3[32];
                tmem_ld32(s_addr, x0);
                tmem_ld32(s_addr + 32, x1);
                tmem_ld32(s_addr + 64, x2);
                tmem_ld32(s_addr + 96, x3);
                tmem_wait_ld();
                if (quarter == 0) FA_TRACE(1 + t, j, 2);
                float mx = -INFINITY;
                if (need_mask) {
#pragma unroll
                    for (int c = 0; c < 32; c++) {
                        if (c > limit) x0[c] = 0xFF800000u;        // -inf
                        if (32 + c > limit) x1[c] = 0xFF800000u;
                        if (64 + c > limit) x2[c] = 0xFF800000u;
                        if (96 + c > limit) x3[c] = 0xFF800000u;
                    }
                }
                {
                    // four independent chains (short dependency depth: two warps share a scheduler)
                    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        m0 = fmaxf(m0, fmaxf(__uint_as_float(x0[c]), __uint_as_float(x0[c + 1])));
                        m1 = fmaxf(m1, fmaxf(__uint_as_float(x1[c]), __uint_as_float(x1[c + 1])));
                        m2 = fmaxf(m2, fmaxf(__uint_as_float(x2[c]), __uint_as_float(x2[c + 1])));
                        m3 = fmaxf(m3, fmaxf(__uint_as_float(x3[c]), __uint_as_float(x3[c + 1])));
                    }
                    mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
                }
                mx *= p.scale_log2;
                if (j == 0) {
                    m_used = mx;
                } else {
                    const bool grow = mx > m_used + kLazyRescaleLog2;
                    if (__any_sync(0xffffffffu, grow)) {
                        // S_t(j) being complete implies PV_t(j-1) is complete: O_t is quiescent
                        const float alpha = grow ? fast_exp2(m_used - mx) : 1.0f;
                        if (grow) m_used = mx;
                        l_run *= alpha;
                        uint32_t r[32];
#pragma unroll 1
                        for (int ch = 0; ch < 4; ch++) {
                            tmem_ld32(o_addr + ch * 32, r);
                            tmem_wait_ld();
#pragma unroll
                            for (int c = 0; c < 32; c++) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
                            tmem_st32(o_addr + ch * 32, r);
                        }
                    }
                }
                // P = 2^(s*scale - m): fp16 hi (and lo = P - hi when kSplitP) written over S.  Each
                // 64-column half of S becomes 32 columns of hi followed by 32 columns of lo.
                float ls[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};  // independent partial sums
                const float neg_m = -m_used;
                auto emit = [&](uint32_t (&x)[32], int chunk) {
                    uint32_t hi[16], lo[16];
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        // masked scores are -inf: exp2 gives exactly 0
                        const float p0 = fast_exp2(fmaf(__uint_as_float(x[c]), p.scale_log2, neg_m));
                        const float p1 = fast_exp2(fmaf(__uint_as_float(x[c + 1]), p.scale_log2, neg_m));
                        ls[c & 6] += p0;
                        ls[(c & 6) + 1] += p1;
                        if (kSplitP) split_hi_lo(p0, p1, hi[c >> 1], lo[c >> 1]);
                        else hi[c >> 1] = pack_half2(p0, p1);
                    }
                    if (kSplitP) {
                        tmem_st16(s_addr + (chunk >> 1) * 64 + (chunk & 1) * 16, hi);
                        tmem_st16(s_addr + (chunk >> 1) * 64 + 32 + (chunk & 1) * 16, lo);
                    } else {
                        tmem_st16(s_addr + chunk * 16, hi);
                    }
                };
                emit(x0, 0);
                emit(x1, 1);
                emit(x2, 2);
                emit(x3, 3);
                l_run += ((ls[0] + ls[1]) + (ls[2] + ls[3])) + ((ls[4] + ls[5]) + (ls[6] + ls[7]));
                if (t == 0 && k0 + kTile > p.seq_kv) {
                    // keys past seq_kv carry P = 0, but their V rows may hold anything (even NaN):
                    // zero them in shared memory before the MMA reads the tile
                    const int s = j & 1;
                    ok = mbar_wait(&sh->v_full[s], (j >> 1) & 1, abort_flag);
                    if (!ok) break;
                    const int first_bad = p.seq_kv - k0;
                    uint8_t* vt = v_smem + s * kTileBytes;
                    for (int i = row; i < (kTile - first_bad) * 16; i += 128) {
                        const int rr = first_bad + (i >> 4), u = i & 15;
                        *reinterpret_cast<uint4*>(vt + (u >> 3) * kChunkBytes + rr * 128 + (((u & 7) ^ (rr & 7)) << 4)) =
                            make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();
                }
                __syncwarp();
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&sh->p_ready[t]);
                if (quarter == 0) FA_TRACE(1 + t, j, 3);
            }
            if (ok) ok = mbar_wait(&sh->o_final[t], 0, abort_flag);
            if (ok) {
                tc_fence_after_sync();
                const float inv = 1.0f / l_run;
                const int head = head0 + t;
                const bool store = row < rows_here;
                uint32_t r[32];
#pragma unroll 1
                for (int ch = 0; ch < 4; ch++) {
                    __syncwarp();
                    tmem_ld32(o_addr + ch * 32, r);
                    tmem_wait_ld();
                    if (store) {
                    const size_t base = ((size_t)q_pos * p.num_heads + head) * kTile + ch * 32;
                    if (p.out_fp16) {
                        uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(p.out) + base);
#pragma unroll
                        for (int v = 0; v < 4; v++) {
                            uint4 o;
                            o.x = pack_half2(__uint_as_float(r[v * 8 + 0]) * inv, __uint_as_float(r[v * 8 + 1]) * inv);
                            o.y = pack_half2(__uint_as_float(r[v * 8 + 2]) * inv, __uint_as_float(r[v * 8 + 3]) * inv);
                            o.z = pack_half2(__uint_as_float(r[v * 8 + 4]) * inv, __uint_as_float(r[v * 8 + 5]) * inv);
                            o.w = pack_half2(__uint_as_float(r[v * 8 + 6]) * inv, __uint_as_float(r[v * 8 + 7]) * inv);
                            dst[v] = o;
                        }
                    } else {
                        float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.out) + base);
#pragma unroll
                        for (int v = 0; v < 8; v++)
                            dst[v] = make_float4(__uint_as_float(r[v * 4 + 0]) * inv, __uint_as_float(r[v * 4 + 1]) * inv,
                                                 __uint_as_float(r[v * 4 + 2]) * inv, __uint_as_float(r[v * 4 + 3]) * inv);
                    }
                    }
                }
            } else if (lane == 0) {
                atomicOr(p.status, kStatusTimeout);
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

// ------------------------------------------------------------------------------------ host
int launch_prefill(granite_cuda_compute* c, const GraniteCudaAttentionArgs& a) {
    if (!a.q || !a.k || !a.v || !a.output) return fail(GRANITE_CUDA_NULL_POINTER, "prefill: null buffer");
    if (a.head_dim != kTile) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "prefill: head_dim must be 128");
    if (a.num_kv_heads == 0 || a.num_heads % a.num_kv_heads != 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "prefill: num_heads must be a multiple of num_kv_heads");
    if (a.q_dtype > 1 || a.out_dtype > 1) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "prefill: dtype must be 0 (fp32) or 1 (fp16)");
    const uint32_t max_seq = a.max_seq ? a.max_seq : a.seq_kv;
    if (a.seq_kv == 0 || a.seq_kv > max_seq) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "prefill: seq_kv must be in [1, max_seq]");

    const void* q16 = a.q;
    const void* q16_lo = a.q;
    const size_t q_elems = (size_t)a.seq_q * a.num_heads * kTile;
    const bool split_q = a.q_dtype == 0;
    if (split_q) {
        const size_t half_bytes = (q_elems * 2 + 255) / 256 * 256;
        int rc = c->ensure_scratch(2 * half_bytes);
        if (rc) return rc;
        LaunchScope t(c, "split_q_f16");
        __half* hi = static_cast<__half*>(c->scratch);
        __half* lo = reinterpret_cast<__half*>(static_cast<uint8_t*>(c->scratch) + half_bytes);
        split_f32_to_f16_kernel<<<(unsigned)((q_elems + 255) / 256), 256, 0, c->stream>>>(
            static_cast<const float*>(a.q), hi, lo, q_elems);
        q16 = hi;
        q16_lo = lo;
    }

    FaParams p{};
    p.out = a.output;
    p.out_fp16 = a.out_dtype == 1;
    p.seq_q = (int)a.seq_q;
    p.seq_kv = (int)a.seq_kv;
    p.max_seq = (int)max_seq;
    p.num_heads = (int)a.num_heads;
    p.num_kv_heads = (int)a.num_kv_heads;
    p.group = (int)(a.num_heads / a.num_kv_heads);
    p.pairs = split_q ? p.group : (p.group + 1) / 2;
    p.n_qblocks = (p.seq_q + kTile - 1) / kTile;
    p.start_pos = (int)a.start_pos;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.status = c->d_status;

    const CUtensorMap* qmap = c->tensor_map_2d(q16, (uint64_t)a.num_heads * kTile, a.seq_q,
                                               (uint64_t)a.num_heads * kTile * 2, 64, kTile, 128);
    const CUtensorMap* qlomap = c->tensor_map_2d(q16_lo, (uint64_t)a.num_heads * kTile, a.seq_q,
                                                 (uint64_t)a.num_heads * kTile * 2, 64, kTile, 128);
    const uint64_t kv_rows = (uint64_t)a.num_kv_heads * max_seq;
    const CUtensorMap* kmap = c->tensor_map_2d(a.k, kTile, kv_rows, kTile * 2, 64, kTile, 128);
    const CUtensorMap* vmap = c->tensor_map_2d(a.v, kTile, kv_rows, kTile * 2, 64, kTile, 128);
    if (!qmap || !qlomap || !kmap || !vmap) return GRANITE_CUDA_EXECUTION_FAILED;

    const size_t smem_bytes = 1024 + 6 * kTileBytes + sizeof(FaSmem);
    auto kern = split_q ? prefill_fa_kernel<true, true> : prefill_fa_kernel<true, false>;
    GB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    const int grid = p.n_qblocks * p.num_kv_heads * p.pairs;
#ifdef GB_FA_TRACE
    static unsigned long long* trace_buf = nullptr;
    if (!trace_buf) cudaMallocManaged(&trace_buf, 3 * 64 * sizeof(unsigned long long));
    memset(trace_buf, 0, 3 * 64 * sizeof(unsigned long long));
    p.trace = trace_buf;
#endif
    {
        LaunchScope t(c, "prefill_causal_fa");
        kern<<<grid, kFaThreads, smem_bytes, c->stream>>>(*qmap, *qlomap, *kmap, *vmap, p);
    }
#ifdef GB_FA_TRACE
    cudaStreamSynchronize(c->stream);
    {
        unsigned long long t0 = trace_buf[64 + 1];  // softmax 0, step 0, S ready
        const char* roles[3] = {"mma", "sm0", "sm1"};
        for (int step = 0; step < 16; step++)
            for (int r = 0; r < 3; r++)
                fprintf(stderr, "trace %s step %2d: %8lld %8lld %8lld %8lld\n", roles[r], step,
                        (long long)(trace_buf[r * 64 + step * 4 + 0] - t0), (long long)(trace_buf[r * 64 + step * 4 + 1] - t0),
                        (long long)(trace_buf[r * 64 + step * 4 + 2] - t0), (long long)(trace_buf[r * 64 + step * 4 + 3] - t0));
    }
#endif
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

}  // namespace gb200
