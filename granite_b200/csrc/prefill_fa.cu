// Causal flash-attention prefill on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Replaces flash_attention_prefill (src/backend/metal/kernels/metal_shaders_attention.h:1453,
// dispatched by MetalCompute::multihead_attention with seq_q > 1,
// src/backend/metal/metal_compute.mm:2333-2375); the arithmetic it must match is the CPU loop
// src/llm/transformer.mm:1779-1840 with the causal rule k_pos > start_pos + q_pos -> -inf.
//
// A work item is one 128-row query tile (one query head, one query block) and the KV tiles it may
// see.  CTAs are persistent (one per SM) and run their items back to back: TMEM, barriers and the
// shared-memory rings are set up once, and the next item's Q/K/V loads and first score MMAs
// overlap the current item's last softmax and its epilogue.  S = Q K_j^T is double-buffered in TMEM, so the score MMAs of step j+1 run while
// the softmax of step j is still working, and O += P V_j follows as soon as P is written.
// Roles (384 threads):
//   warp 0      TMA producer: Q once, then K_j / V_j into shared-memory rings (128-byte swizzle)
//   warp 1      one thread issues the score MMAs S_b = Q K_j^T (operands in shared memory)
//   warps 2, 3  one thread each issues half of the output MMAs O += P_b V_j: warp 2 the fp16
//               "hi" part of P, warp 3 the "lo" part (P from TMEM, V from shared memory,
//               MN-major).  A single thread cannot issue 128x128x16 instructions fast enough to
//               keep the tensor pipe busy; three can.
//   warps 4-11  softmax: both warpgroups work on the same 128 rows, the first on key columns
//               0-63 of the tile, the second on 64-127; row maxima and sums are exchanged through
//               shared memory.  thread = query row; S is read with tcgen05.ld, P is written back
//               over S as fp16 hi + lo (P keeps ~22 bits, as the fp32 reference does); the
//               running maximum is only raised when it grows by more than 2^8 (lazy rescale of O)
// TMEM (512 columns): S[0] | S[1] | O | unused, 128 fp32 columns each.
#include <cstdio>
#include <cstring>

#include "compute_internal.h"
#include "ptx.cuh"

namespace gb200 {

// Development aid: built with -DGB_FA_TRACE one CTA records clock64() at the hand-over points of
// its roles (slot = role * 64 + step * 4 + event) and the launcher prints the timeline.
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
constexpr int kMaxStages = 3;

struct FaParams {
    void* out;           // [seq_q, Hq, 128] fp16 or fp32
    int out_fp16;
    int seq_q, seq_kv, max_seq;
    int num_heads, num_kv_heads, group;
    int n_qblocks;
    int start_pos;
    float scale_log2;
    int* status;
    unsigned long long* trace;  // timeline hook, only used in GB_FA_TRACE builds
};

struct FaSmem {
    uint64_t q_full, q_empty, k_full[kMaxStages], k_empty[kMaxStages], v_full[kMaxStages], v_empty[kMaxStages];
    uint64_t s_full[2], s_free[2], p_ready[2], o_final;
    uint32_t tmem_base;
    int abort_flag;
    float xchg[2][2][kTile];  // [step parity][warpgroup][row]: row maxima (and, at the end of an item, row sums) exchanged between the warpgroups
};

static_assert(sizeof(FaSmem) <= 3072, "barriers and exchange slots must fit beside seven 32 KB tiles");

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

__device__ __forceinline__ void softmax_group_sync() {
    asm volatile("bar.sync 1, 256;" ::: "memory");  // the two softmax warpgroups only
}

// kSplitQ: the query tile is given as hi + lo fp16 arrays (fp32 queries) and S = Q_hi K^T + Q_lo K^T.
// kStages: depth of the K and V rings.
template <bool kSplitQ, int kStages>
__global__ void __launch_bounds__(kFaThreads, 1)
prefill_fa_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap qlomap,
                  const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                  FaParams p) {
    // barriers and exchange slots first, then the 1024-byte aligned tiles (128-byte swizzle atoms)
    extern __shared__ __align__(16) uint8_t smem_raw[];
    FaSmem* sh = reinterpret_cast<FaSmem*>(smem_raw);
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + sizeof(FaSmem) + 1023) & ~uintptr_t(1023));
    constexpr int kQTiles = kSplitQ ? 2 : 1;
    uint8_t* q_smem = smem;
    uint8_t* k_smem = smem + kQTiles * kTileBytes;
    uint8_t* v_smem = k_smem + kStages * kTileBytes;
    volatile int* abort_flag = &sh->abort_flag;
    {
        uint32_t dyn_size;
        asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_size));
        if (v_smem + kStages * kTileBytes > smem_raw + dyn_size) {  // cannot happen with a 1 KB aligned window
            if (threadIdx.x == 0) atomicOr(p.status, kStatusLayout);
            return;
        }
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Persistent CTA: work items (query block, head) are ordered heaviest first and dealt to the
    // CTAs in a snake (round r runs left to right when even, right to left when odd), which keeps
    // the summed causal work per CTA within one KV step of the mean.
    const int n_items = p.n_qblocks * p.num_heads;
    const int n_rounds = (n_items + (int)gridDim.x - 1) / (int)gridDim.x;
    struct Item {
        int head, kvh, q0, rows_here, n_kv;
        bool valid;
    };
    auto item_of = [&](int r) {
        Item it;
        const int pos = r * (int)gridDim.x + ((r & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
        it.valid = pos < n_items;
        const int pp = it.valid ? pos : 0;
        it.head = pp % p.num_heads;
        it.kvh = it.head / p.group;
        it.q0 = (p.n_qblocks - 1 - pp / p.num_heads) * kTile;
        it.rows_here = min(kTile, p.seq_q - it.q0);
        const int k_end = min(p.seq_kv, p.start_pos + it.q0 + it.rows_here);  // exclusive: last visible key + 1
        it.n_kv = (k_end + kTile - 1) / kTile;
        return it;
    };

    if (threadIdx.x == 0) {
        mbar_init(&sh->q_full, 1);
        mbar_init(&sh->q_empty, 1);
        for (int i = 0; i < kStages; i++) {
            mbar_init(&sh->k_full[i], 1);
            mbar_init(&sh->k_empty[i], 1);
            mbar_init(&sh->v_full[i], 1);
            mbar_init(&sh->v_empty[i], 2);  // both output-MMA issuers commit
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(&sh->s_full[i], 1);
            mbar_init(&sh->s_free[i], 2);
            mbar_init(&sh->p_ready[i], 256);
        }
        mbar_init(&sh->o_final, 2);
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
    const uint32_t tmem_o = tmem + 2 * kTile;

    if (warp < 4) {
        setmaxnreg_dec<56>();  // producer / MMA warpgroup gives registers up
        if (warp == 0) {
            // -------------------------------------------------------------- TMA producer
            if (lane == 0) {
                tma_prefetch_desc(&qmap);
                tma_prefetch_desc(&kmap);
                tma_prefetch_desc(&vmap);
                int items_done = 0;
                bool ok = true;
                int st = 0;
                uint32_t ph = 1;  // a fresh barrier passes a wait on parity 1
                for (int r = 0; r < n_rounds && ok; r++) {
                    const Item it = item_of(r);
                    if (!it.valid) continue;
                    // the query tile is reloaded once the last score MMA of the previous item is done
                    ok = mbar_wait(&sh->q_empty, (items_done & 1) ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&sh->q_full, kQTiles * kTileBytes);
                    for (int c = 0; c < 2; c++) {
                        tma_load_2d(q_smem + c * kChunkBytes, &qmap, &sh->q_full, it.head * kTile + c * 64, it.q0);
                        if (kSplitQ)
                            tma_load_2d(q_smem + kTileBytes + c * kChunkBytes, &qlomap, &sh->q_full, it.head * kTile + c * 64, it.q0);
                    }
                    items_done++;
                    for (int j = 0; j < it.n_kv; j++) {
                        const int y = it.kvh * p.max_seq + j * kTile;
                        ok = mbar_wait(&sh->k_empty[st], ph, abort_flag);
                        if (!ok) break;
                        mbar_arrive_expect_tx(&sh->k_full[st], kTileBytes);
                        for (int c = 0; c < 2; c++)
                            tma_load_2d(k_smem + st * kTileBytes + c * kChunkBytes, &kmap, &sh->k_full[st], c * 64, y);
                        ok = mbar_wait(&sh->v_empty[st], ph, abort_flag);
                        if (!ok) break;
                        mbar_arrive_expect_tx(&sh->v_full[st], kTileBytes);
                        for (int c = 0; c < 2; c++)
                            tma_load_2d(v_smem + st * kTileBytes + c * kChunkBytes, &vmap, &sh->v_full[st], c * 64, y);
                        if (++st == kStages) {
                            st = 0;
                            ph ^= 1;
                        }
                    }
                }
                if (!ok) atomicOr(p.status, kStatusTimeout);
            }
        } else if (warp == 1) {
            // -------------------------------------------------------------- score MMAs: S_b = Q K_j^T
            if (lane == 0) {
                constexpr uint32_t idesc_qk = umma_idesc_f16(kTile, kTile, false, false);
                const uint32_t q_lo = desc_lo(smem_u32(q_smem), 16);
                const uint32_t k_lo0 = desc_lo(smem_u32(k_smem), 16);
                bool ok = true;
                int st = 0, items_done = 0;
                uint32_t ph = 0;
                int g = 0;  // KV steps issued so far by this CTA, across items: S buffer = g & 1
                for (int r = 0; r < n_rounds && ok; r++) {
                    const Item it = item_of(r);
                    if (!it.valid) continue;
                    ok = mbar_wait(&sh->q_full, items_done & 1, abort_flag);
                    items_done++;
                    for (int j = 0; j < it.n_kv && ok; j++, g++) {
                        const int b = g & 1;
                        FA_TRACE(0, j, 0);
                        ok = mbar_wait(&sh->k_full[st], ph, abort_flag);
                        FA_TRACE(0, j, 1);
                        // S_b still holds P of step g-2 until both output-MMA halves of that step are done
                        if (ok && g >= 2) ok = mbar_wait(&sh->s_free[b], ((g >> 1) - 1) & 1, abort_flag);
                        if (!ok) break;
                        FA_TRACE(0, j, 2);
                        tc_fence_after_sync();
                        const uint32_t d = tmem + b * kTile;
                        const uint32_t k_lo = k_lo0 + st * (kTileBytes >> 4);
                        // K-major operands: 8 steps of 16 along head_dim (32 bytes inside the swizzled
                        // row, the second 64-wide block 16 KB further)
#pragma unroll
                        for (int ks = 0; ks < 8; ks++) {
                            const uint32_t off = ((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4;
                            umma_ss_words(d, q_lo + off, k_lo + off, kDescHiSw128, idesc_qk, ks > 0 ? 1u : 0u);
                        }
                        if (kSplitQ) {
#pragma unroll
                            for (int ks = 0; ks < 8; ks++) {
                                const uint32_t off = ((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4;
                                umma_ss_words(d, q_lo + (kTileBytes >> 4) + off, k_lo + off, kDescHiSw128, idesc_qk, 1u);
                            }
                        }
                        tc_commit(&sh->s_full[b]);
                        tc_commit(&sh->k_empty[st]);
                        if (j + 1 == it.n_kv) tc_commit(&sh->q_empty);  // the query tile may be replaced
                        FA_TRACE(0, j, 3);
                        if (++st == kStages) {
                            st = 0;
                            ph ^= 1;
                        }
                    }
                }
                if (!ok) atomicOr(p.status, kStatusTimeout);
            }
        } else {
            // -------------------------------------------------------------- output MMAs: O += P_b V_j
            // warp 2 multiplies the hi half of P, warp 3 the lo half; O was zeroed by the softmax
            // warps, so every MMA accumulates and the two issuers need no order between them
            if (lane == 0) {
                constexpr uint32_t idesc_pv = umma_idesc_f16(kTile, kTile, false, true);
                const uint32_t part = warp - 2;  // 0: hi, 1: lo
                const uint32_t v_lo0 = desc_lo(smem_u32(v_smem), kChunkBytes);
                bool ok = true;
                int st = 0;
                uint32_t ph = 0;
                int g = 0;
                for (int r = 0; r < n_rounds && ok; r++) {
                    const Item it = item_of(r);
                    if (!it.valid) continue;
                    for (int j = 0; j < it.n_kv; j++, g++) {
                        const int b = g & 1;
                        if (part == 0) FA_TRACE(1, j, 0);
                        ok = mbar_wait(&sh->v_full[st], ph, abort_flag) && mbar_wait(&sh->p_ready[b], (g >> 1) & 1, abort_flag);
                        if (!ok) break;
                        if (part == 0) FA_TRACE(1, j, 1);
                        tc_fence_after_sync();
                        const uint32_t v_lo = v_lo0 + st * (kTileBytes >> 4);
                        // P: each 64-column half of S_b became 32 columns of hi + 32 of lo (8 columns per
                        // 16 keys); V MN-major: 16 keys = 2 KB further per step, second 64 dims via LBO
#pragma unroll
                        for (int ks = 0; ks < 8; ks++) {
                            const uint32_t a = tmem + b * kTile + (ks >> 2) * 64 + (ks & 3) * 8 + part * 32;
                            umma_ts_words(tmem_o, a, v_lo + ks * (2048 >> 4), kDescHiSw128, idesc_pv, 1u);
                        }
                        tc_commit(&sh->s_free[b]);
                        tc_commit(&sh->v_empty[st]);
                        if (j + 1 == it.n_kv) tc_commit(&sh->o_final);
                        if (part == 0) FA_TRACE(1, j, 2);
                        if (++st == kStages) {
                            st = 0;
                            ph ^= 1;
                        }
                    }
                }
                if (!ok) atomicOr(p.status, kStatusTimeout);
            }
        }
    } else {
        setmaxnreg_inc<224>();
        // ------------------------------------------------------------------ softmax + epilogue
        const int wg = (warp - 4) >> 2;          // 0: key columns 0-63 of each tile, 1: columns 64-127
        const int quarter = warp & 3;            // TMEM lane quarter this warp may touch
        const int row = quarter * 32 + lane;     // query row inside the tile
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
        const uint32_t o_addr = lane_base + 2 * kTile + wg * 64;  // this thread's half of the O row
        bool ok = true;
        int g = 0, items_done = 0;  // KV steps / items handled so far by this CTA
        for (int r = 0; r < n_rounds; r++) {
        const Item it = item_of(r);
        if (!it.valid) continue;
        const int q0 = it.q0, n_kv = it.n_kv, head = it.head, rows_here = it.rows_here;
        if (warp == 4) FA_TRACE(3, r, 0);
        const int q_pos = q0 + row;
        const int last_visible = min(p.start_pos + q_pos, p.seq_kv - 1);  // key index
        {
            // O starts at zero so that every output MMA can accumulate
            uint32_t z[32];
#pragma unroll
            for (int c = 0; c < 32; c++) z[c] = 0u;
            tmem_st32(o_addr, z);
            tmem_st32(o_addr + 32, z);
            tmem_wait_st();
        }
        float m_used = -INFINITY, l_run = 0.f;
        for (int j = 0; j < n_kv; j++, g++) {
            const int b = g & 1;
            const uint32_t s_addr = lane_base + b * kTile + wg * 64;
            if (warp == 4) FA_TRACE(2, j, 0);
            if (ok) ok = mbar_wait(&sh->s_full[b], (g >> 1) & 1, abort_flag);
            if (warp == 4) FA_TRACE(2, j, 1);
            if (!ok) {  // keep the barrier count intact so nobody is left waiting
                softmax_group_sync();
                continue;
            }
            tc_fence_after_sync();
            const int k0 = j * kTile;
            const bool need_mask = (k0 + kTile - 1 > p.start_pos + q0) || (k0 + kTile > p.seq_kv);
            const int limit = last_visible - k0 - wg * 64;  // own column c is visible iff c <= limit
            // this thread's 64 scores into registers: two loads in flight, one wait
            uint32_t x0[32], x1[32];
            tmem_ld32(s_addr, x0);
            tmem_ld32(s_addr + 32, x1);
            tmem_wait_ld();
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < 32; c++) {
                    if (c > limit) x0[c] = 0xFF800000u;  // -inf
                    if (32 + c > limit) x1[c] = 0xFF800000u;
                }
            }
            float mx;
            {
                float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                for (int c = 0; c < 32; c += 4) {
                    m0 = fmaxf(m0, fmaxf(__uint_as_float(x0[c]), __uint_as_float(x0[c + 1])));
                    m1 = fmaxf(m1, fmaxf(__uint_as_float(x0[c + 2]), __uint_as_float(x0[c + 3])));
                    m2 = fmaxf(m2, fmaxf(__uint_as_float(x1[c]), __uint_as_float(x1[c + 1])));
                    m3 = fmaxf(m3, fmaxf(__uint_as_float(x1[c + 2]), __uint_as_float(x1[c + 3])));
                }
                mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
            }
            // the other warpgroup holds the other 64 columns of the same row
            sh->xchg[b][wg][row] = mx;
            softmax_group_sync();
            mx = fmaxf(mx, sh->xchg[b][wg ^ 1][row]) * p.scale_log2;
            if (warp == 4) FA_TRACE(2, j, 2);
            if (j == 0) {
                m_used = mx;
            } else {
                const bool grow = mx > m_used + kLazyRescaleLog2;
                if (__any_sync(0xffffffffu, grow)) {
                    // O must be quiescent: wait until both halves of the previous output MMA are done
                    ok = mbar_wait(&sh->s_free[(g - 1) & 1], ((g - 1) >> 1) & 1, abort_flag);
                    tc_fence_after_sync();
                    const float alpha = grow ? fast_exp2(m_used - mx) : 1.0f;
                    if (grow) m_used = mx;
                    l_run *= alpha;
                    uint32_t r[32];
#pragma unroll 1
                    for (int ch = 0; ch < 2; ch++) {
                        tmem_ld32(o_addr + ch * 32, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; c++) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
                        tmem_st32(o_addr + ch * 32, r);
                    }
                }
            }
            // P = 2^(s*scale - m): fp16 hi in columns [0,32) of this thread's half, lo in [32,64)
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
                    split_hi_lo(p0, p1, hi[c >> 1], lo[c >> 1]);
                }
                tmem_st16(s_addr + chunk * 16, hi);
                tmem_st16(s_addr + 32 + chunk * 16, lo);
            };
            emit(x0, 0);
            emit(x1, 1);
            l_run += ((ls[0] + ls[1]) + (ls[2] + ls[3])) + ((ls[4] + ls[5]) + (ls[6] + ls[7]));
            if (wg == 0 && k0 + kTile > p.seq_kv) {
                // keys past seq_kv carry P = 0, but their V rows may hold anything (even NaN):
                // zero them in shared memory before the MMAs read the tile
                const int st = g % kStages;
                ok = mbar_wait(&sh->v_full[st], (g / kStages) & 1, abort_flag);
                const int first_bad = p.seq_kv - k0;
                uint8_t* vt = v_smem + st * kTileBytes;
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
            mbar_arrive(&sh->p_ready[b]);
            if (warp == 4) FA_TRACE(2, j, 3);
        }
        // row sums of the two halves
        sh->xchg[g & 1][wg][row] = l_run;
        softmax_group_sync();
        const float l_total = l_run + sh->xchg[g & 1][wg ^ 1][row];
        softmax_group_sync();  // the slot is reused by the next item's first step
        if (warp == 4) FA_TRACE(3, r, 1);
        if (ok) ok = mbar_wait(&sh->o_final, items_done & 1, abort_flag);
        if (warp == 4) FA_TRACE(3, r, 2);
        items_done++;
        if (ok) {
            tc_fence_after_sync();
            const float inv = 1.0f / l_total;
            const bool store = row < rows_here;
            uint32_t r[32];
#pragma unroll 1
            for (int ch = 0; ch < 2; ch++) {
                __syncwarp();
                tmem_ld32(o_addr + ch * 32, r);
                tmem_wait_ld();
                if (store) {
                    const size_t base = ((size_t)q_pos * p.num_heads + head) * kTile + wg * 64 + ch * 32;
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
        if (warp == 4) FA_TRACE(3, r, 3);
        }  // items
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

    // Q (1 or 2 tiles) + K and V rings: 3 stages fit beside one query tile, 2 beside two
    const int stages = split_q ? 2 : 3;
    size_t smem_bytes = (sizeof(FaSmem) + 1023) / 1024 * 1024 + 1024 + (size_t)((split_q ? 2 : 1) + 2 * stages) * kTileBytes;
    if (smem_bytes > (size_t)c->smem_optin) smem_bytes = (size_t)c->smem_optin;  // the window is 1 KB aligned in practice
    auto kern = split_q ? prefill_fa_kernel<true, 2> : prefill_fa_kernel<false, 3>;
    GB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    const int n_items = p.n_qblocks * p.num_heads;
    const int grid = n_items < c->sm_count ? n_items : c->sm_count;  // persistent CTAs, one per SM
#ifdef GB_FA_TRACE
    static unsigned long long* trace_buf = nullptr;
    if (!trace_buf) cudaMallocManaged(&trace_buf, 4 * 64 * sizeof(unsigned long long));
    memset(trace_buf, 0, 4 * 64 * sizeof(unsigned long long));
    p.trace = trace_buf;
#endif
    {
        LaunchScope t(c, "prefill_causal_fa");
        kern<<<grid, kFaThreads, smem_bytes, c->stream>>>(*qmap, *qlomap, *kmap, *vmap, p);
    }
#ifdef GB_FA_TRACE
    cudaStreamSynchronize(c->stream);
    {
        const unsigned long long t0 = trace_buf[3 * 64 + 0];  // first item start
        const char* roles[4] = {"qk ", "pvh", "smx", "itm"};
        for (int step = 0; step < 16; step++)
            for (int r = 0; r < 4; r++)
                fprintf(stderr, "trace %s step %2d: %8lld %8lld %8lld %8lld\n", roles[r], step,
                        (long long)(trace_buf[r * 64 + step * 4 + 0] - t0), (long long)(trace_buf[r * 64 + step * 4 + 1] - t0),
                        (long long)(trace_buf[r * 64 + step * 4 + 2] - t0), (long long)(trace_buf[r * 64 + step * 4 + 3] - t0));
    }
#endif
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

}  // namespace gb200
