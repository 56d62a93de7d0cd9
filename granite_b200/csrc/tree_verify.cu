// Tree-masked attention for speculative-decoding verification on tcgen05/TMEM.
//
// Replaces attention_tree_f16kv / attention_tree_nocontext_f16kv
// (src/backend/metal/kernels/metal_shaders_attention.h:1677, :1869, dispatched by
// MetalCompute::attention_tree, src/backend/metal/metal_compute.mm:2463-2529); the arithmetic it
// must match is the CPU loop src/llm/transformer.mm:2044-2126 with the ancestor mask of
// src/llm/transformer.mm:823-840.  Beyond the reference it takes a batch of sequences and a
// committed prefix that lives in the paged pool (block table) as well as in a contiguous cache.
//
// Every draft node attends to the whole committed prefix and, among the tree nodes, to itself
// and its ancestors.  For one (sequence, KV head) the query rows are (query head of the group,
// node): 64 node slots per head, two heads per 128-row tile, two tiles per CTA.  The prefix is
// consumed in 128-key tiles (8 pages each when paged); the last step is the 64-key tile of the
// tree's own K/V, whose scores are masked by a 64-bit ancestor word per node.
// Same machinery as the causal prefill kernel: TMA -> 128-byte-swizzled shared memory ->
// tcgen05.mma with S and O in TMEM, P written back over S as fp16 hi + lo, lazy rescale of O.
#include "compute_internal.h"
#include "ptx.cuh"

namespace gb200 {

constexpr int kTvThreads = 384;
constexpr int kTvTile = 128;
constexpr int kTvTileBytes = kTvTile * kTvTile * 2;
constexpr int kTvChunkBytes = kTvTileBytes / 2;
constexpr int kNodeSlots = 64;        // tree nodes per sequence the kernel is laid out for
constexpr int kTvPage = 16;
constexpr float kTvLazyLog2 = 8.0f;

struct TreeParams {
    float* out;                 // [batch, Hq, N, 128] fp32
    const int32_t* parents;     // [batch, N]
    const int32_t* tables;      // [batch, max_blocks] (paged) or nullptr
    const int32_t* cache_lens;  // [batch] or nullptr
    int batch, num_heads, num_kv_heads, group, num_nodes;
    int cache_len;              // used when cache_lens == nullptr
    int cache_stride;           // contiguous cache: rows per (sequence, KV head)
    int max_blocks, num_blocks;
    int ctas_per_unit;          // CTAs per (sequence, KV head)
    float scale_log2;
    int* status;
};

struct TreeSmem {
    uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_ready[2], o_final[2];
    uint32_t tmem_base;
    int abort_flag;
    int parents[kNodeSlots];
};

// Ancestor word of one node: bit j set when the node may attend to tree node j (itself or an
// ancestor).  Follows src/llm/transformer.mm:829-839; the walk is cut after n hops, which changes
// nothing for an acyclic parent array.  Parents outside [-1, n) end the walk (and are reported).
__device__ __forceinline__ unsigned long long ancestor_word(const int* parents, int node, int n) {
    unsigned long long w = 1ull << node;
    int cur = parents[node];
    for (int hops = 0; cur >= 0 && cur < n && hops < n; hops++) {
        w |= 1ull << cur;
        cur = parents[cur];
    }
    return w;
}

// masks[b * n + i] = ancestor word of node i of sequence b.
__global__ void tree_mask_kernel(const int32_t* parents, unsigned long long* masks, int batch, int n, int* status) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= batch * n) return;
    const int b = idx / n, i = idx % n;
    const int32_t* p = parents + (size_t)b * n;
    if (p[i] < -1 || p[i] >= n) atomicOr(status, kStatusBadParent);
    masks[idx] = ancestor_word(p, i, n);
}

template <bool kSplitQ, bool kPaged>
__global__ void __launch_bounds__(kTvThreads, 1)
tree_verify_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap qlomap,
                   const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                   const __grid_constant__ CUtensorMap ktmap, const __grid_constant__ CUtensorMap vtmap,
                   TreeParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_smem = smem;
    uint8_t* k_smem = smem + 2 * kTvTileBytes;
    uint8_t* v_smem = smem + 4 * kTvTileBytes;
    TreeSmem* sh = reinterpret_cast<TreeSmem*>(smem + 6 * kTvTileBytes);
    volatile int* abort_flag = &sh->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int item = blockIdx.x;
    const int sub = item % p.ctas_per_unit; item /= p.ctas_per_unit;
    const int kvh = item % p.num_kv_heads;
    const int b = item / p.num_kv_heads;
    // heads of the group owned by this CTA: two per tile; one tile when the query is split
    const int heads_per_cta = kSplitQ ? 2 : 4;
    const int g0 = sub * heads_per_cta;                 // first head (inside the group)
    const bool valid1 = !kSplitQ && (g0 + 2 < p.group);
    const int N = p.num_nodes;

    int cache_len = p.cache_lens ? p.cache_lens[b] : p.cache_len;
    const int cap = kPaged ? p.max_blocks * kTvPage : p.cache_stride;
    if (cache_len < 0 || cache_len > cap) {
        if (threadIdx.x == 0) atomicOr(p.status, kStatusBadSeqLen);
        cache_len = 0;
    }
    const int n_prefix = (cache_len + kTvTile - 1) / kTvTile;
    const int n_steps = n_prefix + 1;  // the last step is the tree tile

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
    if (threadIdx.x < kNodeSlots) {
        int par = -1;
        if ((int)threadIdx.x < N) {
            par = p.parents[(size_t)b * N + threadIdx.x];
            if (par < -1 || par >= N) {
                atomicOr(p.status, kStatusBadParent);
                par = -1;
            }
        }
        sh->parents[threadIdx.x] = par;
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
        // ------------------------------------------------------------------ TMA producer (whole warp)
        if (lane == 0) {
            tma_prefetch_desc(&qmap);
            tma_prefetch_desc(&kmap);
            tma_prefetch_desc(&vmap);
            tma_prefetch_desc(&ktmap);
            tma_prefetch_desc(&vtmap);
            // Q rows: z = absolute head, y = node; a box is 64 halfs x 64 nodes x 2 heads (16 KB)
            const int z0 = b * p.num_heads + kvh * p.group + g0;
            if (kSplitQ) {
                mbar_arrive_expect_tx(&sh->q_full, 2 * kTvTileBytes);
                for (int c = 0; c < 2; c++) {
                    tma_load_3d(q_smem + c * kTvChunkBytes, &qmap, &sh->q_full, c * 64, 0, z0);
                    tma_load_3d(q_smem + kTvTileBytes + c * kTvChunkBytes, &qlomap, &sh->q_full, c * 64, 0, z0);
                }
            } else {
                mbar_arrive_expect_tx(&sh->q_full, (valid1 ? 2 : 1) * kTvTileBytes);
                for (int t = 0; t < (valid1 ? 2 : 1); t++)
                    for (int c = 0; c < 2; c++)
                        tma_load_3d(q_smem + t * kTvTileBytes + c * kTvChunkBytes, &qmap, &sh->q_full, c * 64, 0, z0 + 2 * t);
            }
        }
        // page entries of the next prefix tile are fetched one tile ahead (lanes 0-7, one page each)
        auto load_entry = [&](int j) {
            int e = 0;
            if (kPaged && j < n_prefix && lane < 8) {
                const int logical = j * 8 + lane;
                if (logical * kTvPage < cache_len) {
                    e = p.tables[(size_t)b * p.max_blocks + logical];
                    if (e < 0 || e >= p.num_blocks) {
                        atomicOr(p.status, kStatusBadTable);
                        e = 0;
                    }
                }
            }
            return e;
        };
        int entry_next = load_entry(0);
        for (int j = 0; j < n_steps; j++) {
            const int s = j & 1;
            const uint32_t ph = ((j >> 1) & 1) ^ 1;
            const bool tree_step = j == n_prefix;
            const int entry = entry_next;
            entry_next = load_entry(j + 1);
            const uint32_t bytes = tree_step ? kTvTileBytes / 2 : kTvTileBytes;
            int ok = 1;
            if (lane == 0) {
                ok = mbar_wait(&sh->k_empty[s], ph, abort_flag) && mbar_wait(&sh->v_empty[s], ph, abort_flag);
                if (ok) {
                    mbar_arrive_expect_tx(&sh->k_full[s], bytes);
                    mbar_arrive_expect_tx(&sh->v_full[s], bytes);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) {
                if (lane == 0) atomicOr(p.status, kStatusTimeout);
                break;
            }
            uint8_t* kd = k_smem + s * kTvTileBytes;
            uint8_t* vd = v_smem + s * kTvTileBytes;
            if (tree_step) {
                // tree K/V [batch, Hkv, N, 128]: 64-row boxes; rows >= N are zero-filled by TMA
                if (lane < 4) {
                    const int c = lane & 1;
                    const bool is_v = lane >= 2;
                    tma_load_3d((is_v ? vd : kd) + c * kTvChunkBytes, is_v ? &vtmap : &ktmap,
                                is_v ? &sh->v_full[s] : &sh->k_full[s], c * 64, 0, b * p.num_kv_heads + kvh);
                }
            } else if (kPaged) {
                // lane = (tensor, page, chunk): 8 pages x 2 chunks for K, the same for V
                const int pg = (lane >> 1) & 7, c = lane & 1;
                const bool is_v = lane >= 16;
                const int e = __shfl_sync(0xffffffffu, entry, pg);
                tma_load_2d((is_v ? vd : kd) + c * kTvChunkBytes + pg * 2048, is_v ? &vmap : &kmap,
                            is_v ? &sh->v_full[s] : &sh->k_full[s], kvh * kTvTile + c * 64, e * kTvPage);
            } else if (lane < 4) {
                const int c = lane & 1;
                const bool is_v = lane >= 2;
                tma_load_2d((is_v ? vd : kd) + c * kTvChunkBytes, is_v ? &vmap : &kmap,
                            is_v ? &sh->v_full[s] : &sh->k_full[s], c * 64,
                            (b * p.num_kv_heads + kvh) * p.cache_stride + j * kTvTile);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_qk = umma_idesc_f16(kTvTile, kTvTile, false, false);
            constexpr uint32_t idesc_pv = umma_idesc_f16(kTvTile, kTvTile, false, true);
            constexpr uint32_t idesc_qk_tree = umma_idesc_f16(kTvTile, kNodeSlots, false, false);
            const uint32_t q_addr = smem_u32(q_smem), k_addr = smem_u32(k_smem), v_addr = smem_u32(v_smem);
            const uint32_t q_lo[2] = {desc_lo(q_addr, 16), desc_lo(q_addr + kTvTileBytes, 16)};
            const uint32_t k_lo[2] = {desc_lo(k_addr, 16), desc_lo(k_addr + kTvTileBytes, 16)};
            const uint32_t v_lo[2] = {desc_lo(v_addr, kTvChunkBytes), desc_lo(v_addr + kTvTileBytes, kTvChunkBytes)};
            auto issue_qk = [&](int t, int s, bool tree_step) {
                const uint32_t idesc = tree_step ? idesc_qk_tree : idesc_qk;
                const uint32_t d = tmem + t * kTvTile;
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    const uint32_t off = ((ks >> 2) * kTvChunkBytes + (ks & 3) * 32) >> 4;
                    umma_ss_words(d, q_lo[t] + off, k_lo[s] + off, kDescHiSw128, idesc, ks > 0 ? 1u : 0u);
                }
                if (kSplitQ) {
#pragma unroll
                    for (int ks = 0; ks < 8; ks++) {
                        const uint32_t off = ((ks >> 2) * kTvChunkBytes + (ks & 3) * 32) >> 4;
                        umma_ss_words(d, q_lo[1] + off, k_lo[s] + off, kDescHiSw128, idesc, 1u);
                    }
                }
            };
            auto issue_pv = [&](int t, int s, bool acc, bool tree_step) {
                const int nks = tree_step ? 4 : 8;  // 16 keys per step
                const uint32_t d = tmem + 2 * kTvTile + t * kTvTile;
#pragma unroll
                for (int ks = 0; ks < 8; ks++) {
                    if (ks < nks) {
                        const uint32_t vl = v_lo[s] + ks * (2048 >> 4);
                        const uint32_t a_hi = tmem + t * kTvTile + (ks >> 2) * 64 + (ks & 3) * 8;
                        umma_ts_words(d, a_hi, vl, kDescHiSw128, idesc_pv, (acc || ks > 0) ? 1u : 0u);
                        umma_ts_words(d, a_hi + 32, vl, kDescHiSw128, idesc_pv, 1u);
                    }
                }
            };
            bool ok = mbar_wait(&sh->q_full, 0, abort_flag) && mbar_wait(&sh->k_full[0], 0, abort_flag);
            if (ok) {
                tc_fence_after_sync();
                issue_qk(0, 0, n_prefix == 0);
                tc_commit(&sh->s_full[0]);
                if (valid1) {
                    issue_qk(1, 0, n_prefix == 0);
                    tc_commit(&sh->s_full[1]);
                }
                tc_commit(&sh->k_empty[0]);
            }
            for (int j = 0; j < n_steps && ok; j++) {
                const int s = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                const bool more = j + 1 < n_steps;
                const int s2 = (j + 1) & 1;
                const uint32_t ph2 = ((j + 1) >> 1) & 1;
                const bool tree_now = j == n_prefix, tree_next = j + 1 == n_prefix;
                ok = mbar_wait(&sh->v_full[s], ph, abort_flag) && mbar_wait(&sh->p_ready[0], j & 1, abort_flag);
                if (!ok) break;
                tc_fence_after_sync();
                issue_pv(0, s, j > 0, tree_now);
                if (!more) tc_commit(&sh->o_final[0]);
                if (more) {
                    ok = mbar_wait(&sh->k_full[s2], ph2, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_qk(0, s2, tree_next);
                    tc_commit(&sh->s_full[0]);
                }
                if (valid1) {
                    ok = mbar_wait(&sh->p_ready[1], j & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_pv(1, s, j > 0, tree_now);
                    if (!more) tc_commit(&sh->o_final[1]);
                }
                tc_commit(&sh->v_empty[s]);
                if (more) {
                    if (valid1) {
                        issue_qk(1, s2, tree_next);
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
        const int t = (warp - 4) >> 2;
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        if (t == 0 || valid1) {
            const uint32_t lane_base = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
            const uint32_t s_addr = lane_base + t * kTvTile;
            const uint32_t o_addr = lane_base + 2 * kTvTile + t * kTvTile;
            const int node = row & (kNodeSlots - 1);
            const int g = g0 + 2 * t + (row >> 6);  // head inside the group
            const bool row_valid = node < N && g < p.group;
            const unsigned long long anc = node < N ? ancestor_word(sh->parents, node, N) : 1ull;
            float m_used = -INFINITY, l_run = 0.f;
            bool ok = true;
            for (int j = 0; j < n_steps; j++) {
                ok = mbar_wait(&sh->s_full[t], j & 1, abort_flag);
                if (!ok) break;
                tc_fence_after_sync();
                const bool tree_step = j == n_prefix;
                const int k0 = j * kTvTile;
                const bool need_mask = tree_step || (k0 + kTvTile > cache_len);
                const int limit = cache_len - 1 - k0;  // prefix tile: column c is visible iff c <= limit
                auto visible = [&](int col) {
                    return tree_step ? ((anc >> col) & 1ull) != 0 : col <= limit;
                };
                // S row into registers (128 columns for a prefix tile, 64 for the tree tile)
                uint32_t x0[32], x1[32], x2[32], x3[32];
                tmem_ld32(s_addr, x0);
                tmem_ld32(s_addr + 32, x1);
                if (!tree_step) {
                    tmem_ld32(s_addr + 64, x2);
                    tmem_ld32(s_addr + 96, x3);
                }
                tmem_wait_ld();
                if (tree_step) {
#pragma unroll
                    for (int c = 0; c < 32; c++) {
                        if (!((anc >> c) & 1ull)) x0[c] = 0xFF800000u;         // -inf
                        if (!((anc >> (32 + c)) & 1ull)) x1[c] = 0xFF800000u;
                        x2[c] = 0xFF800000u;
                        x3[c] = 0xFF800000u;
                    }
                } else if (need_mask) {
#pragma unroll
                    for (int c = 0; c < 32; c++) {
                        if (c > limit) x0[c] = 0xFF800000u;
                        if (32 + c > limit) x1[c] = 0xFF800000u;
                        if (64 + c > limit) x2[c] = 0xFF800000u;
                        if (96 + c > limit) x3[c] = 0xFF800000u;
                    }
                }
                float mx;
                {
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
                    const bool grow = mx > m_used + kTvLazyLog2;
                    if (__any_sync(0xffffffffu, grow)) {
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
                float ls[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                const float neg_m = -m_used;
                auto emit = [&](uint32_t (&x)[32], int chunk) {
                    uint32_t hi[16], lo[16];
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        const float p0 = fast_exp2(fmaf(__uint_as_float(x[c]), p.scale_log2, neg_m));
                        const float p1 = fast_exp2(fmaf(__uint_as_float(x[c + 1]), p.scale_log2, neg_m));
                        ls[c & 6] += p0;
                        ls[(c & 6) + 1] += p1;
                        split_hi_lo(p0, p1, hi[c >> 1], lo[c >> 1]);
                    }
                    tmem_st16(s_addr + (chunk >> 1) * 64 + (chunk & 1) * 16, hi);
                    tmem_st16(s_addr + (chunk >> 1) * 64 + 32 + (chunk & 1) * 16, lo);
                };
                emit(x0, 0);
                emit(x1, 1);
                if (!tree_step) {
                    emit(x2, 2);
                    emit(x3, 3);
                }
                l_run += ((ls[0] + ls[1]) + (ls[2] + ls[3])) + ((ls[4] + ls[5]) + (ls[6] + ls[7]));
                if (t == 0 && !tree_step && k0 + kTvTile > cache_len) {
                    // prefix keys past cache_len carry P = 0 but their V rows may hold anything
                    const int s = j & 1;
                    ok = mbar_wait(&sh->v_full[s], (j >> 1) & 1, abort_flag);
                    if (!ok) break;
                    const int first_bad = cache_len - k0;
                    uint8_t* vt = v_smem + s * kTvTileBytes;
                    for (int i = row; i < (kTvTile - first_bad) * 16; i += 128) {
                        const int rr = first_bad + (i >> 4), u = i & 15;
                        *reinterpret_cast<uint4*>(vt + (u >> 3) * kTvChunkBytes + rr * 128 + (((u & 7) ^ (rr & 7)) << 4)) =
                            make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();
                }
                __syncwarp();
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&sh->p_ready[t]);
            }
            if (ok) ok = mbar_wait(&sh->o_final[t], 0, abort_flag);
            if (ok) {
                tc_fence_after_sync();
                const float inv = 1.0f / l_run;
                const int head = kvh * p.group + g;
                uint32_t r[32];
#pragma unroll 1
                for (int ch = 0; ch < 4; ch++) {
                    __syncwarp();
                    tmem_ld32(o_addr + ch * 32, r);
                    tmem_wait_ld();
                    if (row_valid) {
                        float4* dst = reinterpret_cast<float4*>(
                            p.out + (((size_t)b * p.num_heads + head) * N + node) * kTvTile + ch * 32);
#pragma unroll
                        for (int v = 0; v < 8; v++)
                            dst[v] = make_float4(__uint_as_float(r[v * 4 + 0]) * inv, __uint_as_float(r[v * 4 + 1]) * inv,
                                                 __uint_as_float(r[v * 4 + 2]) * inv, __uint_as_float(r[v * 4 + 3]) * inv);
                    }
                }
            } else if (lane == 0) {
                atomicOr(p.status, kStatusTimeout);
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
    }
}

__global__ void tree_split_q_kernel(const float* __restrict__ src, __half* __restrict__ hi,
                                    __half* __restrict__ lo, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float x = src[i];
        const __half h = __float2half_rn(x);
        hi[i] = h;
        lo[i] = __float2half_rn(x - __half2float(h));
    }
}

// ------------------------------------------------------------------------------------ host
int launch_tree_mask(granite_cuda_compute* c, const int32_t* parents, uint64_t* masks, uint32_t batch, uint32_t n) {
    if (!parents || !masks) return fail(GRANITE_CUDA_NULL_POINTER, "tree mask: null buffer");
    if (n == 0 || n > (uint32_t)kNodeSlots)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "tree mask: num_nodes must be in [1, 64]");
    if (batch == 0) return GRANITE_CUDA_SUCCESS;
    LaunchScope t(c, "tree_mask");
    const uint32_t total = batch * n;
    tree_mask_kernel<<<(total + 127) / 128, 128, 0, c->stream>>>(parents, reinterpret_cast<unsigned long long*>(masks),
                                                                 (int)batch, (int)n, c->d_status);
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

int launch_tree_verify(granite_cuda_compute* c, const GraniteCudaTreeAttentionArgs& a) {
    if (!a.q || !a.k_tree || !a.v_tree || !a.parent_indices || !a.output)
        return fail(GRANITE_CUDA_NULL_POINTER, "attention_tree: null buffer");
    if (a.head_dim != kTvTile) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: head_dim must be 128");
    if (a.num_nodes == 0 || a.num_nodes > (uint32_t)kNodeSlots)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: num_nodes must be in [1, 64]");
    if (a.num_kv_heads == 0 || a.num_heads % a.num_kv_heads != 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: num_heads must be a multiple of num_kv_heads");
    if (a.q_dtype > 1) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: q_dtype must be 0 (fp32) or 1 (fp16)");
    if (a.batch_size == 0) return GRANITE_CUDA_SUCCESS;
    const bool paged = a.block_tables != nullptr;
    const bool has_cache = a.cache_lens != nullptr || a.cache_len > 0;
    if (has_cache && (!a.k_cache || !a.v_cache)) return fail(GRANITE_CUDA_NULL_POINTER, "attention_tree: null cache");
    if (paged && (a.block_size != (uint32_t)kTvPage || a.num_blocks == 0 || a.max_blocks_per_seq == 0))
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: paged prefix needs block_size 16 and a non-empty pool");
    const uint32_t cache_stride = a.cache_stride ? a.cache_stride : a.cache_len;
    if (!paged && has_cache && a.cache_len > cache_stride)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: cache_len exceeds cache_stride");

    const bool split_q = a.q_dtype == 0;
    const size_t q_elems = (size_t)a.batch_size * a.num_heads * a.num_nodes * kTvTile;
    const void* q16 = a.q;
    const void* q16_lo = a.q;
    if (split_q) {
        const size_t half_bytes = (q_elems * 2 + 255) / 256 * 256;
        int rc = c->ensure_scratch(2 * half_bytes);
        if (rc) return rc;
        LaunchScope t(c, "split_q_f16");
        __half* hi = static_cast<__half*>(c->scratch);
        __half* lo = reinterpret_cast<__half*>(static_cast<uint8_t*>(c->scratch) + half_bytes);
        tree_split_q_kernel<<<(unsigned)((q_elems + 255) / 256), 256, 0, c->stream>>>(static_cast<const float*>(a.q), hi, lo, q_elems);
        q16 = hi;
        q16_lo = lo;
    }

    TreeParams p{};
    p.out = a.output;
    p.parents = a.parent_indices;
    p.tables = a.block_tables;
    p.cache_lens = a.cache_lens;
    p.batch = (int)a.batch_size;
    p.num_heads = (int)a.num_heads;
    p.num_kv_heads = (int)a.num_kv_heads;
    p.group = (int)(a.num_heads / a.num_kv_heads);
    p.num_nodes = (int)a.num_nodes;
    p.cache_len = (int)a.cache_len;
    p.cache_stride = (int)cache_stride;
    p.max_blocks = (int)a.max_blocks_per_seq;
    p.num_blocks = (int)a.num_blocks;
    p.ctas_per_unit = split_q ? (p.group + 1) / 2 : (p.group + 3) / 4;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.status = c->d_status;

    // Q / tree K / tree V as [heads, nodes, 128]: box = 64 halfs x 64 nodes x 2 heads (Q) or 1 head (K/V)
    const uint64_t qz = (uint64_t)a.batch_size * a.num_heads;
    const CUtensorMap* qmap = c->tensor_map_3d(q16, kTvTile, a.num_nodes, qz, kTvTile * 2, (uint64_t)a.num_nodes * kTvTile * 2,
                                               64, kNodeSlots, 2, 128);
    const CUtensorMap* qlomap = c->tensor_map_3d(q16_lo, kTvTile, a.num_nodes, qz, kTvTile * 2,
                                                 (uint64_t)a.num_nodes * kTvTile * 2, 64, kNodeSlots, 2, 128);
    const uint64_t tz = (uint64_t)a.batch_size * a.num_kv_heads;
    const CUtensorMap* ktmap = c->tensor_map_3d(a.k_tree, kTvTile, a.num_nodes, tz, kTvTile * 2,
                                                (uint64_t)a.num_nodes * kTvTile * 2, 64, kNodeSlots, 1, 128);
    const CUtensorMap* vtmap = c->tensor_map_3d(a.v_tree, kTvTile, a.num_nodes, tz, kTvTile * 2,
                                                (uint64_t)a.num_nodes * kTvTile * 2, 64, kNodeSlots, 1, 128);
    const CUtensorMap *kmap = ktmap, *vmap = vtmap;  // placeholders when there is no prefix
    if (has_cache) {
        if (paged) {
            const uint64_t rows = (uint64_t)a.num_blocks * kTvPage, width = (uint64_t)a.num_kv_heads * kTvTile;
            kmap = c->tensor_map_2d(a.k_cache, width, rows, width * 2, 64, kTvPage, 128);
            vmap = c->tensor_map_2d(a.v_cache, width, rows, width * 2, 64, kTvPage, 128);
        } else {
            const uint64_t rows = (uint64_t)a.batch_size * a.num_kv_heads * cache_stride;
            kmap = c->tensor_map_2d(a.k_cache, kTvTile, rows, kTvTile * 2, 64, kTvTile, 128);
            vmap = c->tensor_map_2d(a.v_cache, kTvTile, rows, kTvTile * 2, 64, kTvTile, 128);
        }
    }
    if (!qmap || !qlomap || !ktmap || !vtmap || !kmap || !vmap) return GRANITE_CUDA_EXECUTION_FAILED;

    const size_t smem_bytes = 1024 + 6 * kTvTileBytes + sizeof(TreeSmem);
    void (*kern)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, TreeParams);
    if (split_q) kern = paged ? tree_verify_kernel<true, true> : tree_verify_kernel<true, false>;
    else kern = paged ? tree_verify_kernel<false, true> : tree_verify_kernel<false, false>;
    GB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    const int grid = p.batch * p.num_kv_heads * p.ctas_per_unit;
    {
        LaunchScope t(c, "tree_verify");
        kern<<<grid, kTvThreads, smem_bytes, c->stream>>>(*qmap, *qlomap, *kmap, *vmap, *ktmap, *vtmap, p);
    }
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

}  // namespace gb200
