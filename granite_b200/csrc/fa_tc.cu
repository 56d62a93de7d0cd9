// Tensor-core attention for the two contraction-shaped paths, on tcgen05 + TMEM fed by TMA:
//
//   causal prefill        replaces flash_attention_prefill
//                         (src/backend/metal/kernels/metal_shaders_attention.h:1453, dispatched by
//                         MetalCompute::multihead_attention with seq_q > 1,
//                         src/backend/metal/metal_compute.mm:2333-2375); arithmetic to match: the CPU
//                         loop src/llm/transformer.mm:1779-1840 with k_pos > start_pos + q_pos -> -inf
//   tree verification     replaces attention_tree_f16kv / attention_tree_nocontext_f16kv
//                         (metal_shaders_attention.h:1677, :1869, dispatched by
//                         MetalCompute::attention_tree, metal_compute.mm:2463-2529); arithmetic to
//                         match: src/llm/transformer.mm:2044-2126 with the ancestor mask of :823-840.
//                         Beyond the reference: a batch of sequences, and a committed prefix that
//                         lives in the paged pool (block table) as well as in a contiguous cache.
//
// One pipeline serves both.  A work item is one or two 128-row query tiles that share every K/V
// tile (prefill: one query head at one query block; tree: the four query heads of a group, 2 heads x
// 64 node slots per tile) and the K/V tiles they may see.  CTAs are
// persistent, one per SM, and run their items back to back.  A "virtual step" is (K/V tile j,
// query tile t); S of consecutive virtual steps alternates between two TMEM buffers, so the score
// MMAs of the next virtual step run while the softmax of the current one is still working.
// Roles (384 threads):
//   warp 0      TMA producer: Q once per item, then K_j / V_j into shared-memory rings
//               (128-byte swizzle; a paged tile is 8 pages = 8 boxes of 4 KB issued by eight lanes).  It also
//               works out the CTA's items at start-up, and starts loading before tensor memory is allocated
//   warp 1      one thread issues the score MMAs S_b = Q_t K_j^T (operands in shared memory)
//   warps 2, 3  one thread each issues half of the output MMAs O_t += P_b V_j: warp 2 the fp16
//               "hi" part of P, warp 3 the "lo" part (P from TMEM, V from shared memory,
//               MN-major).  A single thread cannot issue 128x128x16 instructions fast enough to
//               keep the tensor pipe busy; three can.
//   warps 4-11  softmax: the two warps that may touch a TMEM lane quarter take 16 of its 32 rows
//               each and read S in the 16-lane fragment shape of tcgen05.ld, which spreads a row's
//               128 columns over the four threads of a quad: row maxima and sums are two shuffles,
//               nothing goes through shared memory and no warp waits for another inside a step.
//               P is written back over S as fp16 hi + lo (P keeps ~22 bits, as the fp32 reference
//               does); the running maximum is only raised when it grows by more than 2^8 (lazy
//               rescale of O).  With one tile per item O alternates between the two accumulators and
//               a finished item is read out behind the next item's first MMAs.
// TMEM (512 columns): S[0] | S[1] | O[0] | O[1], 128 fp32 columns each.
#include <cstring>

#include "compute_internal.h"
#include "ptx.cuh"

namespace gb200 {

constexpr int kTcThreads = 384;
constexpr int kT = 128;                      // query rows per tile, keys per K/V tile, head_dim
constexpr int kTileBytes = kT * kT * 2;      // 32 KB: one [128 x 128] fp16 tile
constexpr int kChunkBytes = kTileBytes / 2;  // 16 KB: one 64-column (128-byte) swizzle block
constexpr int kNodeSlots = 64;               // tree nodes per sequence the kernel is laid out for
constexpr int kPageRows = 16;
constexpr float kLazyLog2 = 8.0f;
constexpr int kMaxStages = 3;
constexpr uint32_t kNegInf = 0xFF800000u;

struct TcParams {
    int num_heads, num_kv_heads, group;
    int units_per_kvh;   // items per KV head (prefill: per query block; tree: per sequence)
    float scale_log2;
    int* status;
    // prefill
    void* out;           // [seq_q, Hq, 128] fp16 or fp32
    int out_fp16;
    int seq_q, seq_kv, max_seq, n_qblocks, start_pos;
    // tree
    float* tree_out;            // [batch, Hq, N, 128] fp32
    const int32_t* parents;     // [batch, N]
    const int32_t* tables;      // [batch, max_blocks] (paged) or nullptr
    const int32_t* cache_lens;  // [batch] or nullptr
    int batch, num_nodes, cache_len, cache_stride, max_blocks, num_blocks;
    int d_chunks;               // head_dim / 64: 2 (head_dim 128) or 1 (head_dim 64, half of every tile slot is used)
    int slot_shift;             // tree: a tile is (128 >> slot_shift) query heads x (1 << slot_shift) node slots
};

struct TcItem {
    int head0;      // first query head of the item
    int kvh;
    int b;          // tree: sequence
    int q0;         // prefill: first query row
    int rows_here;  // prefill: live rows of the query block
    int n_steps;    // K/V tiles to walk (tree: prefix tiles + 1)
    int n_prefix;   // tree: prefix tiles
    int cache_len;  // tree: prefix length
    bool valid;
};

constexpr int kMaxCachedItems = 32;  // work items of a CTA kept in shared memory (later rounds are derived on the fly)

struct TcSmem {
    uint64_t q_full, q_empty, k_full[kMaxStages], k_empty[kMaxStages], v_full[kMaxStages], v_empty[kMaxStages];
    uint64_t s_full[2], s_free[2], p_ready[2];
    // "the item's output MMAs are done", one barrier per item parity: a deferred read-out waits for item r while
    // item r + 1 runs, and a one-step item r + 1 could otherwise complete the same barrier a second time before a
    // slow warp has looked at it (the wait would then block on a phase that never ends)
    uint64_t o_final[2];
    uint32_t tmem_base;
    int abort_flag;
    TcItem items[kMaxCachedItems];  // item of round r, worked out once at start-up instead of by every role at every item boundary
};
static_assert(sizeof(TcSmem) <= 3072, "the barriers must fit beside seven 32 KB tiles");


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


// kTree:   tree verification (else causal prefill).   kPaged: tree prefix in the paged pool.
// kSplitQ: queries given as fp16 hi + lo arrays (fp32 queries): S = Q_hi K^T + Q_lo K^T; one tile only.
// kTiles:  query tiles per item (1 or 2).
template <bool kTree, bool kPaged, bool kSplitQ, int kTiles>
__global__ void __launch_bounds__(kTcThreads, 1)
fa_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap qlomap,
             const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
             const __grid_constant__ CUtensorMap ktmap, const __grid_constant__ CUtensorMap vtmap, TcParams p) {
    static_assert(!(kSplitQ && kTiles == 2), "split queries take both query slots");
    constexpr int kQSlots = kSplitQ ? 2 : kTiles;
    constexpr int kStages = kQSlots == 1 ? 3 : 2;
    // barriers first, then the 1024-byte aligned tiles (128-byte swizzle atoms)
    extern __shared__ __align__(16) uint8_t smem_raw[];
    TcSmem* sh = reinterpret_cast<TcSmem*>(smem_raw);
    uint8_t* q_smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + sizeof(TcSmem) + 1023) & ~uintptr_t(1023));
    uint8_t* k_smem = q_smem + kQSlots * kTileBytes;
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
    const int N = p.num_nodes;
    const int hd = p.d_chunks * 64;  // head_dim
    // K/V tile layout in shared memory.  Contiguous caches: [chunk][128 rows][64 halfs] (8-row groups 1 KB
    // apart, the second 64 dims 16 KB further).  Paged pool: one TMA box per page lands as
    // [row group][chunk][8 rows][64], so the groups are head_dim * 16 bytes apart and the second 64 dims
    // of a group follow its first after 1 KB; the MMA descriptors take either pitch.
    const uint32_t group_bytes = kPaged ? 1024u * p.d_chunks : 1024u;
    const uint32_t chunk_off = kPaged ? 1024u : (uint32_t)kChunkBytes;

    // ---- work items.  Prefill: ordered heaviest query block first and dealt to the CTAs in a snake
    // (round r left to right when even, right to left when odd), which keeps the summed causal work
    // per CTA within about one K/V step of the mean.  Tree: equal items, same dealing.
    const int n_items = kTree ? p.batch * p.num_kv_heads * p.units_per_kvh
                              : p.n_qblocks * p.batch * p.num_kv_heads * p.units_per_kvh;
    const int n_rounds = (n_items + (int)gridDim.x - 1) / (int)gridDim.x;
    auto derive_item = [&](int r) {
        TcItem it;
        const int pos = r * (int)gridDim.x + ((r & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
        it.valid = pos < n_items;
        int pp = it.valid ? pos : 0;
        const int unit = pp % p.units_per_kvh;
        pp /= p.units_per_kvh;
        it.kvh = pp % p.num_kv_heads;
        pp /= p.num_kv_heads;
        if (kTree) {
            it.b = pp;
            it.head0 = it.kvh * p.group + unit * (kT >> p.slot_shift) * kTiles;  // 128 / slots heads per tile
            int len = p.cache_lens ? p.cache_lens[it.b] : p.cache_len;
            const int cap = kPaged ? p.max_blocks * kPageRows : p.cache_stride;
            if (len < 0 || len > cap) {
                atomicOr(p.status, kStatusBadSeqLen);
                len = 0;
            }
            it.cache_len = len;
            it.n_prefix = (len + kT - 1) / kT;
            it.n_steps = it.n_prefix + 1;  // the last step is the tree tile
            it.q0 = 0;
            it.rows_here = kT;
        } else {
            // pp = qblock_rank * batch + b: the heaviest query blocks of every sequence come first
            it.b = pp % p.batch;
            pp /= p.batch;
            it.head0 = it.kvh * p.group + unit * kTiles;  // one head per tile
            it.q0 = (p.n_qblocks - 1 - pp) * kT;
            it.rows_here = min(kT, p.seq_q - it.q0);
            const int k_end = min(p.seq_kv, p.start_pos + it.q0 + it.rows_here);  // exclusive: last visible key + 1
            it.n_steps = (k_end + kT - 1) / kT;
            it.n_prefix = it.n_steps;
            it.cache_len = p.seq_kv;  // paged K/V: pages past the live length are not looked up
        }
        return it;
    };

    // Warp 0 sets everything up that the loads need - the barriers (lane 0) and the items of the first
    // rounds (one per lane) - and then goes straight on as the producer: it only ARRIVES at the start-up
    // barrier, so the first query and K/V tiles are already in flight while warp 1 allocates tensor memory.
    static_assert(kMaxCachedItems == 32, "one item per lane of warp 0");
    if (warp == 0 && lane < min(n_rounds, kMaxCachedItems)) sh->items[lane] = derive_item(lane);
    auto item_of = [&](int r) { return r < kMaxCachedItems ? sh->items[r] : derive_item(r); };
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
        mbar_init(&sh->o_final[0], 2);
        mbar_init(&sh->o_final[1], 2);
        sh->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        tmem_alloc(&sh->tmem_base, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    if (warp == 0) {
        __syncwarp();
        asm volatile("bar.arrive 1, %0;" ::"r"(kTcThreads) : "memory");
    } else {
        asm volatile("bar.sync 1, %0;" ::"r"(kTcThreads) : "memory");
    }
    tc_fence_after_sync();
    const uint32_t tmem = warp == 0 ? 0u : sh->tmem_base;  // the producer never touches tensor memory

    if (warp < 4) {
        setmaxnreg_dec<56>();  // producer / MMA warpgroup gives registers up
        if (warp == 0) {
            // -------------------------------------------------------------- TMA producer (whole warp)
            if (lane == 0) {
                tma_prefetch_desc(&qmap);
                tma_prefetch_desc(&kmap);
                tma_prefetch_desc(&vmap);
                if (kTree) {
                    tma_prefetch_desc(&ktmap);
                    tma_prefetch_desc(&vtmap);
                }
            }
            int st = 0, items_done = 0;
            uint32_t ph = 1;  // a fresh barrier passes a wait on parity 1
            int alive = 1;
            for (int r = 0; r < n_rounds && alive; r++) {
                const TcItem it = item_of(r);
                if (!it.valid) continue;
                if (lane == 0) {
                    // the query tiles are replaced once the last score MMA of the previous item is done
                    alive = mbar_wait(&sh->q_empty, (items_done & 1) ^ 1, abort_flag);
                    if (alive) {
                        mbar_arrive_expect_tx(&sh->q_full, kQSlots * p.d_chunks * kChunkBytes);
                        for (int c = 0; c < p.d_chunks; c++) {
                            if (kTree) {
                                // Q [batch*Hq, N, 128]: a box is 64 halfs x node slots x heads per tile (16 KB)
                                const int z0 = it.b * p.num_heads + it.head0;
                                for (int t = 0; t < kTiles; t++)
                                    tma_load_3d(q_smem + t * kTileBytes + c * kChunkBytes, &qmap, &sh->q_full, c * 64, 0, z0 + (kT >> p.slot_shift) * t);
                                if (kSplitQ)
                                    tma_load_3d(q_smem + kTileBytes + c * kChunkBytes, &qlomap, &sh->q_full, c * 64, 0, z0);
                            } else {
                                for (int t = 0; t < kTiles; t++)
                                    tma_load_2d(q_smem + t * kTileBytes + c * kChunkBytes, &qmap, &sh->q_full,
                                                (it.head0 + t) * hd + c * 64, it.b * p.seq_q + it.q0);
                                if (kSplitQ)
                                    tma_load_2d(q_smem + kTileBytes + c * kChunkBytes, &qlomap, &sh->q_full,
                                                it.head0 * hd + c * 64, it.b * p.seq_q + it.q0);
                            }
                        }
                    }
                }
                alive = __shfl_sync(0xffffffffu, alive, 0);
                if (!alive) break;
                items_done++;
                // page entries of the next prefix tile are fetched one tile ahead (lanes 0-7, one page each)
                auto load_entry = [&](int j) {
                    int e = 0;
                    if (kPaged && j < it.n_prefix && lane < 8) {
                        const int logical = j * 8 + lane;
                        if (logical * kPageRows < it.cache_len) {
                            e = p.tables[(size_t)it.b * p.max_blocks + logical];
                            if (e < 0 || e >= p.num_blocks) {
                                atomicOr(p.status, kStatusBadTable);
                                e = 0;
                            }
                        }
                    }
                    return e;
                };
                int entry_next = load_entry(0);
                for (int j = 0; j < it.n_steps; j++) {
                    const bool tree_step = kTree && j == it.n_prefix;
                    const int entry = entry_next;
                    entry_next = load_entry(j + 1);
                    const uint32_t bytes = (uint32_t)(p.d_chunks * kChunkBytes) >> (tree_step ? 1 : 0);  // the tree tile has 64 rows
                    uint8_t* kd = k_smem + st * kTileBytes;
                    uint8_t* vd = v_smem + st * kTileBytes;
                    const int c = lane & 1;
                    // K first: its slot is released as soon as the score MMAs that read it are done,
                    // a whole softmax earlier than the V slot, so K runs further ahead
#pragma unroll
                    for (int is_v = 0; is_v < 2; is_v++) {
                        uint64_t* full = is_v ? &sh->v_full[st] : &sh->k_full[st];
                        if (lane == 0) {
                            alive = mbar_wait(is_v ? &sh->v_empty[st] : &sh->k_empty[st], ph, abort_flag);
                            if (alive) mbar_arrive_expect_tx(full, bytes);
                        }
                        alive = __shfl_sync(0xffffffffu, alive, 0);
                        if (!alive) break;
                        uint8_t* dst = is_v ? vd : kd;
                        if (tree_step) {
                            if (kPaged) {
                                // tree K/V [batch*Hkv, N, 128] in the grouped layout: lane = (row group, chunk),
                                // 8-row boxes; rows >= N are zero-filled by TMA
                                const int g = lane >> 1;
                                if (lane < 16 && c < p.d_chunks)
                                    tma_load_3d(dst + g * group_bytes + c * 1024, is_v ? &vtmap : &ktmap, full, c * 64, g * 8,
                                                it.b * p.num_kv_heads + it.kvh);
                            } else if (lane < p.d_chunks) {
                                // tree K/V [batch*Hkv, N, 128]: 64-row boxes; rows >= N are zero-filled by TMA
                                tma_load_3d(dst + c * kChunkBytes, is_v ? &vtmap : &ktmap, full, c * 64, 0,
                                            it.b * p.num_kv_heads + it.kvh);
                            }
                        } else if (kPaged) {
                            // lane = page: one box per 16-row page (both row groups, all chunks of the head)
                            const int e = __shfl_sync(0xffffffffu, entry, lane & 7);
                            if (lane < 8)
                                tma_load_4d(dst + lane * 2 * group_bytes, is_v ? &vmap : &kmap, full, it.kvh * hd, 0, 0, e * 2);
                        } else if (lane < p.d_chunks) {
                            // contiguous cache [.., max rows, 128]: one 128-row box per chunk
                            const int y = kTree ? (it.b * p.num_kv_heads + it.kvh) * p.cache_stride + j * kT
                                                : (it.b * p.num_kv_heads + it.kvh) * p.max_seq + j * kT;
                            tma_load_2d(dst + c * kChunkBytes, is_v ? &vmap : &kmap, full, c * 64, y);
                        }
                    }
                    if (!alive) break;
                    if (++st == kStages) {
                        st = 0;
                        ph ^= 1;
                    }
                }
            }
            if (!alive && lane == 0) atomicOr(p.status, kStatusTimeout);
        } else if (warp == 1) {
            // -------------------------------------------------------------- score MMAs: S_b = Q_t K_j^T
            if (lane == 0) {
                constexpr uint32_t idesc_qk = umma_idesc_f16(kT, kT, false, false);
                constexpr uint32_t idesc_qk_tree = umma_idesc_f16(kT, kNodeSlots, false, false);
                const uint32_t q_lo0 = desc_lo(smem_u32(q_smem), 16);
                const uint32_t k_lo0 = desc_lo(smem_u32(k_smem), 16);
                const uint32_t k_hi = desc_hi_sw128(group_bytes);
                bool ok = true;
                int st = 0, items_done = 0;
                int vs = 0;  // virtual steps issued so far across items: S buffer = vs & 1
                uint32_t ph = 0;
                for (int r = 0; r < n_rounds && ok; r++) {
                    const TcItem it = item_of(r);
                    if (!it.valid) continue;
                    ok = mbar_wait(&sh->q_full, items_done & 1, abort_flag);
                    items_done++;
                    for (int j = 0; j < it.n_steps && ok; j++) {
                        ok = mbar_wait(&sh->k_full[st], ph, abort_flag);
                        const uint32_t idesc = (kTree && j == it.n_prefix) ? idesc_qk_tree : idesc_qk;  // 64 keys in the tree tile
                        const uint32_t k_lo = k_lo0 + st * (kTileBytes >> 4);
#pragma unroll
                        for (int t = 0; t < kTiles; t++, vs++) {
                            const int b = vs & 1;
                            // S_b still holds P of virtual step vs-2 until both output-MMA halves of it are done
                            if (ok && vs >= 2) ok = mbar_wait(&sh->s_free[b], ((vs >> 1) - 1) & 1, abort_flag);
                            if (!ok) break;
                            tc_fence_after_sync();
                            const uint32_t d = tmem + b * kT;
                            const uint32_t q_lo = q_lo0 + t * (kTileBytes >> 4);
                            // K-major operands: 8 steps of 16 along head_dim (32 bytes inside the swizzled
                            // row, the second 64-wide block 16 KB further)
#pragma unroll
                            for (int ks = 0; ks < 8; ks++) {
                                if (ks < 4 * p.d_chunks) {
                                    const uint32_t off = ((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4;
                                    const uint32_t off_k = ((ks >> 2) * chunk_off + (ks & 3) * 32) >> 4;
                                    umma_ss_words2(d, q_lo + off, kDescHiSw128, k_lo + off_k, k_hi, idesc, ks > 0 ? 1u : 0u);
                                }
                            }
                            if (kSplitQ) {
#pragma unroll
                                for (int ks = 0; ks < 8; ks++) {
                                    if (ks < 4 * p.d_chunks) {
                                        const uint32_t off = ((ks >> 2) * kChunkBytes + (ks & 3) * 32) >> 4;
                                        const uint32_t off_k = ((ks >> 2) * chunk_off + (ks & 3) * 32) >> 4;
                                        umma_ss_words2(d, q_lo0 + (kTileBytes >> 4) + off, kDescHiSw128, k_lo + off_k, k_hi, idesc, 1u);
                                    }
                                }
                            }
                            tc_commit(&sh->s_full[b]);
                        }
                        if (!ok) break;
                        tc_commit(&sh->k_empty[st]);
                        if (j + 1 == it.n_steps) tc_commit(&sh->q_empty);  // the query tiles may be replaced
                        if (++st == kStages) {
                            st = 0;
                            ph ^= 1;
                        }
                    }
                }
                if (!ok) atomicOr(p.status, kStatusTimeout);
            }
        } else {
            // -------------------------------------------------------------- output MMAs: O_t += P_b V_j
            // warp 2 multiplies the hi half of P, warp 3 the lo half; O was zeroed by the softmax
            // warps, so every MMA accumulates and the two issuers need no order between them
            if (lane == 0) {
                const uint32_t idesc_pv = umma_idesc_f16(kT, hd, false, true);  // N = head_dim output columns
                const uint32_t part = warp - 2;  // 0: hi, 1: lo
                const uint32_t v_lo0 = desc_lo(smem_u32(v_smem), chunk_off);  // leading offset: the second 64 dims
                const uint32_t v_hi = desc_hi_sw128(group_bytes);
                bool ok = true;
                int st = 0, vs = 0, items_done = 0;
                uint32_t ph = 0;
                for (int r = 0; r < n_rounds && ok; r++) {
                    const TcItem it = item_of(r);
                    if (!it.valid) continue;
                    // one tile per item: O alternates between the two accumulators from item to item,
                    // so the previous item's result can be read out while this one accumulates
                    const uint32_t o_sel = kTiles == 1 ? (items_done & 1) : 0;
                    uint64_t* o_final = &sh->o_final[items_done & 1];
                    items_done++;
                    for (int j = 0; j < it.n_steps && ok; j++) {
                        ok = mbar_wait(&sh->v_full[st], ph, abort_flag);
                        const uint32_t v_lo = v_lo0 + st * (kTileBytes >> 4);
                        const int nks = (kTree && j == it.n_prefix) ? 4 : 8;  // 16 keys per step; the tree tile has 64
#pragma unroll
                        for (int t = 0; t < kTiles; t++, vs++) {
                            const int b = vs & 1;
                            if (ok) ok = mbar_wait(&sh->p_ready[b], (vs >> 1) & 1, abort_flag);
                            if (!ok) break;
                            tc_fence_after_sync();
                            const uint32_t d = tmem + 2 * kT + (t + o_sel) * kT;
                            // P: hi in columns 0-63 of S_b, lo in 64-127, 8 columns per 16 keys;
                            // V MN-major: 16 keys = two row groups further per step, second 64 dims via LBO
#pragma unroll
                            for (int ks = 0; ks < 8; ks++) {
                                if (ks < nks) {
                                    const uint32_t a = tmem + b * kT + part * 64 + ks * 8;
                                    umma_ts_words(d, a, v_lo + ks * (2 * group_bytes >> 4), v_hi, idesc_pv, 1u);
                                }
                            }
                            tc_commit(&sh->s_free[b]);
                        }
                        if (!ok) break;
                        tc_commit(&sh->v_empty[st]);
                        if (j + 1 == it.n_steps) tc_commit(o_final);
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
        // Rows are split, not columns: the two warps that may touch a TMEM lane quarter take 16 of
        // its 32 rows each, and read S in the 16-lane fragment shape, which spreads a row's 128
        // columns over the four threads of a quad.  Row maxima and sums are then two shuffles inside
        // the quad - no shared memory, no barrier between the warps, and every warp overwrites only
        // rows it has itself read.  Each thread works on two rows (g and g + 8 of its 16) x 32 columns.
        const int wg = (warp - 4) >> 2;
        const int quarter = warp & 3;            // TMEM lane quarter this warp may touch
        const int tq = lane & 3;                 // position in the quad: columns 8i + 2 tq + {0, 1}
        const int row_of[2] = {quarter * 32 + wg * 16 + (lane >> 2), quarter * 32 + wg * 16 + (lane >> 2) + 8};
        const uint32_t frag_base = tmem + (static_cast<uint32_t>(quarter * 32 + wg * 16) << 16);
        const int row = quarter * 32 + lane;     // 0..127 over the first warpgroup: work index for clearing a V tail
        bool ok = true;
        int vs = 0, kvs = 0, items_done = 0;     // virtual steps, K/V steps, items handled so far

        // Read-out of a finished item.  With one tile per item it is deferred: the item's O stays in
        // its accumulator while the next item starts in the other one, and one 64-column half is
        // written after each of the next item's first softmax steps, behind the MMAs of those steps.
        constexpr bool kDefer = kTiles == 1;
        struct Readout {
            int halves_left;     // 0: nothing pending
            uint64_t* o_final;   // the item's "output MMAs done" barrier ...
            uint32_t phase;      // ... and its parity for this item
            uint32_t o_frag;     // the item's O accumulator, this warp's 16 lanes
            float inv[2];        // 1 / row sum of the thread's two rows
            bool store[2];       // the row is a live output row
            size_t base[2];      // element offset of the row's first output value
        } pend;
        pend.halves_left = 0;
        auto readout_half = [&](Readout& e) {
            const int h = p.d_chunks - e.halves_left;
            ok = __all_sync(0xffffffffu, ok);  // warp-uniform before anything that the whole warp must execute together
            if (h == 0) {
                if (ok) ok = mbar_wait(e.o_final, e.phase, abort_flag);
                ok = __all_sync(0xffffffffu, ok);  // warp-uniform: the tcgen05.ld below needs the whole warp
                tc_fence_after_sync();
            }
            e.halves_left--;
            if (!ok) return;
            uint32_t rr[32];
            __syncwarp();
            tmem_ld_16x256b_x8(e.o_frag + h * 64, rr);
            tmem_wait_ld();
            if (!kTree && p.out_fp16) {
                // a thread holds pairs of columns; a 4 x 4 exchange inside the quad turns four pairs of
                // one 8-column group into one 16-byte piece per lane: the quad then writes 64
                // contiguous bytes of a row per store instruction
#pragma unroll
                for (int r = 0; r < 2; r++) {
#pragma unroll
                    for (int blk = 0; blk < 2; blk++) {
                        uint32_t v[4];
#pragma unroll
                        for (int i = 0; i < 4; i++)
                            v[i] = pack_half2(__uint_as_float(rr[4 * (4 * blk + i) + 2 * r]) * e.inv[r],
                                              __uint_as_float(rr[4 * (4 * blk + i) + 2 * r + 1]) * e.inv[r]);
                        quad_transpose(v, lane);  // now: columns 8 (4 blk + tq) .. + 7 of the row
                        if (e.store[r])
                            *reinterpret_cast<uint4*>(static_cast<__half*>(p.out) + e.base[r] + h * 64 + 8 * (4 * blk + tq)) =
                                make_uint4(v[0], v[1], v[2], v[3]);
                    }
                }
            } else {
                float* outp = kTree ? p.tree_out : static_cast<float*>(p.out);
#pragma unroll
                for (int r = 0; r < 2; r++)
                    if (e.store[r]) {
#pragma unroll
                        for (int i = 0; i < 8; i++)  // a quad writes 32 contiguous bytes of the row
                            *reinterpret_cast<float2*>(outp + e.base[r] + h * 64 + 8 * i + 2 * tq) =
                                make_float2(__uint_as_float(rr[4 * i + 2 * r]) * e.inv[r], __uint_as_float(rr[4 * i + 2 * r + 1]) * e.inv[r]);
                    }
            }
        };

        for (int r = 0; r < n_rounds; r++) {
            const TcItem it = item_of(r);
            if (!it.valid) continue;
            // prefill: the last key a row may see; tree: the row's ancestor word, pre-shifted to this
            // thread's first column
            int last_visible[2];
            unsigned long long anc[2] = {1ull >> (2 * tq), 1ull >> (2 * tq)};  // rows past the last node see column 0 only
#pragma unroll
            for (int q = 0; q < 2; q++) {
                last_visible[q] = kTree ? it.cache_len - 1 : min(p.start_pos + it.q0 + row_of[q], p.seq_kv - 1);
                const int node = row_of[q] & ((1 << p.slot_shift) - 1);
                if (kTree && node < N) {
                    const int32_t* par = p.parents + (size_t)it.b * N;
                    if (par[node] < -1 || par[node] >= N) atomicOr(p.status, kStatusBadParent);
                    anc[q] = ancestor_word(par, node, N) >> (2 * tq);
                }
            }
            float m_used_t[kTiles][2], l_run_t[kTiles][2];  // running maximum and (per-thread part of the) sum, per tile and row
            const int o_sel = kDefer ? (items_done & 1) : 0;  // accumulator of this item (see the output MMAs)
            {
                // O starts at zero so that every output MMA can accumulate
                uint32_t z[32];
#pragma unroll
                for (int c = 0; c < 32; c++) z[c] = 0u;
#pragma unroll
                for (int t = 0; t < kTiles; t++) {
#pragma unroll
                    for (int q = 0; q < 2; q++) {
                        m_used_t[t][q] = -INFINITY;
                        l_run_t[t][q] = 0.f;
                    }
#pragma unroll
                    for (int h = 0; h < 2; h++)
                        if (h < p.d_chunks) tmem_st_16x256b_x8(frag_base + 2 * kT + (t + o_sel) * kT + h * 64, z);  // own rows only
                }
                tmem_wait_st();
            }
            for (int j = 0; j < it.n_steps; j++, kvs++) {
                const bool tree_step = kTree && j == it.n_prefix;
                const int k0 = j * kT;
                // prefill: the diagonal tile and a ragged last tile; tree prefix: a ragged last tile
                const bool need_mask = kTree ? (!tree_step && k0 + kT > it.cache_len)
                                             : ((k0 + kT - 1 > p.start_pos + it.q0) || (k0 + kT > p.seq_kv));
                // not unrolled: the two tiles of an item share one copy of the softmax code
#pragma unroll 1
                for (int t = 0; t < kTiles; t++, vs++) {
                    const int ti = (kTiles == 2 && t) ? kTiles - 1 : 0;
                    float m_used[2] = {m_used_t[ti][0], m_used_t[ti][1]};
                    float l_run[2] = {l_run_t[ti][0], l_run_t[ti][1]};
                    const int b = vs & 1;
                    const uint32_t s_frag = frag_base + b * kT;
                    const uint32_t o_frag = frag_base + 2 * kT + (t + o_sel) * kT;
                    // No vote and no early exit in the pace-setting loop (they cost 1-3 % of a launch): a wait that gives
                    // up only clears the flag.  Every later wait then returns at once through the abort flag, the steps
                    // that are left run on stale scores, and nothing of the item is stored (the read-out checks the flag).
                    ok &= mbar_wait(&sh->s_full[b], (vs >> 1) & 1, abort_flag);
                    tc_fence_after_sync();
                    // the two rows' scores: x[h][4i + 2q + e] = row q, column 64 h + 8 i + 2 tq + e
                    uint32_t x[2][32];
                    tmem_ld_16x256b_x8(s_frag, x[0]);
                    if (!tree_step) tmem_ld_16x256b_x8(s_frag + 64, x[1]);  // the tree tile has 64 key columns only
                    tmem_wait_ld();
                    if (tree_step) {
#pragma unroll
                        for (int i = 0; i < 8; i++)
#pragma unroll
                            for (int q = 0; q < 2; q++)
#pragma unroll
                                for (int e = 0; e < 2; e++) {
                                    if (!((anc[q] >> (8 * i + e)) & 1ull)) x[0][4 * i + 2 * q + e] = kNegInf;
                                    x[1][4 * i + 2 * q + e] = kNegInf;
                                }
                    } else if (need_mask) {
#pragma unroll
                        for (int q = 0; q < 2; q++) {
                            const int limit = last_visible[q] - k0 - 2 * tq;  // own column 64 h + 8 i + e is visible iff <= limit
#pragma unroll
                            for (int h = 0; h < 2; h++)
#pragma unroll
                                for (int i = 0; i < 8; i++)
#pragma unroll
                                    for (int e = 0; e < 2; e++)
                                        if (64 * h + 8 * i + e > limit) x[h][4 * i + 2 * q + e] = kNegInf;
                        }
                    }
                    float mx[2];
#pragma unroll
                    for (int q = 0; q < 2; q++) {
                        float mm[2] = {-INFINITY, -INFINITY};  // independent chains
#pragma unroll
                        for (int h = 0; h < 2; h++)
#pragma unroll
                            for (int i = 0; i < 8; i++)
                                mm[h] = max3(mm[h], __uint_as_float(x[h][4 * i + 2 * q]), __uint_as_float(x[h][4 * i + 2 * q + 1]));
                        float m = fmaxf(mm[0], mm[1]);
                        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                        mx[q] = m * p.scale_log2;
                    }
                    if (j == 0) {
                        m_used[0] = mx[0];
                        m_used[1] = mx[1];
                    } else {
                        const bool grow0 = mx[0] > m_used[0] + kLazyLog2, grow1 = mx[1] > m_used[1] + kLazyLog2;
                        if (__any_sync(0xffffffffu, grow0 || grow1)) {
                            // O_t must be quiescent: wait until both halves of its previous output MMA are done
                            ok = __all_sync(0xffffffffu, ok && mbar_wait(&sh->s_free[(vs - kTiles) & 1], ((vs - kTiles) >> 1) & 1, abort_flag));
                            tc_fence_after_sync();
                            const float alpha0 = grow0 ? fast_exp2(m_used[0] - mx[0]) : 1.0f;
                            const float alpha1 = grow1 ? fast_exp2(m_used[1] - mx[1]) : 1.0f;
                            if (grow0) m_used[0] = mx[0];
                            if (grow1) m_used[1] = mx[1];
                            l_run[0] *= alpha0;
                            l_run[1] *= alpha1;
                            uint32_t rr[32];
#pragma unroll 1
                            for (int h = 0; h < p.d_chunks; h++) {
                                tmem_ld_16x256b_x8(o_frag + h * 64, rr);
                                tmem_wait_ld();
#pragma unroll
                                for (int i = 0; i < 8; i++) {
                                    rr[4 * i + 0] = __float_as_uint(__uint_as_float(rr[4 * i + 0]) * alpha0);
                                    rr[4 * i + 1] = __float_as_uint(__uint_as_float(rr[4 * i + 1]) * alpha0);
                                    rr[4 * i + 2] = __float_as_uint(__uint_as_float(rr[4 * i + 2]) * alpha1);
                                    rr[4 * i + 3] = __float_as_uint(__uint_as_float(rr[4 * i + 3]) * alpha1);
                                }
                                tmem_st_16x256b_x8(o_frag + h * 64, rr);
                            }
                        }
                    }
                    {
                        // P = 2^(s*scale - m) as fp16 hi + lo: a pair of neighbouring keys is one 32-bit
                        // column, hi in columns 0-63 of the S buffer, lo in 64-127.  Every warp has read
                        // all of its rows' scores before it overwrites them.
                        const uint64_t scale2 = f32x2(p.scale_log2, p.scale_log2);
                        const uint64_t neg_m2[2] = {f32x2(-m_used[0], -m_used[0]), f32x2(-m_used[1], -m_used[1])};
                        uint64_t ls[2][2] = {{0ull, 0ull}, {0ull, 0ull}};  // [row][chain] partial sums, packed pairs
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            if (tree_step && h == 1) continue;
                            uint32_t hi[16], lo[16];
#pragma unroll
                            for (int i = 0; i < 8; i++)
#pragma unroll
                                for (int q = 0; q < 2; q++) {
                                    // masked scores are -inf: exp2 gives exactly 0
                                    float t0, t1;
                                    f32x2_get(fma_f32x2(f32x2(__uint_as_float(x[h][4 * i + 2 * q]), __uint_as_float(x[h][4 * i + 2 * q + 1])),
                                                        scale2, neg_m2[q]), t0, t1);
                                    const uint64_t pp = f32x2(fast_exp2(t0), fast_exp2(t1));
                                    ls[q][i & 1] = add_f32x2(ls[q][i & 1], pp);
                                    split_hi_lo_x2(pp, hi[2 * i + q], lo[2 * i + q]);
                                }
                            tmem_st_16x128b_x8(s_frag + 32 * h, hi);
                            tmem_st_16x128b_x8(s_frag + 64 + 32 * h, lo);
                        }
#pragma unroll
                        for (int q = 0; q < 2; q++) {
                            float la, lb;
                            f32x2_get(add_f32x2(ls[q][0], ls[q][1]), la, lb);
                            l_run[q] += la + lb;
                        }
                    }
                    if (t == 0 && wg == 0 && need_mask && k0 + kT > (kTree ? it.cache_len : p.seq_kv)) {
                        // keys past the live length carry P = 0, but their V rows may hold anything (even
                        // NaN): zero them in shared memory before the MMAs read the tile
                        const int st = kvs % kStages;
                        ok = __all_sync(0xffffffffu, ok && mbar_wait(&sh->v_full[st], (kvs / kStages) & 1, abort_flag));
                        const int first_bad = (kTree ? it.cache_len : p.seq_kv) - k0;
                        uint8_t* vt = v_smem + st * kTileBytes;
                        const int row_units = 8 * p.d_chunks;  // 16-byte units per V row
                        for (int i = row; i < (kT - first_bad) * row_units; i += 128) {
                            const int vr = first_bad + i / row_units, u = i % row_units;
                            *reinterpret_cast<uint4*>(vt + (vr >> 3) * group_bytes + (u >> 3) * chunk_off + (vr & 7) * 128 +
                                                      (((u & 7) ^ (vr & 7)) << 4)) = make_uint4(0, 0, 0, 0);
                        }
                        fence_proxy_async_smem();
                    }
                    __syncwarp();
                    tmem_wait_st();
                    tc_fence_before_sync();
                    mbar_arrive(&sh->p_ready[b]);
#pragma unroll
                    for (int q = 0; q < 2; q++) {
                        m_used_t[ti][q] = m_used[q];
                        l_run_t[ti][q] = l_run[q];
                    }
                    if (kDefer && pend.halves_left > 0) readout_half(pend);  // behind the MMAs of this step
                }
            }
            while (kDefer && pend.halves_left > 0) readout_half(pend);  // an item shorter than the read-out
#pragma unroll
            for (int t = 0; t < kTiles; t++) {
                Readout e;
                e.halves_left = p.d_chunks;
                e.o_final = &sh->o_final[items_done & 1];
                e.phase = (items_done >> 1) & 1;
                e.o_frag = frag_base + 2 * kT + (t + o_sel) * kT;
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    // the row's sum: the quad's four partial sums
                    float l = l_run_t[t][q];
                    l += __shfl_xor_sync(0xffffffffu, l, 1);
                    l += __shfl_xor_sync(0xffffffffu, l, 2);
                    e.inv[q] = __frcp_rn(l);
                    if (kTree) {
                        const int node = row_of[q] & ((1 << p.slot_shift) - 1);
                        const int head = it.head0 + (kT >> p.slot_shift) * t + (row_of[q] >> p.slot_shift);
                        e.store[q] = node < N && head < (it.kvh + 1) * p.group;
                        e.base[q] = (((size_t)it.b * p.num_heads + head) * N + node) * hd;
                    } else {
                        e.store[q] = row_of[q] < it.rows_here;
                        e.base[q] = (((size_t)it.b * p.seq_q + it.q0 + row_of[q]) * p.num_heads + it.head0 + t) * hd;
                    }
                }
                if (kDefer) {
                    pend = e;
                } else {
                    while (e.halves_left > 0) readout_half(e);
                }
            }
            items_done++;
        }  // items
        while (kDefer && pend.halves_left > 0) readout_half(pend);
        if (!ok && lane == 0) atomicOr(p.status, kStatusTimeout);
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
typedef void (*TcKernel)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, TcParams);

static int launch_tc(granite_cuda_compute* c, TcKernel kern, const char* name, int n_items, int q_slots,
                     const CUtensorMap* qmap, const CUtensorMap* qlomap, const CUtensorMap* kmap,
                     const CUtensorMap* vmap, const CUtensorMap* ktmap, const CUtensorMap* vtmap, const TcParams& p) {
    // Q slots + K and V rings: 3 stages fit beside one query slot, 2 beside two
    const int stages = q_slots == 1 ? 3 : 2;
    size_t smem_bytes = (sizeof(TcSmem) + 1023) / 1024 * 1024 + 1024 + (size_t)(q_slots + 2 * stages) * kTileBytes;
    if (smem_bytes > (size_t)c->smem_optin) smem_bytes = (size_t)c->smem_optin;  // the window is 1 KB aligned in practice
    GB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    const int grid = n_items < c->sm_count ? n_items : c->sm_count;  // persistent CTAs, one per SM
    {
        LaunchScope t(c, name);
        kern<<<grid, kTcThreads, smem_bytes, c->stream>>>(*qmap, *qlomap, *kmap, *vmap, *ktmap, *vtmap, p);
    }
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

// fp32 queries -> hi / lo fp16 arrays in the scratch arena
static int split_queries(granite_cuda_compute* c, const void* q, size_t n, const void** hi_out, const void** lo_out) {
    const size_t half_bytes = (n * 2 + 255) / 256 * 256;
    int rc = c->ensure_scratch(2 * half_bytes);
    if (rc) return rc;
    LaunchScope t(c, "split_q_f16");
    __half* hi = static_cast<__half*>(c->scratch);
    __half* lo = reinterpret_cast<__half*>(static_cast<uint8_t*>(c->scratch) + half_bytes);
    split_f32_to_f16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(static_cast<const float*>(q), hi, lo, n);
    *hi_out = hi;
    *lo_out = lo;
    return GRANITE_CUDA_SUCCESS;
}

int launch_prefill(granite_cuda_compute* c, const GraniteCudaAttentionArgs& a) {
    if (!a.q || !a.k || !a.v || !a.output) return fail(GRANITE_CUDA_NULL_POINTER, "prefill: null buffer");
    if (a.head_dim != 128 && a.head_dim != 64) return launch_generic_prefill(c, a);  // the plain kernel takes the other head dims
    const uint32_t D = a.head_dim;
    if (a.num_kv_heads == 0 || a.num_heads % a.num_kv_heads != 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "prefill: num_heads must be a multiple of num_kv_heads");
    if (a.q_dtype > 1 || a.out_dtype > 1) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "prefill: dtype must be 0 (fp32) or 1 (fp16)");
    const uint32_t max_seq = a.max_seq ? a.max_seq : a.seq_kv;
    if (a.seq_kv == 0 || a.seq_kv > max_seq) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "prefill: seq_kv must be in [1, max_seq]");

    const uint32_t batch = a.batch_size ? a.batch_size : 1;
    if ((uint64_t)batch * a.seq_q >= (1ull << 31) || (uint64_t)batch * a.num_kv_heads * max_seq >= (1ull << 31))
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "prefill: batch * rows exceeds the tensor-map coordinate range");

    const bool split_q = a.q_dtype == 0;
    const void *q16 = a.q, *q16_lo = a.q;
    if (split_q) {
        int rc = split_queries(c, a.q, (size_t)batch * a.seq_q * a.num_heads * D, &q16, &q16_lo);
        if (rc) return rc;
    }
    TcParams p{};
    p.d_chunks = (int)D / 64;
    p.batch = (int)batch;
    p.num_heads = (int)a.num_heads;
    p.num_kv_heads = (int)a.num_kv_heads;
    p.group = (int)(a.num_heads / a.num_kv_heads);
    const int tiles = 1;  // one query head per item: measured faster than a GQA pair sharing K/V tiles
    p.units_per_kvh = p.group / tiles;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.status = c->d_status;
    p.out = a.output;
    p.out_fp16 = a.out_dtype == 1;
    p.seq_q = (int)a.seq_q;
    p.seq_kv = (int)a.seq_kv;
    p.max_seq = (int)max_seq;
    p.n_qblocks = (p.seq_q + kT - 1) / kT;
    p.start_pos = (int)a.start_pos;

    const uint64_t q_rows = (uint64_t)batch * a.seq_q;
    const CUtensorMap* qmap = c->tensor_map_2d(q16, (uint64_t)a.num_heads * D, q_rows, (uint64_t)a.num_heads * D * 2, 64, kT, 128);
    const CUtensorMap* qlomap = c->tensor_map_2d(q16_lo, (uint64_t)a.num_heads * D, q_rows, (uint64_t)a.num_heads * D * 2, 64, kT, 128);
    const uint64_t kv_rows = (uint64_t)batch * a.num_kv_heads * max_seq;
    const CUtensorMap* kmap = c->tensor_map_2d(a.k, D, kv_rows, D * 2, 64, kT, 128);
    const CUtensorMap* vmap = c->tensor_map_2d(a.v, D, kv_rows, D * 2, 64, kT, 128);
    if (!qmap || !qlomap || !kmap || !vmap) return GRANITE_CUDA_EXECUTION_FAILED;

    TcKernel kern = split_q ? fa_tc_kernel<false, false, true, 1> : fa_tc_kernel<false, false, false, 1>;
    const int n_items = p.n_qblocks * p.batch * p.num_kv_heads * p.units_per_kvh;
    return launch_tc(c, kern, "prefill_causal_fa", n_items, split_q ? 2 : tiles, qmap, qlomap, kmap, vmap, kmap, vmap, p);
}

// Causal attention of a chunk of new tokens against the sequence's paged cache: the prefill
// kernel with its K/V tiles gathered page by page through the block table.
int launch_paged_prefill(granite_cuda_compute* c, const GraniteCudaPagedPrefillArgs& a) {
    if (!a.q || !a.k_cache || !a.v_cache || !a.block_table || !a.output)
        return fail(GRANITE_CUDA_NULL_POINTER, "paged_prefill_attention: null buffer");
    if ((a.head_dim != 128 && a.head_dim != 64) || a.block_size != (uint32_t)kPageRows) return launch_generic_paged_prefill(c, a);
    const uint32_t D = a.head_dim;
    if (a.num_blocks == 0 || a.max_blocks_per_seq == 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "paged_prefill_attention: empty pool or table");
    if (a.num_kv_heads == 0 || a.num_heads % a.num_kv_heads != 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "paged_prefill_attention: num_heads must be a multiple of num_kv_heads");
    if (a.q_dtype > 1 || a.out_dtype > 1)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "paged_prefill_attention: dtype must be 0 (fp32) or 1 (fp16)");
    if (a.seq_q == 0) return GRANITE_CUDA_SUCCESS;
    const uint64_t seq_kv = (uint64_t)a.start_pos + a.seq_q;
    if (seq_kv > (uint64_t)a.max_blocks_per_seq * kPageRows)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "paged_prefill_attention: the chunk ends beyond the block table");

    const bool split_q = a.q_dtype == 0;
    const void *q16 = a.q, *q16_lo = a.q;
    if (split_q) {
        int rc = split_queries(c, a.q, (size_t)a.seq_q * a.num_heads * D, &q16, &q16_lo);
        if (rc) return rc;
    }
    TcParams p{};
    p.d_chunks = (int)D / 64;
    p.num_heads = (int)a.num_heads;
    p.num_kv_heads = (int)a.num_kv_heads;
    p.group = (int)(a.num_heads / a.num_kv_heads);
    p.units_per_kvh = p.group;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.status = c->d_status;
    p.out = a.output;
    p.out_fp16 = a.out_dtype == 1;
    p.seq_q = (int)a.seq_q;
    p.seq_kv = (int)seq_kv;
    p.max_seq = (int)seq_kv;
    p.n_qblocks = (p.seq_q + kT - 1) / kT;
    p.start_pos = (int)a.start_pos;
    p.tables = a.block_table;
    p.batch = 1;
    p.max_blocks = (int)a.max_blocks_per_seq;
    p.num_blocks = (int)a.num_blocks;

    const CUtensorMap* qmap = c->tensor_map_2d(q16, (uint64_t)a.num_heads * D, a.seq_q, (uint64_t)a.num_heads * D * 2, 64, kT, 128);
    const CUtensorMap* qlomap = c->tensor_map_2d(q16_lo, (uint64_t)a.num_heads * D, a.seq_q, (uint64_t)a.num_heads * D * 2, 64, kT, 128);
    const uint64_t rows = (uint64_t)a.num_blocks * kPageRows, width = (uint64_t)a.num_kv_heads * D;
    const CUtensorMap* kmap = c->tensor_map_page_groups(a.k_cache, width, rows, D);
    const CUtensorMap* vmap = c->tensor_map_page_groups(a.v_cache, width, rows, D);
    if (!qmap || !qlomap || !kmap || !vmap) return GRANITE_CUDA_EXECUTION_FAILED;

    TcKernel kern = split_q ? fa_tc_kernel<false, true, true, 1> : fa_tc_kernel<false, true, false, 1>;
    const int n_items = p.n_qblocks * p.num_kv_heads * p.units_per_kvh;
    return launch_tc(c, kern, "paged_prefill_fa", n_items, split_q ? 2 : 1, qmap, qlomap, kmap, vmap, kmap, vmap, p);
}

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
    if ((a.head_dim != 128 && a.head_dim != 64) || (a.block_tables != nullptr && a.block_size != (uint32_t)kPageRows))
        return launch_generic_tree(c, a);  // the plain kernel takes the other head dims and page sizes
    const uint32_t D = a.head_dim;
    if (a.num_nodes == 0 || a.num_nodes > (uint32_t)kNodeSlots)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: num_nodes must be in [1, 64]");
    if (a.num_kv_heads == 0 || a.num_heads % a.num_kv_heads != 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: num_heads must be a multiple of num_kv_heads");
    if (a.q_dtype > 1) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: q_dtype must be 0 (fp32) or 1 (fp16)");
    if (a.batch_size == 0) return GRANITE_CUDA_SUCCESS;
    const bool paged = a.block_tables != nullptr;
    const bool has_cache = a.cache_lens != nullptr || a.cache_len > 0;
    if (has_cache && (!a.k_cache || !a.v_cache)) return fail(GRANITE_CUDA_NULL_POINTER, "attention_tree: null cache");
    if (paged && (a.block_size != (uint32_t)kPageRows || a.num_blocks == 0 || a.max_blocks_per_seq == 0))
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: paged prefix needs block_size 16 and a non-empty pool");
    const uint32_t cache_stride = a.cache_stride ? a.cache_stride : a.cache_len;
    if (!paged && has_cache && a.cache_len > cache_stride)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "attention_tree: cache_len exceeds cache_stride");

    const bool split_q = a.q_dtype == 0;
    const void *q16 = a.q, *q16_lo = a.q;
    if (split_q) {
        int rc = split_queries(c, a.q, (size_t)a.batch_size * a.num_heads * a.num_nodes * D, &q16, &q16_lo);
        if (rc) return rc;
    }
    TcParams p{};
    p.d_chunks = (int)D / 64;
    p.num_heads = (int)a.num_heads;
    p.num_kv_heads = (int)a.num_kv_heads;
    p.group = (int)(a.num_heads / a.num_kv_heads);
    // A 128-row tile holds heads x node slots.  Small trees leave room for more heads per tile: as many
    // as the node count allows (16, 32 or 64 slots), but no more than the GQA group has.
    int slot_shift = a.num_nodes <= 16 ? 4 : a.num_nodes <= 32 ? 5 : 6;
    while (slot_shift < 6 && (kT >> slot_shift) >= 2 * p.group) slot_shift++;
    const int heads_per_tile = kT >> slot_shift, slots = 1 << slot_shift;
    p.slot_shift = slot_shift;
    const int tiles = (!split_q && p.group % (2 * heads_per_tile) == 0) ? 2 : 1;  // two tiles share the K/V tiles
    p.units_per_kvh = (p.group + heads_per_tile * tiles - 1) / (heads_per_tile * tiles);
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.status = c->d_status;
    p.tree_out = a.output;
    p.parents = a.parent_indices;
    p.tables = a.block_tables;
    p.cache_lens = a.cache_lens;
    p.batch = (int)a.batch_size;
    p.num_nodes = (int)a.num_nodes;
    p.cache_len = (int)a.cache_len;
    p.cache_stride = (int)cache_stride;
    p.max_blocks = (int)a.max_blocks_per_seq;
    p.num_blocks = (int)a.num_blocks;

    // Q / tree K / tree V as [heads, nodes, 128]: box = 64 halfs x node slots x heads per tile (Q), 64 nodes x 1 head (K/V)
    const uint64_t qz = (uint64_t)a.batch_size * a.num_heads;
    const uint64_t node_pitch = (uint64_t)a.num_nodes * D * 2;
    const CUtensorMap* qmap = c->tensor_map_3d(q16, D, a.num_nodes, qz, D * 2, node_pitch, 64, slots, heads_per_tile, 128);
    const CUtensorMap* qlomap = c->tensor_map_3d(q16_lo, D, a.num_nodes, qz, D * 2, node_pitch, 64, slots, heads_per_tile, 128);
    const uint64_t tz = (uint64_t)a.batch_size * a.num_kv_heads;
    // with a paged prefix the tiles are laid out in 8-row groups (see the kernel), so the tree tile comes in 8-row boxes
    const uint32_t tree_box_rows = paged ? 8 : kNodeSlots;
    const CUtensorMap* ktmap = c->tensor_map_3d(a.k_tree, D, a.num_nodes, tz, D * 2, node_pitch, 64, tree_box_rows, 1, 128);
    const CUtensorMap* vtmap = c->tensor_map_3d(a.v_tree, D, a.num_nodes, tz, D * 2, node_pitch, 64, tree_box_rows, 1, 128);
    const CUtensorMap *kmap = ktmap, *vmap = vtmap;  // placeholders when there is no prefix
    if (has_cache) {
        if (paged) {
            const uint64_t rows = (uint64_t)a.num_blocks * kPageRows, width = (uint64_t)a.num_kv_heads * D;
            kmap = c->tensor_map_page_groups(a.k_cache, width, rows, D);
            vmap = c->tensor_map_page_groups(a.v_cache, width, rows, D);
        } else {
            const uint64_t rows = (uint64_t)a.batch_size * a.num_kv_heads * cache_stride;
            kmap = c->tensor_map_2d(a.k_cache, D, rows, D * 2, 64, kT, 128);
            vmap = c->tensor_map_2d(a.v_cache, D, rows, D * 2, 64, kT, 128);
        }
    }
    if (!qmap || !qlomap || !ktmap || !vtmap || !kmap || !vmap) return GRANITE_CUDA_EXECUTION_FAILED;

    TcKernel kern;
    if (split_q) kern = paged ? fa_tc_kernel<true, true, true, 1> : fa_tc_kernel<true, false, true, 1>;
    else if (tiles == 2) kern = paged ? fa_tc_kernel<true, true, false, 2> : fa_tc_kernel<true, false, false, 2>;
    else kern = paged ? fa_tc_kernel<true, true, false, 1> : fa_tc_kernel<true, false, false, 1>;
    const int n_items = p.batch * p.num_kv_heads * p.units_per_kvh;
    return launch_tc(c, kern, "tree_verify", n_items, split_q ? 2 : tiles, qmap, qlomap, kmap, vmap, ktmap, vtmap, p);
}

}  // namespace gb200
