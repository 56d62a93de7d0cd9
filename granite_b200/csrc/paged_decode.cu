// Split-KV flash-decode over the block-table KV cache (and, with an identity table, over the
// contiguous cache).  HBM-bound: every K/V byte of a sequence is read exactly once for all the
// query heads that share it.
//
// Replaces paged_flash_attention_decode_d128 / batched_paged_attention_decode
// (src/backend/metal/kernels/metal_shaders_attention.h:3660, :2186) and
// flash_attention_decode_d128 (:2982); the arithmetic it must match is the CPU loop
// src/llm/transformer.mm:1779-1840 applied to rows fetched by the paged addressing rule
// (include/granite/metal_compute.h:853-861).
//
// Shape of the work.  All pages of all sequences form one linear list (head-tile major, then
// sequence, then page).  The list is cut into one equal contiguous range per CTA (one CTA per
// SM), so the load is balanced to a page whatever the length distribution.  A range that holds
// a whole sequence writes its output directly; a sequence cut by a range boundary leaves
// un-normalised partials (m, l, o); the warp that finishes the sequence's last pages combines them.
//
// Small batches of short sequences (single-user decoding) skip the page list: a few CTAs per (sequence, KV head)
// share the sequence's pages and the last of them to finish combines their partials - one launch, no plan
// kernel, no merge pass ("direct" below).
//
// Inside a CTA: one producer warp walks the block table and has TMA copy each page - 16 rows of
// up to 8 KV heads, one contiguous 32 KB piece of the pool - into a ring of shared-memory slots
// (128-byte swizzle, mbarrier full/empty pairs).  Eight consumer warps each own one KV head of
// the tile: S^T = K * Q^T and O^T += V^T * P^T on mma.sync m16n8k16 with the group's query heads
// as the 8-wide N dimension, online softmax across the warp by shuffles, fp32 state.  Q and P
// are split into fp16 hi + lo parts so the fp32 inputs of the reference are not rounded.
#include <mutex>

#include "compute_internal.h"
#include "ptx.cuh"

namespace gb200 {

constexpr int kHeadDim = 128;  // the benchmarked head size; the decode kernel is also built for 64
constexpr int kPageTokens = 16;
constexpr int kConsumerWarps = 8;
constexpr int kDecodeThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxSlots = 64;
constexpr int kMaxGatherDst = 16;
constexpr int kSelfPlanMaxBatch = 192;  // sequences a CTA plans for itself (one per thread, prefix array in shared memory)
constexpr int kDirectMinPages = 4;  // direct mode: pages a CTA should at least have before a sequence is shared out further

struct DecodeParams {
    const float* q;
    const int32_t* tables;
    const int32_t* seq_lens;
    float* out;
    int batch, num_heads, num_kv_heads, group;
    int max_blocks, num_blocks;
    int uniform_len;      // used when seq_lens == nullptr
    int tile_heads;       // KV heads per CTA tile: 8, 4, 2 or 1
    int tile_shift;       // log2(tile_heads)
    int n_head_tiles;     // num_kv_heads / tile_heads
    int heads_per_warp;   // query heads of the group owned by one consumer warp
    int active_warps;     // consumer warps that own at least one query head
    // Fewer than eight KV heads in the tile (1, 2 or 4): the warps of a head do not split its query heads -
    // all of them would then read every page - but its PAGES: warp `sub` of a head takes every page_split-th page
    // for all query heads of the group, and the warps' partial results are combined through shared memory at
    // the end of each segment.  1: off (every warp walks every page).
    int page_split;
    int slot_arrivals;    // warps that release a page slot (active_warps, or tile_heads when pages are split)
    int dump_offset;      // byte offset of the warps' exchange area behind the barriers
    int dump_bytes;       // bytes of one warp's dump
    int per_round;        // pages the producer issues per round (two slots each)
    // >= 1: small batches of short sequences - `direct` CTAs per (sequence, KV head), each with an equal share of
    // the sequence's pages, its eight warps sharing those; no plan kernel and no merge pass: one launch.  With more
    // than one CTA per pair each leaves a partial, and the one that arrives last at the pair's counter combines
    // them.  The grid is (direct, num_kv_heads, batch) CTAs - three-dimensional so that no role divides to find its
    // place.  0: the range walk over all pages (one-dimensional grid).
    int direct;
    unsigned* direct_done;  // [batch * num_kv_heads] arrival counters, zero between launches (the last arrival wraps them)
    int slots;            // ring depth
    int n_ctas;
    int contiguous;       // 1: k/v are [batch, Hkv, max_seq, D], table is the identity
    int max_seq;
    float scale_log2;     // scale * log2(e)
    int* status;
    int* page_prefix;     // [batch + 1]
    // 1: no plan kernel ran - every CTA builds the page prefix sums of the (small) batch in its own shared memory,
    // finds the first sequence of its range there, and the page counters reset themselves
    int self_plan;
    int plan_offset;      // byte offset of that prefix array behind the barriers
    int* cta_first_seq;   // [n_ctas]
    int d;                // head_dim: 128 or 64
    float* part_o;        // [2 * n_ctas][num_heads][d]
    float2* part_ml;      // [2 * n_ctas][num_heads]
    int* pages_done;      // [batch][n_head_tiles][consumer warps]: pages of cut sequences finished so far
    int fused_merge;      // 1: the warp that finishes a cut sequence merges it; 0: decode_merge_kernel follows
    // optional gather: every final output row is also stored into these buffers (other GPUs' peer-mapped
    // memory or this GPU's own), at row gather_row0 + sequence.  A destination row holds gather_heads
    // query heads (num_heads, or more when the heads are sharded across GPUs) and this call's heads
    // start at gather_head0 of it.
    float* gather[kMaxGatherDst];
    int n_gather;
    long long gather_row0;
    int gather_heads, gather_head0;
};

// Element offset of (sequence b, local query head hq) in a gather destination.
__device__ __forceinline__ size_t gather_offset(const DecodeParams& p, int b, int hq) {
    return ((size_t)(p.gather_row0 + b) * p.gather_heads + p.gather_head0 + hq) * p.d;
}

// Final output element(s) of (sequence b, query head hq): the local row and every gather destination.
// Plain stores: nothing waits for the peers; visibility to a consumer on another GPU is the caller's
// ordering (end of the kernel plus whatever it uses between ranks).
__device__ __forceinline__ void store_out(const DecodeParams& p, int b, int hq, int idx, float v) {
    p.out[((size_t)b * p.num_heads + hq) * p.d + idx] = v;
    for (int r = 0; r < p.n_gather; r++)
        p.gather[r][gather_offset(p, b, hq) + idx] = v;
}
__device__ __forceinline__ void store_out4(const DecodeParams& p, int b, int hq, int idx, float4 v) {
    *reinterpret_cast<float4*>(p.out + ((size_t)b * p.num_heads + hq) * p.d + idx) = v;
    for (int r = 0; r < p.n_gather; r++)
        *reinterpret_cast<float4*>(p.gather[r] + gather_offset(p, b, hq) + idx) = v;
}

__device__ __forceinline__ long long range_start(long long total, int n_ctas, int c) {
    return (total * c) / n_ctas;
}

// ------------------------------------------------------------------------------------ plan
// One block.  Builds the page prefix sum, validates lengths, zeroes the rows of empty
// sequences and finds the first sequence of every CTA's range.
__global__ void __launch_bounds__(1024) decode_plan_kernel(DecodeParams p) {
    __shared__ int warp_sums[32];
    __shared__ int carry;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        carry = 0;
        p.page_prefix[0] = 0;
    }
    __syncthreads();
    if (p.fused_merge)
        for (int i = tid; i < p.batch * p.n_head_tiles * kConsumerWarps; i += 1024) p.pages_done[i] = 0;
    const int max_len = p.contiguous ? p.max_seq : p.max_blocks * kPageTokens;
    for (int base = 0; base < p.batch; base += 1024) {
        int b = base + tid;
        int pages = 0;
        if (b < p.batch) {
            int len = p.seq_lens ? p.seq_lens[b] : p.uniform_len;
            if (len < 0 || len > max_len) {
                atomicOr(p.status, kStatusBadSeqLen);
                len = 0;
            }
            pages = (len + kPageTokens - 1) / kPageTokens;
        }
        int incl = pages;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = warp_sums[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int v = __shfl_up_sync(0xffffffffu, w, o);
                if (lane >= o) w += v;
            }
            warp_sums[lane] = w;
        }
        __syncthreads();
        int before = carry + (warp > 0 ? warp_sums[warp - 1] : 0);
        if (b < p.batch) p.page_prefix[b + 1] = before + incl;
        __syncthreads();
        if (tid == 1023) carry = before + incl;
        __syncthreads();
    }
    __threadfence_block();
    __syncthreads();
    const int total = p.page_prefix[p.batch];
    // rows of empty sequences are defined to be zero (rare: one thread per such row)
    for (int b = tid; b < p.batch; b += 1024) {
        if (p.page_prefix[b + 1] == p.page_prefix[b]) {
            for (int h = 0; h < p.num_heads; h++)
                for (int i = 0; i < p.d; i++) store_out(p, b, h, i, 0.f);
        }
    }
    const long long T = (long long)total * p.n_head_tiles;
    for (int c = tid; c < p.n_ctas; c += 1024) {
        int first = 0;
        if (total > 0) {
            long long P0 = range_start(T, p.n_ctas, c);
            int p0 = (int)(P0 % total);
            // largest b with prefix[b] <= p0 and prefix[b+1] > p0
            int lo = 0, hi = p.batch;  // invariant: prefix[lo] <= p0 < prefix[hi]
            while (hi - lo > 1) {
                int mid = (lo + hi) >> 1;
                if (p.page_prefix[mid] <= p0) lo = mid; else hi = mid;
            }
            first = lo;
        }
        p.cta_first_seq[c] = first;
    }
}

// ------------------------------------------------------------------------------------ main
struct Segment {
    int seq;         // sequence index
    int head_tile;   // which tile of KV heads
    int page_begin;  // first logical page of the segment inside the sequence
    int npages;      // pages in the segment
    int seq_pages;   // pages of the whole sequence
    int slot;        // partial slot (2*cta or 2*cta+1); -1 when the segment is the whole sequence
};

// Direct mode: pages per CTA when `n` CTAs share a sequence of `pages` pages (the last shares may be short or empty).
__host__ __device__ __forceinline__ int direct_share(int pages, int n) { return (pages + n - 1) / n; }

// Walks the CTA's range; every role calls it with the same arguments and sees the same segments.
struct SegmentWalker {
    long long P, P1;
    int total, batch, b, cta, index;
    const int* prefix;
    int direct_pages;  // direct mode: pages of this CTA's sequence, -1 once handed out; -2: not direct
    int n_direct;      // direct mode: CTAs per (sequence, KV head)
    __device__ SegmentWalker(const DecodeParams& p, int cta_, const int* prefix_) {
        direct_pages = -2;
        if (p.direct) {
            // CTA = (share, KV head, sequence): an equal share of the sequence's pages is its one segment
            cta = cta_;
            n_direct = p.direct;
            index = (int)blockIdx.x;  // which share
            total = (int)blockIdx.y;  // the head tile
            b = (int)blockIdx.z;
            int len = p.seq_lens ? p.seq_lens[b] : p.uniform_len;
            const int max_len = p.contiguous ? p.max_seq : p.max_blocks * kPageTokens;
            if (len < 0 || len > max_len) {
                atomicOr(p.status, kStatusBadSeqLen);
                len = 0;
            }
            direct_pages = (len + kPageTokens - 1) / kPageTokens;
            return;
        }
        prefix = prefix_;
        batch = p.batch;
        total = prefix[batch];
        cta = cta_;
        long long T = (long long)total * p.n_head_tiles;
        P = range_start(T, p.n_ctas, cta);
        P1 = range_start(T, p.n_ctas, cta + 1);
        if (p.self_plan) {
            // largest b with prefix[b] <= p0 (what the plan kernel tabulates per CTA otherwise)
            const int p0 = total > 0 ? (int)(P % total) : 0;
            int lo = 0, hi = batch;
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (prefix[mid] <= p0) lo = mid; else hi = mid;
            }
            b = lo;
        } else {
            b = p.cta_first_seq[cta];
        }
        index = 0;
    }
    __device__ bool next(Segment& s) {
        if (direct_pages != -2) {
            if (direct_pages <= 0) return false;  // handed out already, or an empty sequence
            const int share = direct_share(direct_pages, n_direct);
            s.seq = b;
            s.head_tile = total;
            s.page_begin = index * share;
            s.npages = min(share, direct_pages - s.page_begin);
            s.seq_pages = direct_pages;
            s.slot = direct_pages > share ? cta : -1;  // a partial when other CTAs hold pages of the sequence too
            direct_pages = -1;
            return s.npages > 0;
        }
        if (P >= P1) return false;
        int ht = (int)(P / total);
        int pg = (int)(P - (long long)ht * total);
        if (pg == 0) b = 0;
        while (prefix[b + 1] <= pg) b++;  // skips empty sequences; prefix[batch] == total > pg
        int seq_begin = prefix[b], seq_end = prefix[b + 1];
        long long room = P1 - P;
        int end = seq_end;
        if ((long long)(end - pg) > room) end = pg + (int)room;
        s.seq = b;
        s.head_tile = ht;
        s.page_begin = pg - seq_begin;
        s.npages = end - pg;
        s.seq_pages = seq_end - seq_begin;
        bool whole = (pg == seq_begin) && (end == seq_end);
        s.slot = whole ? -1 : 2 * cta + (index == 0 ? 0 : 1);
        index++;
        P += s.npages;
        return true;
    }
};

// ------------------------------------------------------------------------------------ merge
// A sequence cut by range boundaries leaves one partial (m, l, o) per CTA that touched it.  The
// consumer warp that finishes the last of its pages (counted per warp index, since the same warp
// index owns the same heads in every CTA) combines them:
//     out = sum_c 2^(m_c-M) o_c / sum_c 2^(m_c-M) l_c
// always in CTA order, so the result does not depend on which warp came last.  Nothing waits: a
// warp that is not last simply moves on.  Partials are read through L2 (written by other SMs).
constexpr int kMaxMergeParts = 256;  // >= the largest grid the decode kernel is launched with
template <int D>
__device__ __forceinline__ void merge_cut_sequence(const DecodeParams& p, const int* prefix, int b, int ht, int hq0, int n_q, int lane) {
    const int total = prefix[p.batch];
    const int s0 = prefix[b], s1 = prefix[b + 1];
    const long long T = (long long)total * p.n_head_tiles;
    const long long A = (long long)ht * total + s0, B = (long long)ht * total + s1;  // the sequence's pages [A, B)
    auto cta_of = [&](long long P) {
        int c = (int)((P * p.n_ctas) / T);
        if (c >= p.n_ctas) c = p.n_ctas - 1;
        while (c + 1 < p.n_ctas && range_start(T, p.n_ctas, c + 1) <= P) c++;
        while (c > 0 && range_start(T, p.n_ctas, c) > P) c--;
        return c;
    };
    const int c_lo = cta_of(A), c_hi = cta_of(B - 1);
    const int n = min(c_hi - c_lo + 1, kMaxMergeParts);
    // The first contributing range may hold the sequence as its second partial (slot 1); every
    // later one starts inside the sequence, so the sequence is its first segment (slot 0).
    // Ranges in between can be empty when there are fewer pages than CTAs: those wrote nothing.
    int slot_l[kMaxMergeParts / 32];
#pragma unroll
    for (int k = 0; k < kMaxMergeParts / 32; k++) {
        const int i = k * 32 + lane;
        slot_l[k] = -1;
        if (i < n) {
            const int c = c_lo + i;
            const bool empty = i > 0 && range_start(T, p.n_ctas, c) == range_start(T, p.n_ctas, c + 1);
            if (!empty) slot_l[k] = i == 0 ? 2 * c + (range_start(T, p.n_ctas, c) >= A ? 0 : 1) : 2 * c;
        }
    }
    for (int h = 0; h < n_q; h++) {
        const int hq = hq0 + h;
        float w_l[kMaxMergeParts / 32], l_l[kMaxMergeParts / 32];
        float M = -INFINITY;
#pragma unroll
        for (int k = 0; k < kMaxMergeParts / 32; k++) {
            w_l[k] = -INFINITY;
            l_l[k] = 0.f;
            if (k * 32 < n && slot_l[k] >= 0) {
                const float2 ml = __ldcg(p.part_ml + (size_t)slot_l[k] * p.num_heads + hq);
                w_l[k] = ml.x;
                l_l[k] = ml.y;
            }
            M = fmaxf(M, w_l[k]);
        }
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, sh));
        float L = 0.f;
#pragma unroll
        for (int k = 0; k < kMaxMergeParts / 32; k++) {
            w_l[k] = slot_l[k] >= 0 ? fast_exp2(w_l[k] - M) : 0.f;
            L += w_l[k] * l_l[k];
        }
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) L += __shfl_xor_sync(0xffffffffu, L, sh);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < kMaxMergeParts / 32; k++) {
            if (k * 32 >= n) break;
            const int lim = min(32, n - k * 32);
            for (int j = 0; j < lim; j++) {
                const int slot = __shfl_sync(0xffffffffu, slot_l[k], j);
                const float w = __shfl_sync(0xffffffffu, w_l[k], j);
                if (slot < 0 || lane * 4 >= D) continue;
                const float4 o = __ldcg(reinterpret_cast<const float4*>(p.part_o + ((size_t)slot * p.num_heads + hq) * D) + lane);
                acc.x += w * o.x;
                acc.y += w * o.y;
                acc.z += w * o.z;
                acc.w += w * o.w;
            }
        }
        if (lane * 4 < D) {
            const float inv = 1.0f / L;
            store_out4(p, b, hq, lane * 4, make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv));
        }
    }
}

// Direct mode with several CTAs per (sequence, KV head): partial `i` of the pair sits in slot `first_slot + i`
// (the CTA's index); at most 32 of them, one per lane for the weights.  Always combined in slot order.
template <int D>
__device__ __forceinline__ void merge_direct(const DecodeParams& p, int b, int hq0, int n_q, int first_slot, int parts, int lane) {
    // Four heads and four partials at a time, every load of a batch issued before the first is used: the partials
    // come from L2 (other SMs wrote them), and one warp walking them one by one would pay that latency per load.
    constexpr int kH = 4, kJ = 4;
    const bool col_ok = lane * 4 < D;
    for (int h0 = 0; h0 < n_q; h0 += kH) {
        float m[kH], l[kH], w[kH], L[kH];
#pragma unroll
        for (int u = 0; u < kH; u++) {
            m[u] = -INFINITY;
            l[u] = 0.f;
            if (lane < parts && h0 + u < n_q) {
                const float2 ml = __ldcg(p.part_ml + (size_t)(first_slot + lane) * p.num_heads + hq0 + h0 + u);
                m[u] = ml.x;
                l[u] = ml.y;
            }
        }
#pragma unroll
        for (int u = 0; u < kH; u++) {
            float M = m[u];
#pragma unroll
            for (int sh = 16; sh > 0; sh >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, sh));
            w[u] = (lane < parts && h0 + u < n_q) ? fast_exp2(m[u] - M) : 0.f;
            L[u] = w[u] * l[u];
#pragma unroll
            for (int sh = 16; sh > 0; sh >>= 1) L[u] += __shfl_xor_sync(0xffffffffu, L[u], sh);
        }
        float4 acc[kH];
#pragma unroll
        for (int u = 0; u < kH; u++) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j0 = 0; j0 < parts; j0 += kJ) {
            float4 o[kH][kJ];
#pragma unroll
            for (int u = 0; u < kH; u++)
#pragma unroll
                for (int v = 0; v < kJ; v++) {
                    o[u][v] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (col_ok && j0 + v < parts && h0 + u < n_q)
                        o[u][v] = __ldcg(reinterpret_cast<const float4*>(p.part_o + ((size_t)(first_slot + j0 + v) * p.num_heads + hq0 + h0 + u) * D) + lane);
                }
#pragma unroll
            for (int v = 0; v < kJ; v++)  // always in slot order
#pragma unroll
                for (int u = 0; u < kH; u++) {
                    const float wj = __shfl_sync(0xffffffffu, w[u], (j0 + v) & 31);  // 0 beyond the last partial (o is 0 there too)
                    acc[u].x += wj * o[u][v].x;
                    acc[u].y += wj * o[u][v].y;
                    acc[u].z += wj * o[u][v].z;
                    acc[u].w += wj * o[u][v].w;
                }
        }
#pragma unroll
        for (int u = 0; u < kH; u++)
            if (col_ok && h0 + u < n_q) {
                const float inv = 1.0f / L[u];
                store_out4(p, b, hq0 + h0 + u, lane * 4, make_float4(acc[u].x * inv, acc[u].y * inv, acc[u].z * inv, acc[u].w * inv));
            }
    }
}

#ifndef GB_DECODE_PAGES_PER_ITER_D128
#define GB_DECODE_PAGES_PER_ITER_D128 1
#endif
#ifndef GB_DECODE_PAGES_PER_ITER_D64
#define GB_DECODE_PAGES_PER_ITER_D64 2
#endif
// kSplit: the build for tiles of fewer than eight KV heads, whose warps share a head's pages (page_split > 1) -
// a build of its own so that the exchange and merge code costs the eight-head kernel no registers.
template <int NT, int D, bool kSplit, int PP = (D == 64 ? GB_DECODE_PAGES_PER_ITER_D64 : GB_DECODE_PAGES_PER_ITER_D128)>
__global__ void __launch_bounds__(kDecodeThreads, 1)
paged_decode_kernel(const __grid_constant__ CUtensorMap kmap,
                    const __grid_constant__ CUtensorMap vmap, const __grid_constant__ DecodeParams p) {
    {
        // The parameters span several constant-cache lines, all cold at the start of a launch: one load from each
        // line now lets their misses overlap instead of stalling the roles one field at a time (a short call is
        // mostly start-up latency).
        int touch = 0;
#pragma unroll
        for (int i = 0; i < (int)sizeof(DecodeParams); i += 64) touch |= reinterpret_cast<const int*>(&p)[i / 4];
        asm volatile("" ::"r"(touch));
    }
    constexpr int kDSteps = D / 16;                     // 16-wide steps along head_dim
    constexpr int kChunks = D / 64;                     // 128-byte swizzle blocks per row
    constexpr int kHeadPageBytes = kPageTokens * D * 2;  // one head's K (or V) page
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzle wants 1024-byte aligned slots
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int slot_bytes = p.tile_heads * kHeadPageBytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)p.slots * slot_bytes);
    uint64_t* empty = full + kMaxSlots;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + kMaxSlots);
    // page split: per KV head of the tile, "the other warps have dumped" and "the dumps have been read"
    uint64_t* dumped = empty + kMaxSlots + 8;
    uint64_t* drained = dumped + 4;
    float* dump_area = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(empty + kMaxSlots) + p.dump_offset);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // one barrier pair per thread (a single thread initialising up to 136 barriers costs over a thousand clocks,
    // which a short call feels)
    for (int i = threadIdx.x; i < p.slots; i += kDecodeThreads) {
        mbar_init(&full[i], 1);
        mbar_init(&empty[i], p.slot_arrivals);
    }
    if (threadIdx.x >= kDecodeThreads - 4) {
        const int i = threadIdx.x - (kDecodeThreads - 4);
        mbar_init(&dumped[i], max(p.page_split - 1, 1));
        mbar_init(&drained[i], 1);
    }
    if (threadIdx.x == 0) *abort_flag = 0;
    mbar_fence_init();
    const int* prefix = p.page_prefix;
    if (p.self_plan) {
        // The plan for a small batch, by every CTA for itself (one sequence per thread): page counts, their
        // inclusive scan, the prefix array in shared memory.  Saves the plan kernel's launch in front of every step.
        int* s_prefix = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(empty + kMaxSlots) + p.plan_offset);
        int* s_warp = s_prefix + p.batch + 1;  // [kDecodeThreads / 32] warp totals
        int pages = 0;
        if ((int)threadIdx.x < p.batch) {
            int len = p.seq_lens ? p.seq_lens[threadIdx.x] : p.uniform_len;
            const int max_len = p.contiguous ? p.max_seq : p.max_blocks * kPageTokens;
            if (len < 0 || len > max_len) {
                atomicOr(p.status, kStatusBadSeqLen);
                len = 0;
            }
            pages = (len + kPageTokens - 1) / kPageTokens;
        }
        int incl = pages;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        for (int w = 0; w < warp; w++) incl += s_warp[w];
        if ((int)threadIdx.x < p.batch) s_prefix[threadIdx.x + 1] = incl;
        if (threadIdx.x == 0) s_prefix[0] = 0;
        __syncthreads();
        if (blockIdx.x == 0 && (int)threadIdx.x < p.batch && pages == 0) {
            // rows of empty sequences are defined to be zero (rare: one thread per such sequence)
            for (int h = 0; h < p.num_heads; h++)
                for (int i = 0; i < p.d; i++) store_out(p, threadIdx.x, h, i, 0.f);
        }
        prefix = s_prefix;
    } else {
        __syncthreads();
    }
    if (!p.direct && prefix[p.batch] == 0) return;

    const int cta_linear = (int)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x);
    SegmentWalker walk(p, cta_linear, prefix);
    if (p.direct && walk.direct_pages == 0) {
        // an empty sequence: its rows are defined to be zero (the plan kernel does this otherwise)
        if (walk.index == 0)
            for (int i = threadIdx.x; i < p.group * p.d; i += kDecodeThreads) store_out(p, walk.b, walk.total * p.group + i / p.d, i % p.d, 0.f);
        return;
    }
    Segment seg;
    int slot = 0;
    uint32_t phase = 0;
    auto advance = [&]() {
        if (++slot == p.slots) {
            slot = 0;
            phase ^= 1;
        }
    };

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------ producer warp
        if (lane == 0) {
            tma_prefetch_desc(&kmap);
            tma_prefetch_desc(&vmap);
        }
        // One TMA instruction moves a whole K (or V) page of the head tile: the box spans
        // {64 halfs, 16 rows, the head's 64-wide chunks, tile_heads heads} and lands as
        // [head][chunk][row][64].
        while (walk.next(seg)) {
            const int head0 = seg.head_tile * p.tile_heads;
            for (int j0 = 0; j0 < seg.npages; j0 += 32) {
                int e = 0;
                if (j0 + lane < seg.npages) {
                    int logical = seg.page_begin + j0 + lane;
                    if (p.contiguous) {
                        e = logical;
                    } else {
                        e = p.tables[(size_t)seg.seq * p.max_blocks + logical];
                        if (e < 0 || e >= p.num_blocks) {
                            atomicOr(p.status, kStatusBadTable);
                            e = 0;
                        }
                    }
                }
                const int n = min(32, seg.npages - j0);
                // Several pages per round: lane 2k issues K of the round's k-th page, lane 2k + 1 its V, each after
                // its own slot has been released, so the boxes of a round are in flight together.  (A round never
                // uses more than half the ring, so a slot's parity is unambiguous.)
                const int per_round = p.per_round;
                for (int jj0 = 0; jj0 < n; jj0 += per_round) {
                    const int cnt = min(per_round, n - jj0);
                    const int entry = __shfl_sync(0xffffffffu, e, (jj0 + (lane >> 1)) & 31);
                    int ok = 1;
                    if (lane < 2 * cnt) {
                        int my_slot = slot + lane;
                        uint32_t my_phase = phase;
                        if (my_slot >= p.slots) {
                            my_slot -= p.slots;
                            my_phase ^= 1;
                        }
                        ok = mbar_wait(&empty[my_slot], my_phase ^ 1, abort_flag);
                        if (ok) {
                            mbar_arrive_expect_tx(&full[my_slot], slot_bytes);
                            // contiguous cache: dim 3 runs over (sequence, head); pool: over heads
                            const int w = p.contiguous ? seg.seq * p.num_kv_heads + head0 : head0;
                            tma_load_4d(smem + (size_t)my_slot * slot_bytes, (lane & 1) ? &vmap : &kmap, &full[my_slot], 0,
                                        entry * kPageTokens, 0, w);
                        }
                    }
                    if (!__all_sync(0xffffffffu, ok)) {
                        if (lane == 0) atomicOr(p.status, kStatusTimeout);
                        return;
                    }
                    slot += 2 * cnt;
                    if (slot >= p.slots) {
                        slot -= p.slots;
                        phase ^= 1;
                    }
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumer warps
    const int kvh_local = warp & (p.tile_heads - 1);
    const int sub = warp >> p.tile_shift;
    constexpr bool split = kSplit;  // the launcher picks the build by p.page_split > 1
    const int first_q = split ? 0 : sub * p.heads_per_warp;  // first query head of the group owned here
    if (first_q >= p.group) return;              // idle warp (not counted in active_warps)
    const int n_q = min(p.heads_per_warp, p.group - first_q);
    int segments_done = 0;                       // page split: parity of the exchange barriers
    const int g = lane >> 2, t = lane & 3;

    // per-lane shared-memory offsets of the ldmatrix rows
    const int k_row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int k_unit = lane >> 4;
    const int v_row = (lane & 7) + ((lane >> 4) & 1) * 8;
    const int v_unit = (lane >> 3) & 1;
    const uint32_t smem_base = smem_u32(smem) + kvh_local * kHeadPageBytes;
    // cut sequences whose last pages this warp finished: merged after the walk (at most the first
    // and the last segment of a range are cut), so that the page ring never waits for a merge
    int merge_seq[2] = {-1, -1}, merge_ht[2] = {0, 0};

    while (walk.next(seg)) {
        const int kvh = seg.head_tile * p.tile_heads + kvh_local;
        const int hq0 = kvh * p.group + first_q;
        const int len = p.seq_lens ? p.seq_lens[seg.seq] : p.uniform_len;

        // Q^T as the B operand: lane (g,t) holds head nt*8+g, dims ks*16 + {2t,2t+1, 2t+8,2t+9}
        uint32_t qhi[NT][kDSteps][2], qlo[NT][kDSteps][2];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int n = nt * 8 + g;
            const bool valid = n < n_q;
            const float* qp = p.q + ((size_t)seg.seq * p.num_heads + hq0 + (valid ? n : 0)) * D;
#pragma unroll
            for (int ks = 0; ks < kDSteps; ks++) {
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    float2 v = make_float2(0.f, 0.f);
                    if (valid) v = *reinterpret_cast<const float2*>(qp + ks * 16 + half * 8 + 2 * t);
                    v.x *= p.scale_log2;
                    v.y *= p.scale_log2;
                    __half2 hi = __floats2half2_rn(v.x, v.y);
                    float2 back = __half22float2(hi);
                    __half2 lo = __floats2half2_rn(v.x - back.x, v.y - back.y);
                    qhi[nt][ks][half] = *reinterpret_cast<uint32_t*>(&hi);
                    qlo[nt][ks][half] = *reinterpret_cast<uint32_t*>(&lo);
                }
            }
        }

        float m_run[NT][2], l_run[NT][2], o[NT][kDSteps][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            m_run[nt][0] = m_run[nt][1] = -INFINITY;
            l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
            for (int mt = 0; mt < kDSteps; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) o[nt][mt][i] = 0.f;
        }

        // PP pages per iteration.  With head_dim 64 a page is half the bytes for the same chain of
        // waits, shuffles and exponentials, so two pages share one softmax round (32 tokens) and
        // their MMA chains interleave.
        for (int j = 0; j < seg.npages; j += PP) {
            int ntok[PP], slot_k[PP], slot_v[PP];
            uint32_t ph_k[PP], ph_v[PP];
            bool has[PP];
#pragma unroll
            for (int pp = 0; pp < PP; pp++) {
                has[pp] = j + pp < seg.npages;
                ntok[pp] = 0;
                slot_k[pp] = slot_v[pp] = 0;
                ph_k[pp] = ph_v[pp] = 0;
                if (has[pp]) {
                    ntok[pp] = min(kPageTokens, len - (seg.page_begin + j + pp) * kPageTokens);
                    slot_k[pp] = slot; ph_k[pp] = phase; advance();
                    slot_v[pp] = slot; ph_v[pp] = phase; advance();
                }
            }
            if (split && (j / PP) % p.page_split != sub) continue;  // another warp of this head takes these pages

            // ---- S^T = K Q^T
            float sa[PP][NT][4], sb[PP][NT][4];
            uint32_t kbase[PP];
#pragma unroll
            for (int pp = 0; pp < PP; pp++) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) sa[pp][nt][i] = sb[pp][nt][i] = 0.f;
                kbase[pp] = smem_base + slot_k[pp] * slot_bytes + k_row * 128;
                // the outcome is made warp-uniform: a lane that gave up must not leave the others to the
                // warp-wide ldmatrix / shuffles that follow
                if (has[pp] && !__all_sync(0xffffffffu, mbar_wait(&full[slot_k[pp]], ph_k[pp], abort_flag))) {
                    if (lane == 0) atomicOr(p.status, kStatusTimeout);
                    return;
                }
            }
#pragma unroll
            for (int ks = 0; ks < kDSteps; ks++) {
                const int unit = (ks & 3) * 2 + k_unit;
#pragma unroll
                for (int pp = 0; pp < PP; pp++) {
                    if (pp > 0 && !has[pp]) continue;  // warp-uniform
                    uint32_t a[4];
                    ldmatrix_x4(a, kbase[pp] + (ks >> 2) * 2048 + ((unit ^ (k_row & 7)) << 4));
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        mma_16816(sa[pp][nt], a, qhi[nt][ks][0], qhi[nt][ks][1]);
                        mma_16816(sb[pp][nt], a, qlo[nt][ks][0], qlo[nt][ks][1]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) {
#pragma unroll
                for (int pp = 0; pp < PP; pp++)
                    if (has[pp]) mbar_arrive(&empty[slot_k[pp]]);
            }

            // ---- online softmax (lane holds tokens g, g+8 of each page for heads 2t, 2t+1 of each n-tile)
            uint32_t phi[PP][NT][2], plo[PP][NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                float s[PP][4];
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int pp = 0; pp < PP; pp++) {
                    s[pp][0] = sa[pp][nt][0] + sb[pp][nt][0];
                    s[pp][1] = sa[pp][nt][1] + sb[pp][nt][1];
                    s[pp][2] = sa[pp][nt][2] + sb[pp][nt][2];
                    s[pp][3] = sa[pp][nt][3] + sb[pp][nt][3];
                    if (g >= ntok[pp]) s[pp][0] = s[pp][1] = -INFINITY;
                    if (g + 8 >= ntok[pp]) s[pp][2] = s[pp][3] = -INFINITY;
                    mx0 = fmaxf(mx0, fmaxf(s[pp][0], s[pp][2]));
                    mx1 = fmaxf(mx1, fmaxf(s[pp][1], s[pp][3]));
                }
#pragma unroll
                for (int sh = 4; sh < 32; sh <<= 1) {
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
                }
                const float mn0 = fmaxf(m_run[nt][0], mx0), mn1 = fmaxf(m_run[nt][1], mx1);
                const float alpha0 = fast_exp2(m_run[nt][0] - mn0);
                const float alpha1 = fast_exp2(m_run[nt][1] - mn1);
                m_run[nt][0] = mn0;
                m_run[nt][1] = mn1;
                float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
                for (int pp = 0; pp < PP; pp++) {
                    const float p0 = fast_exp2(s[pp][0] - mn0), p1 = fast_exp2(s[pp][1] - mn1);
                    const float p2 = fast_exp2(s[pp][2] - mn0), p3 = fast_exp2(s[pp][3] - mn1);
                    if (pp == 0) {
                        sum0 = p0 + p2;
                        sum1 = p1 + p3;
                    } else {
                        sum0 += p0 + p2;
                        sum1 += p1 + p3;
                    }
                    __half2 h01 = __floats2half2_rn(p0, p1), h23 = __floats2half2_rn(p2, p3);
                    float2 b01 = __half22float2(h01), b23 = __half22float2(h23);
                    __half2 l01 = __floats2half2_rn(p0 - b01.x, p1 - b01.y);
                    __half2 l23 = __floats2half2_rn(p2 - b23.x, p3 - b23.y);
                    // C-fragment layout -> B-fragment layout: transpose the 8x8 (token, head) blocks
                    phi[pp][nt][0] = movmatrix_trans(*reinterpret_cast<uint32_t*>(&h01));
                    phi[pp][nt][1] = movmatrix_trans(*reinterpret_cast<uint32_t*>(&h23));
                    plo[pp][nt][0] = movmatrix_trans(*reinterpret_cast<uint32_t*>(&l01));
                    plo[pp][nt][1] = movmatrix_trans(*reinterpret_cast<uint32_t*>(&l23));
                }
                l_run[nt][0] = l_run[nt][0] * alpha0 + sum0;
                l_run[nt][1] = l_run[nt][1] * alpha1 + sum1;
#pragma unroll
                for (int mt = 0; mt < kDSteps; mt++) {
                    o[nt][mt][0] *= alpha0;
                    o[nt][mt][1] *= alpha1;
                    o[nt][mt][2] *= alpha0;
                    o[nt][mt][3] *= alpha1;
                }
            }

            // ---- O^T += V^T P^T
            uint32_t vbase[PP];
#pragma unroll
            for (int pp = 0; pp < PP; pp++) {
                vbase[pp] = smem_base + slot_v[pp] * slot_bytes + v_row * 128;
                if (!has[pp]) continue;
                if (!__all_sync(0xffffffffu, mbar_wait(&full[slot_v[pp]], ph_v[pp], abort_flag))) {
                    if (lane == 0) atomicOr(p.status, kStatusTimeout);
                    return;
                }
                if (ntok[pp] < kPageTokens) {
                    // rows past the sequence end may hold anything (even NaN): zero them so that
                    // 0 * garbage cannot poison the accumulators
                    uint8_t* vptr = smem + (size_t)slot_v[pp] * slot_bytes + kvh_local * kHeadPageBytes;
                    constexpr int kRowUnits = D / 8;  // 16-byte units per row
                    for (int i = lane; i < (kPageTokens - ntok[pp]) * kRowUnits; i += 32) {
                        int r = ntok[pp] + i / kRowUnits, u = i % kRowUnits;
                        int chunk = u >> 3, unit = u & 7;
                        *reinterpret_cast<uint4*>(vptr + chunk * 2048 + r * 128 + ((unit ^ (r & 7)) << 4)) =
                            make_uint4(0, 0, 0, 0);
                    }
                    __syncwarp();
                }
            }
#pragma unroll
            for (int mt = 0; mt < kDSteps; mt++) {
                const int unit = (mt & 3) * 2 + v_unit;
#pragma unroll
                for (int pp = 0; pp < PP; pp++) {
                    if (pp > 0 && !has[pp]) continue;  // warp-uniform; an absent page's slot holds other data
                    uint32_t a[4];
                    ldmatrix_x4_trans(a, vbase[pp] + (mt >> 2) * 2048 + ((unit ^ (v_row & 7)) << 4));
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        mma_16816(o[nt][mt], a, phi[pp][nt][0], phi[pp][nt][1]);
                        mma_16816(o[nt][mt], a, plo[pp][nt][0], plo[pp][nt][1]);
                    }
                }
            }
            __syncwarp();
#pragma unroll
            for (int pp = 0; pp < PP; pp++) {
                if (!has[pp]) continue;
                if (ntok[pp] < kPageTokens) fence_proxy_async_smem();
                if (lane == 0) mbar_arrive(&empty[slot_v[pp]]);
            }
        }

        if (split) {
            // ---- the warps of this head combine their shares of the segment's pages.  Every lane's state
            // (running maxima, partial sums, accumulator fragment) is dumped as it stands - all warps hold the same
            // fragment layout - and warp 0 of the head folds the dumps into its own, lane by lane.
            constexpr int kPerLane = NT * (kDSteps * 4 + 4);
            const uint32_t par = segments_done & 1;
            segments_done++;
            if (sub > 0) {
                // the previous segment's dumps must have been read before they are overwritten
                if (!__all_sync(0xffffffffu, mbar_wait(&drained[kvh_local], par ^ 1, abort_flag))) {
                    if (lane == 0) atomicOr(p.status, kStatusTimeout);
                    return;
                }
                // (16-byte pieces, lane-interleaved: group 0 of an n-tile is its maxima and sums, group 1 + mt the
                // four accumulators of step mt)
                float4* d = reinterpret_cast<float4*>(dump_area) + ((size_t)(kvh_local * (p.page_split - 1) + (sub - 1)) * (kPerLane / 4)) * 32 + lane;
                int k = 0;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    d[32 * k++] = make_float4(m_run[nt][0], m_run[nt][1], l_run[nt][0], l_run[nt][1]);
#pragma unroll
                    for (int mt = 0; mt < kDSteps; mt++) d[32 * k++] = make_float4(o[nt][mt][0], o[nt][mt][1], o[nt][mt][2], o[nt][mt][3]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&dumped[kvh_local]);
                continue;  // the result is warp 0's business
            }
            if (!__all_sync(0xffffffffu, mbar_wait(&dumped[kvh_local], par, abort_flag))) {
                if (lane == 0) atomicOr(p.status, kStatusTimeout);
                return;
            }
            // The new maxima first, then every dump weighted against them: no dump's arithmetic waits for the one
            // before it, so the shared-memory loads of all of them are in flight together.
            const float4* d0 = reinterpret_cast<const float4*>(dump_area) + ((size_t)(kvh_local * (p.page_split - 1)) * (kPerLane / 4)) * 32 + lane;
            float mn[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                mn[nt][0] = m_run[nt][0];
                mn[nt][1] = m_run[nt][1];
            }
            for (int w = 0; w < p.page_split - 1; w++) {
                const float4* d = d0 + (size_t)w * (kPerLane / 4) * 32;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const float4 ml = d[32 * (nt * (kDSteps + 1))];
                    mn[nt][0] = fmaxf(mn[nt][0], ml.x);
                    mn[nt][1] = fmaxf(mn[nt][1], ml.y);
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const float a0 = fast_exp2(m_run[nt][0] - mn[nt][0]), a1 = fast_exp2(m_run[nt][1] - mn[nt][1]);
                m_run[nt][0] = mn[nt][0];
                m_run[nt][1] = mn[nt][1];
                l_run[nt][0] *= a0;
                l_run[nt][1] *= a1;
#pragma unroll
                for (int mt = 0; mt < kDSteps; mt++) {
                    o[nt][mt][0] *= a0;
                    o[nt][mt][1] *= a1;
                    o[nt][mt][2] *= a0;
                    o[nt][mt][3] *= a1;
                }
            }
            // every dump's weights, then accumulator step by accumulator step over all dumps: the loop over the
            // (at most seven) dumps is unrolled and predicated, so that all of its loads are independent
            constexpr int kMaxDumps = kConsumerWarps - 1;
            float b[kMaxDumps][NT][2];
#pragma unroll
            for (int w = 0; w < kMaxDumps; w++) {
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    b[w][nt][0] = b[w][nt][1] = 0.f;
                    if (w < p.page_split - 1) {
                        const float4 ml = d0[((size_t)w * (kPerLane / 4) + nt * (kDSteps + 1)) * 32];
                        // (a warp that had no page dumps -inf and zeros: weight 0)
                        b[w][nt][0] = fast_exp2(ml.x - mn[nt][0]);
                        b[w][nt][1] = fast_exp2(ml.y - mn[nt][1]);
                        l_run[nt][0] += ml.z * b[w][nt][0];
                        l_run[nt][1] += ml.w * b[w][nt][1];
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
#pragma unroll
                for (int mt = 0; mt < kDSteps; mt++) {
#pragma unroll
                    for (int w = 0; w < kMaxDumps; w++) {
                        if (w < p.page_split - 1) {
                            const float4 ov = d0[((size_t)w * (kPerLane / 4) + nt * (kDSteps + 1) + 1 + mt) * 32];
                            o[nt][mt][0] += ov.x * b[w][nt][0];
                            o[nt][mt][1] += ov.y * b[w][nt][1];
                            o[nt][mt][2] += ov.z * b[w][nt][0];
                            o[nt][mt][3] += ov.w * b[w][nt][1];
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&drained[kvh_local]);
        }
        // ---- segment result
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
#pragma unroll
            for (int sh = 4; sh < 32; sh <<= 1) {
                l_run[nt][0] += __shfl_xor_sync(0xffffffffu, l_run[nt][0], sh);
                l_run[nt][1] += __shfl_xor_sync(0xffffffffu, l_run[nt][1], sh);
            }
#pragma unroll
            for (int jx = 0; jx < 2; jx++) {
                const int n = nt * 8 + 2 * t + jx;
                if (n >= n_q) continue;
                const int hq = hq0 + n;
                if (seg.slot < 0) {
                    const float inv = 1.0f / l_run[nt][jx];
#pragma unroll
                    float* dst = p.out + ((size_t)seg.seq * p.num_heads + hq) * D;
#pragma unroll
                    for (int mt = 0; mt < kDSteps; mt++) {
                        dst[mt * 16 + g] = o[nt][mt][jx] * inv;
                        dst[mt * 16 + g + 8] = o[nt][mt][2 + jx] * inv;
                    }
                } else {
                    float* dst = p.part_o + ((size_t)seg.slot * p.num_heads + hq) * D;
#pragma unroll
                    for (int mt = 0; mt < kDSteps; mt++) {
                        dst[mt * 16 + g] = o[nt][mt][jx];
                        dst[mt * 16 + g + 8] = o[nt][mt][2 + jx];
                    }
                    if (g == 0)
                        p.part_ml[(size_t)seg.slot * p.num_heads + hq] = make_float2(m_run[nt][jx], l_run[nt][jx]);
                }
            }
        }
        if (seg.slot < 0 && p.n_gather > 0) {
            // gather destinations get whole rows as 16-byte stores (a lane's own fragment holds every
            // eighth pair of a row, which would cross NVLink as 32-byte pieces): the warp reads back
            // the rows it has just written
            __syncwarp();
            for (int h = 0; h < n_q; h++) {
                if (lane * 4 >= D) continue;
                const size_t row = ((size_t)seg.seq * p.num_heads + hq0 + h) * D + lane * 4;
                const float4 v = __ldcg(reinterpret_cast<const float4*>(p.out + row));
                for (int r = 0; r < p.n_gather; r++)
                    *reinterpret_cast<float4*>(p.gather[r] + gather_offset(p, seg.seq, hq0 + h) + lane * 4) = v;
            }
        }
        if (kSplit && seg.slot >= 0 && p.direct) {
            // one of several CTAs of this (sequence, KV head): publish the partial and count the arrival; the CTA
            // that arrives last combines all of them (release: fence before the count; acquire: after).  The
            // counter wraps to zero with the last arrival, so it needs no reset between launches.  One acquire-release
            // atomic at GPU scope instead of fence + atomic + fence: the warp barrier orders the other lanes' stores
            // before it and their later loads after it.
            __syncwarp();
            const int parts = (seg.seq_pages + direct_share(seg.seq_pages, p.direct) - 1) / direct_share(seg.seq_pages, p.direct);
            int last = 0;
            if (lane == 0) {
                unsigned old;
                asm volatile("atom.acq_rel.gpu.global.inc.u32 %0, [%1], %2;"
                             : "=r"(old)
                             : "l"(p.direct_done + (size_t)seg.seq * p.n_head_tiles + seg.head_tile), "r"((unsigned)(parts - 1))
                             : "memory");
                last = old == (unsigned)(parts - 1);
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) merge_direct<D>(p, seg.seq, hq0, n_q, seg.slot - (int)blockIdx.x, parts, lane);
        }
        if (seg.slot >= 0 && p.fused_merge) {
            // publish the partial, then count this warp's pages of the sequence; the warp whose
            // count completes the sequence merges (release: fence before the add; acquire: after)
            __threadfence();
            __syncwarp();
            int last = 0;
            if (lane == 0) {
                int* done = p.pages_done + ((size_t)seg.seq * p.n_head_tiles + seg.head_tile) * kConsumerWarps + warp;
                last = atomicAdd(done, seg.npages) + seg.npages == seg.seq_pages;
                if (last) *done = 0;  // nobody else counts on it any more: ready for the next launch without a plan kernel
                __threadfence();
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                if (seg.slot & 1) {
                    merge_seq[1] = seg.seq;
                    merge_ht[1] = seg.head_tile;
                } else {
                    merge_seq[0] = seg.seq;
                    merge_ht[0] = seg.head_tile;
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        if (merge_seq[i] < 0) continue;  // (with split pages only warp 0 of a head ever records one)
        const int kvh = merge_ht[i] * p.tile_heads + kvh_local;
        merge_cut_sequence<D>(p, prefix, merge_seq[i], merge_ht[i], kvh * p.group + first_q, n_q, lane);
    }
}

// ------------------------------------------------------------------------------------ merge
// Separate merge pass, used when the batch is small against the number of CTAs (a sequence is then
// cut into many partials, which one warp would combine too slowly inside the decode kernel).
// grid (batch, num_heads), 256 threads.  Combines the partials of a sequence that was cut by CTA
// range boundaries:  out = sum_c 2^(m_c-M) o_c / sum_c 2^(m_c-M) l_c.  A single long sequence is cut
// by every CTA (a batch of one leaves as many partials as there are SMs), so the partials are
// spread over the block: one thread per partial for the maxima and weights, one warp per eighth
// of the partials (a lane per four output dims) for the weighted sum.
constexpr int kMergeThreads = 256;
__global__ void __launch_bounds__(kMergeThreads) decode_merge_kernel(DecodeParams p) {
    __shared__ float s_w[kMaxMergeParts];
    __shared__ int s_slot[kMaxMergeParts];
    __shared__ float s_red[kMergeThreads / 32];
    __shared__ float s_red2[kMergeThreads / 32];
    __shared__ float4 s_acc[kMergeThreads / 32][32];
    const int b = blockIdx.x, hq = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int total = p.page_prefix[p.batch];
    if (total == 0) return;
    const int s0 = p.page_prefix[b], s1 = p.page_prefix[b + 1];
    if (s1 == s0) return;
    const int ht = hq / (p.tile_heads * p.group);
    const long long T = (long long)total * p.n_head_tiles;
    const long long A = (long long)ht * total + s0, B = (long long)ht * total + s1;  // [A, B)
    auto cta_of = [&](long long P) {
        int c = (int)((P * p.n_ctas) / T);
        if (c >= p.n_ctas) c = p.n_ctas - 1;
        while (c + 1 < p.n_ctas && range_start(T, p.n_ctas, c + 1) <= P) c++;
        while (c > 0 && range_start(T, p.n_ctas, c) > P) c--;
        return c;
    };
    const int c_lo = cta_of(A), c_hi = cta_of(B - 1);
    if (c_lo == c_hi) return;  // whole sequence inside one range: already final
    const int n = min(c_hi - c_lo + 1, kMaxMergeParts);
    // The first contributing range may hold the sequence as its second partial (slot 1); every
    // later one starts inside the sequence, so the sequence is its first segment (slot 0).
    // Ranges in between can be empty when there are fewer pages than CTAs: those wrote nothing.
    float m_own = -INFINITY, l_own = 0.f;
    int slot_own = -1;
    if (tid < n) {
        const int c = c_lo + tid;
        const bool empty = tid > 0 && range_start(T, p.n_ctas, c) == range_start(T, p.n_ctas, c + 1);
        if (!empty) {
            slot_own = tid == 0 ? 2 * c + (range_start(T, p.n_ctas, c) >= A ? 0 : 1) : 2 * c;
            const float2 ml = p.part_ml[(size_t)slot_own * p.num_heads + hq];
            m_own = ml.x;
            l_own = ml.y;
        }
    }
    float M = m_own;
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, sh));
    if (lane == 0) s_red[warp] = M;
    __syncthreads();
    M = s_red[0];
#pragma unroll
    for (int w = 1; w < kMergeThreads / 32; w++) M = fmaxf(M, s_red[w]);
    const float w_own = slot_own >= 0 ? fast_exp2(m_own - M) : 0.f;
    if (tid < n) {
        s_w[tid] = w_own;
        s_slot[tid] = slot_own;
    }
    float L = w_own * l_own;
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) L += __shfl_xor_sync(0xffffffffu, L, sh);
    if (lane == 0) s_red2[warp] = L;
    __syncthreads();
    L = 0.f;
#pragma unroll
    for (int w = 0; w < kMergeThreads / 32; w++) L += s_red2[w];
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = warp; i < n; i += kMergeThreads / 32) {
        const int slot = s_slot[i];
        if (slot < 0) continue;
        const float w = s_w[i];
        if (lane * 4 >= p.d) continue;  // head_dim 64: half of the lanes carry data
        const float4 o = *(reinterpret_cast<const float4*>(p.part_o + ((size_t)slot * p.num_heads + hq) * p.d) + lane);
        acc.x += w * o.x;
        acc.y += w * o.y;
        acc.z += w * o.z;
        acc.w += w * o.w;
    }
    s_acc[warp][lane] = acc;
    __syncthreads();
    if (tid < p.d) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kMergeThreads / 32; w++) sum += reinterpret_cast<const float*>(&s_acc[w][0])[tid];
        store_out(p, b, hq, tid, sum / L);
    }
}

// ------------------------------------------------------------------------------------ host
static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// In-kernel merging costs one warp about a microsecond per handful of partials; it pays when a
// sequence is cut into few pieces, i.e. when there are at least a quarter as many (sequence,
// head tile) pairs as CTAs.  Smaller batches leave tens of partials per sequence to the merge kernel.
static int fused_merge_pays(int batch, int n_head_tiles, int n_ctas) {
    return (long long)batch * n_head_tiles * 4 >= n_ctas ? 1 : 0;
}

// How the eight consumer warps share a tile of `tile_heads` KV heads whose GQA group has `group` query heads, and
// the shared-memory window that goes with it.  Fills the shape fields of `p`; returns false when no tiling fits.
static bool plan_decode_tile(DecodeParams& p, int tile_heads, int group, int D, int smem_optin, size_t* smem_bytes) {
    const int warps_per_head = kConsumerWarps / tile_heads;
    p.tile_heads = tile_heads;
    p.tile_shift = tile_heads == 8 ? 3 : tile_heads == 4 ? 2 : tile_heads == 2 ? 1 : 0;
    p.page_split = 1;
    if (warps_per_head > 1 && group <= 16) {
        // few KV heads: the warps of a head split its pages, each for all query heads of the group
        p.page_split = warps_per_head;
        p.heads_per_warp = group;
        p.active_warps = kConsumerWarps;
        p.slot_arrivals = tile_heads;
    } else {
        p.heads_per_warp = (group + warps_per_head - 1) / warps_per_head;
        if (p.heads_per_warp > 16) return false;
        p.active_warps = ((group + p.heads_per_warp - 1) / p.heads_per_warp) * tile_heads;
        p.slot_arrivals = p.active_warps;
    }
    const int nt = p.heads_per_warp <= 8 ? 1 : 2;
    p.dump_bytes = nt * (D / 16 * 4 + 4) * 32 * (int)sizeof(float);
    p.dump_offset = 128;  // behind the abort flag and the exchange barriers
    const size_t dumps = p.page_split > 1 ? (size_t)(kConsumerWarps - tile_heads) * p.dump_bytes : 0;
    const int slot_bytes = tile_heads * kPageTokens * D * 2;
    const size_t tail = 2 * kMaxSlots * sizeof(uint64_t) + p.dump_offset + dumps;
    int slots = (int)((smem_optin - 1024 - (long long)tail) / slot_bytes);
    if (slots > kMaxSlots) slots = kMaxSlots;
    if (slots < 2) return false;
    p.slots = slots;
    // three pages (six boxes) per producer round, never more than half the ring: measured best for every tile
    // (one page per round: -6 % on eight-head tiles, -18 % on one-head tiles; seven on a 14-deep ring: -10 %)
    p.per_round = slots / 2 < 1 ? 1 : (slots / 2 > 3 ? 3 : slots / 2);
    *smem_bytes = 1024 + (size_t)slots * slot_bytes + tail;
    return true;
}

int launch_paged_decode(granite_cuda_compute* c, const GraniteCudaPagedDecodeArgs& a,
                        bool contiguous, uint32_t max_seq, const DecodeGather* gather) {
    if (gather && gather->n_dst > 0) {
        if (!gather->dst) return fail(GRANITE_CUDA_NULL_POINTER, "decode gather: null destination list");
        if (gather->n_dst > (uint32_t)kMaxGatherDst)
            return fail(GRANITE_CUDA_INVALID_ARGUMENT, "decode gather: at most 16 destinations");
        if (gather->dst_heads != 0 && (uint64_t)gather->head_offset + a.num_heads > gather->dst_heads)
            return fail(GRANITE_CUDA_INVALID_ARGUMENT, "decode gather: head_offset + num_heads exceeds the destination's heads");
        for (uint32_t r = 0; r < gather->n_dst; r++) {
            if (!gather->dst[r]) return fail(GRANITE_CUDA_NULL_POINTER, "decode gather: null destination");
            if (reinterpret_cast<uintptr_t>(gather->dst[r]) & 15)
                return fail(GRANITE_CUDA_INVALID_ARGUMENT, "decode gather: destinations must be 16-byte aligned");
        }
    } else {
        gather = nullptr;
    }
    if (!a.q || !a.k_cache || !a.v_cache || !a.output || (!contiguous && !a.block_tables))
        return fail(GRANITE_CUDA_NULL_POINTER, "paged decode: null buffer");
    if (a.batch_size == 0) return GRANITE_CUDA_SUCCESS;
    if (a.num_kv_heads == 0 || a.num_heads == 0 || a.num_heads % a.num_kv_heads != 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "paged decode: num_heads must be a multiple of num_kv_heads");
    // the plain kernel does not store to gather destinations itself: its rows are pushed afterwards
    auto plain = [&]() {
        if (gather && gather->dst_heads != 0 && gather->dst_heads != a.num_heads)
            return fail(GRANITE_CUDA_INVALID_ARGUMENT,
                        "decode gather: a head-sharded destination needs head_dim 128 or 64 and 16-token pages");
        int rc = launch_generic_decode(c, a, contiguous, max_seq);
        if (rc == GRANITE_CUDA_SUCCESS && gather) {
            const uint64_t row_bytes = (uint64_t)a.num_heads * a.head_dim * 4;
            rc = launch_push_rows(c, nullptr, a.output, gather->dst, gather->n_dst, gather->row_offset * row_bytes,
                                  a.batch_size * row_bytes);
        }
        return rc;
    };
    // shapes outside this kernel's tiling (head_dim 128 or 64, 16-token pages, at most 16 query heads per
    // consumer warp) run on the plain kernel
    if ((a.head_dim != 128 && a.head_dim != 64) || (!contiguous && a.block_size != kPageTokens))
        return plain();
    const int D = (int)a.head_dim;
    const int hkv = (int)a.num_kv_heads;
    // the largest of 8, 4, 2, 1 KV heads per tile that divides the head count (12 heads: three tiles of four)
    const int tile_heads = hkv % 8 == 0 ? 8 : hkv % 4 == 0 ? 4 : hkv % 2 == 0 ? 2 : 1;
    const int group = (int)(a.num_heads / a.num_kv_heads);
    const int n_ctas = c->sm_count < kMaxMergeParts ? c->sm_count : kMaxMergeParts;  // the merge holds up to 8 partials per lane
    // Small batches of short sequences (what single-user decoding is): too few (sequence, head tile) pairs to keep
    // the split partials few, and at most 128 pages per sequence.  A few CTAs per (sequence, KV head) then do the
    // whole job in one launch: each takes an equal share of the sequence's pages (at least four - one SM's TMA
    // unit moves a one-head page box per ~250 clocks, so a whole sequence on one SM would be bound by that), its
    // eight warps share them and combine in shared memory, and the last CTA of a pair to finish combines the
    // pair's partials.
    const uint32_t page_cap = a.seq_lens ? (contiguous ? (max_seq + kPageTokens - 1) / kPageTokens : a.max_blocks_per_seq)
                                         : (a.seq_len + kPageTokens - 1) / kPageTokens;
    const bool direct = group <= 16 && page_cap <= 128 && !fused_merge_pays((int)a.batch_size, hkv / tile_heads, n_ctas) &&
                        (int)a.batch_size * hkv <= kMaxDirectPairs;
    DecodeParams p{};
    size_t smem_bytes = 0;
    if (!plan_decode_tile(p, direct ? 1 : tile_heads, group, D, c->smem_optin, &smem_bytes)) return plain();
    const int nt = p.heads_per_warp <= 8 ? 1 : 2;
    if (contiguous) {
        if (max_seq == 0) return fail(GRANITE_CUDA_INVALID_ARGUMENT, "decode: max_seq must be positive");
    } else if (a.num_blocks == 0 || a.max_blocks_per_seq == 0) {
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "paged decode: empty pool or table");
    }

    p.q = a.q;
    p.tables = a.block_tables;
    p.seq_lens = a.seq_lens;
    p.out = a.output;
    p.batch = (int)a.batch_size;
    p.num_heads = (int)a.num_heads;
    p.num_kv_heads = hkv;
    p.group = group;
    p.max_blocks = (int)a.max_blocks_per_seq;
    p.num_blocks = (int)a.num_blocks;
    p.uniform_len = (int)a.seq_len;
    if (direct) {
        const int pairs = (int)a.batch_size * hkv;
        int per_pair = (int)(page_cap + kDirectMinPages - 1) / kDirectMinPages;
        per_pair = std::min(per_pair, std::min(n_ctas / pairs, 32));  // one lane per partial in the merge
        p.direct = std::max(per_pair, 1);
        p.direct_done = c->d_direct_done;
    }
    p.n_head_tiles = hkv / p.tile_heads;
    p.n_ctas = n_ctas;
    p.contiguous = contiguous ? 1 : 0;
    p.max_seq = (int)max_seq;
    p.scale_log2 = a.scale * 1.4426950408889634f;
    p.status = c->d_status;
    p.d = D;
    p.fused_merge = direct ? 0 : fused_merge_pays(p.batch, p.n_head_tiles, p.n_ctas);
    // Batches of up to 192 sequences whose cut sequences are merged inside the decode kernel need no plan kernel
    // if the prefix array (and nine warp totals) still fits behind the page ring without costing a slot.
    {
        const size_t plan_bytes = ((size_t)p.batch + 1 + kDecodeThreads / 32) * sizeof(int);
        const size_t spare = (size_t)c->smem_optin - smem_bytes;
        if (!direct && p.fused_merge && p.batch <= kSelfPlanMaxBatch && plan_bytes <= spare) {
            p.self_plan = 1;
            p.plan_offset = (int)(smem_bytes - 1024 - (size_t)p.slots * p.tile_heads * kPageTokens * D * 2 - 2 * kMaxSlots * sizeof(uint64_t));
            smem_bytes += plan_bytes;
        }
    }
    if (gather) {
        p.n_gather = (int)gather->n_dst;
        p.gather_row0 = (long long)gather->row_offset;
        p.gather_heads = gather->dst_heads ? (int)gather->dst_heads : p.num_heads;
        p.gather_head0 = (int)gather->head_offset;
        for (uint32_t r = 0; r < gather->n_dst; r++) p.gather[r] = static_cast<float*>(gather->dst[r]);
    }

    // scratch: prefix | first_seq | part_ml | part_o
    size_t off = 0;
    const size_t off_prefix = off; off = align_up(off + (size_t)(p.batch + 1) * 4, 256);
    const size_t off_first = off;  off = align_up(off + (size_t)p.n_ctas * 4, 256);
    const size_t off_ml = off;     off = align_up(off + (size_t)2 * p.n_ctas * p.num_heads * sizeof(float2), 256);
    const size_t off_o = off;      off = align_up(off + (size_t)2 * p.n_ctas * p.num_heads * D * 4, 256);
    const size_t off_done = off;   off = align_up(off + (size_t)p.batch * p.n_head_tiles * kConsumerWarps * 4, 256);
    int rc = c->ensure_scratch(off);
    if (rc) return rc;
    uint8_t* ws = static_cast<uint8_t*>(c->scratch);
    p.page_prefix = reinterpret_cast<int*>(ws + off_prefix);
    p.cta_first_seq = reinterpret_cast<int*>(ws + off_first);
    p.part_ml = reinterpret_cast<float2*>(ws + off_ml);
    p.part_o = reinterpret_cast<float*>(ws + off_o);
    p.pages_done = reinterpret_cast<int*>(ws + off_done);
    if (p.self_plan) {
        // no plan kernel zeroes the page counters: they live in an allocation of their own that starts at zero and
        // that the kernel leaves at zero (the warp that completes a count resets it)
        rc = c->ensure_page_counters((size_t)p.batch * p.n_head_tiles * kConsumerWarps);
        if (rc) return rc;
        p.pages_done = c->d_pages_done;
    }

    const CUtensorMap *kmap, *vmap;
    if (contiguous) {
        // [batch, Hkv, max_seq, D]: rows of one (sequence, head); a box past max_seq reads zeros
        const uint64_t planes = (uint64_t)a.batch_size * hkv;
        kmap = c->tensor_map_pages(a.k_cache, D, max_seq, D * 2, planes, (uint64_t)max_seq * D * 2, kPageTokens, p.tile_heads);
        vmap = c->tensor_map_pages(a.v_cache, D, max_seq, D * 2, planes, (uint64_t)max_seq * D * 2, kPageTokens, p.tile_heads);
    } else {
        // [num_blocks * 16, Hkv, D]
        const uint64_t rows = (uint64_t)a.num_blocks * kPageTokens;
        kmap = c->tensor_map_pages(a.k_cache, D, rows, (uint64_t)hkv * D * 2, hkv, D * 2, kPageTokens, p.tile_heads);
        vmap = c->tensor_map_pages(a.v_cache, D, rows, (uint64_t)hkv * D * 2, hkv, D * 2, kPageTokens, p.tile_heads);
    }
    if (!kmap || !vmap) return GRANITE_CUDA_EXECUTION_FAILED;

    auto kern = p.page_split > 1
                    ? (D == 128 ? (nt == 1 ? paged_decode_kernel<1, 128, true> : paged_decode_kernel<2, 128, true>)
                                : (nt == 1 ? paged_decode_kernel<1, 64, true> : paged_decode_kernel<2, 64, true>))
                    : (D == 128 ? (nt == 1 ? paged_decode_kernel<1, 128, false> : paged_decode_kernel<2, 128, false>)
                                : (nt == 1 ? paged_decode_kernel<1, 64, false> : paged_decode_kernel<2, 64, false>));
    // always the device's opt-in maximum: the limit belongs to the kernel, not to this call, and the
    // allocation-free entry point launches the same kernels with its own (possibly larger) window
    GB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, c->smem_optin));
    if (direct) {
        LaunchScope t(c, contiguous ? "contiguous_decode_direct" : "paged_decode_direct");
        kern<<<dim3(p.direct, hkv, p.batch), kDecodeThreads, smem_bytes, c->stream>>>(*kmap, *vmap, p);
        GB_CUDA_TRY(cudaGetLastError());
        return GRANITE_CUDA_SUCCESS;
    }
    if (!p.self_plan) {
        LaunchScope t(c, "decode_plan");
        decode_plan_kernel<<<1, 1024, 0, c->stream>>>(p);
    }
    {
        LaunchScope t(c, contiguous ? "contiguous_decode_splitkv" : "paged_decode_splitkv");
        kern<<<p.n_ctas, kDecodeThreads, smem_bytes, c->stream>>>(*kmap, *vmap, p);
    }
    if (!p.fused_merge) {
        LaunchScope t(c, "decode_merge");
        decode_merge_kernel<<<dim3(p.batch, p.num_heads), kMergeThreads, 0, c->stream>>>(p);
    }
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}

}  // namespace gb200

// =====================================================================================
// Allocation-free variant of the batched paged decode.
//
// Some hosts cannot let this library allocate: a serving process whose own arena already owns
// all of HBM (a cudaMalloc from a plug-in would fail or fragment it), and latency-critical
// loops where the implicit device-wide synchronisation of cudaMalloc/cudaFree is not
// acceptable.  For them the scratch that the split-KV decode needs (page prefix sums, the first
// sequence of every CTA range, and the partial (m, l, o) of sequences cut by a range boundary)
// lives in the fixed device array below instead of the compute object's growable arena.
// Every GPU that loads the library carries these ~13.8 MB until the process exits.
// =====================================================================================
namespace gb200 {

constexpr int kStaticMaxBatch = 4096;   // sequences per call
constexpr int kStaticMaxHeads = 64;     // query heads
constexpr int kStaticMaxCtas = 192;     // SMs of the device
constexpr size_t kStaticOffStatus = 0;
constexpr size_t kStaticOffPrefix = 256;
constexpr size_t kStaticOffFirst = kStaticOffPrefix + ((size_t)(kStaticMaxBatch + 1) * 4 + 255) / 256 * 256;
constexpr size_t kStaticOffMl = kStaticOffFirst + ((size_t)kStaticMaxCtas * 4 + 255) / 256 * 256;
constexpr size_t kStaticOffO = kStaticOffMl + (size_t)2 * kStaticMaxCtas * kStaticMaxHeads * sizeof(float2);
constexpr size_t kStaticOffDone = kStaticOffO + (size_t)2 * kStaticMaxCtas * kStaticMaxHeads * kHeadDim * 4;
// page counters: at most kStaticMaxHeads / 8 head tiles (eight KV heads per tile, or one tile)
constexpr size_t kStaticScratchBytes = kStaticOffDone + (size_t)kStaticMaxBatch * (kStaticMaxHeads / 8) * kConsumerWarps * 4;

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char g_static_decode_scratch[kStaticScratchBytes];

struct StaticDeviceSetup {
    bool ready = false;
    unsigned char* scratch = nullptr;  // device address of g_static_decode_scratch on this device
    int sm_count = 0;
    int smem_optin = 0;
};
constexpr int kMaxDevices = 64;
static StaticDeviceSetup g_static_setup[kMaxDevices];
static std::mutex g_static_setup_mutex;

// Once per device, with that device current: resolves the device address of the scratch array
// and reads the device's limits.  Allocates nothing.
static int static_decode_setup(int device, StaticDeviceSetup** out) {
    if (device < 0 || device >= kMaxDevices)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "static decode: device index out of range");
    std::lock_guard<std::mutex> lock(g_static_setup_mutex);
    StaticDeviceSetup& s = g_static_setup[device];
    if (!s.ready) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_decode_scratch);
        if (e != cudaSuccess || !ptr) {
            cudaGetLastError();
            return fail(GRANITE_CUDA_BACKEND_NOT_INITIALIZED,
                        std::string("static decode: cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
        }
        int major = 0;
        GB_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
        if (major != 10) return fail(GRANITE_CUDA_BACKEND_NOT_SUPPORTED, "static decode: built for sm_100a only");
        GB_CUDA_TRY(cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, device));
        GB_CUDA_TRY(cudaDeviceGetAttribute(&s.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
        s.scratch = static_cast<unsigned char*>(ptr);
        s.ready = true;
    }
    *out = &s;
    return GRANITE_CUDA_SUCCESS;
}

// A tensor map built on the stack (the compute object's cache would allocate host memory).
static int encode_pool_map(CUtensorMap* map, const void* base, uint64_t heads, uint64_t rows, uint32_t tile_heads) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn enc = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    if (!enc) return fail(GRANITE_CUDA_BACKEND_NOT_INITIALIZED, "static decode: cuTensorMapEncodeTiled unavailable");
    if (reinterpret_cast<uintptr_t>(base) & 15)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "static decode: K/V pools must be 16-byte aligned");
    // same shape as granite_cuda_compute::tensor_map_pages for the pool [rows, heads, 128]
    cuuint64_t dims[4] = {64, rows, kHeadDim / 64, heads};
    cuuint64_t strides[3] = {heads * kHeadDim * 2, 128, kHeadDim * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)kPageTokens, kHeadDim / 64, tile_heads};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(GRANITE_CUDA_EXECUTION_FAILED, "static decode: cuTensorMapEncodeTiled failed with " + std::to_string((int)r));
    return GRANITE_CUDA_SUCCESS;
}

}  // namespace gb200

extern "C" int granite_cuda_batched_paged_attention_decode_static(const GraniteCudaPagedDecodeArgs* args,
                                                                  void* stream, int32_t* device_status) {
    using namespace gb200;
    if (!args) return fail(GRANITE_CUDA_NULL_POINTER, "static decode: args is null");
    const GraniteCudaPagedDecodeArgs& a = *args;
    if (!a.q || !a.k_cache || !a.v_cache || !a.output || !a.block_tables)
        return fail(GRANITE_CUDA_NULL_POINTER, "static decode: null buffer");
    if (a.head_dim != kHeadDim || a.block_size != kPageTokens)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "static decode: head_dim must be 128 and block_size 16");
    if (a.batch_size == 0) return GRANITE_CUDA_SUCCESS;
    if (a.batch_size > (uint32_t)kStaticMaxBatch)
        return fail(GRANITE_CUDA_BUFFER_TOO_SMALL, "static decode: batch_size " + std::to_string(a.batch_size) +
                    " exceeds the fixed scratch (max " + std::to_string(kStaticMaxBatch) + " sequences per call)");
    if (a.num_heads > (uint32_t)kStaticMaxHeads)
        return fail(GRANITE_CUDA_BUFFER_TOO_SMALL, "static decode: num_heads " + std::to_string(a.num_heads) +
                    " exceeds the fixed scratch (max " + std::to_string(kStaticMaxHeads) + " query heads)");
    if (a.num_kv_heads == 0 || a.num_heads == 0 || a.num_heads % a.num_kv_heads != 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "static decode: num_heads must be a multiple of num_kv_heads");
    if (a.num_blocks == 0 || a.max_blocks_per_seq == 0)
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "static decode: empty pool or table");
    const int hkv = (int)a.num_kv_heads;
    int tile_heads;
    if (hkv == 1 || hkv == 2 || hkv == 4) tile_heads = hkv;
    else if (hkv % 8 == 0) tile_heads = 8;
    else return fail(GRANITE_CUDA_INVALID_ARGUMENT, "static decode: num_kv_heads must be 1, 2, 4 or a multiple of 8");
    const int group = (int)(a.num_heads / a.num_kv_heads);

    int device = 0;
    GB_CUDA_TRY(cudaGetDevice(&device));
    StaticDeviceSetup* setup = nullptr;
    int rc = static_decode_setup(device, &setup);
    if (rc) return rc;
    if (setup->sm_count > kStaticMaxCtas)
        return fail(GRANITE_CUDA_BUFFER_TOO_SMALL, "static decode: device has more SMs than the fixed scratch covers");
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    DecodeParams p{};
    size_t smem_bytes = 0;
    if (!plan_decode_tile(p, tile_heads, group, kHeadDim, setup->smem_optin, &smem_bytes))
        return fail(GRANITE_CUDA_INVALID_ARGUMENT, "static decode: more than 16 query heads per consumer warp");
    p.q = a.q;
    p.tables = a.block_tables;
    p.seq_lens = a.seq_lens;
    p.out = a.output;
    p.batch = (int)a.batch_size;
    p.num_heads = (int)a.num_heads;
    p.num_kv_heads = hkv;
    p.group = group;
    p.max_blocks = (int)a.max_blocks_per_seq;
    p.num_blocks = (int)a.num_blocks;
    p.uniform_len = (int)a.seq_len;
    p.n_head_tiles = hkv / tile_heads;
    p.n_ctas = setup->sm_count;
    p.contiguous = 0;
    p.max_seq = 0;
    p.scale_log2 = a.scale * 1.4426950408889634f;

    unsigned char* ws = setup->scratch;
    p.page_prefix = reinterpret_cast<int*>(ws + kStaticOffPrefix);
    p.cta_first_seq = reinterpret_cast<int*>(ws + kStaticOffFirst);
    p.part_ml = reinterpret_cast<float2*>(ws + kStaticOffMl);
    p.part_o = reinterpret_cast<float*>(ws + kStaticOffO);
    p.pages_done = reinterpret_cast<int*>(ws + kStaticOffDone);
    p.fused_merge = fused_merge_pays(p.batch, p.n_head_tiles, p.n_ctas);
    p.d = kHeadDim;
    if (device_status) {
        p.status = device_status;  // the caller owns and clears it
    } else {
        // the array keeps the previous call's contents: the status word must start at zero
        p.status = reinterpret_cast<int*>(ws + kStaticOffStatus);
        GB_CUDA_TRY(cudaMemsetAsync(p.status, 0, sizeof(int), st));
    }
    // prefix sums, first-sequence table and partials are fully rewritten before they are read

    CUtensorMap kmap, vmap;
    const uint64_t rows = (uint64_t)a.num_blocks * kPageTokens;
    if ((rc = encode_pool_map(&kmap, a.k_cache, hkv, rows, tile_heads)) != 0) return rc;
    if ((rc = encode_pool_map(&vmap, a.v_cache, hkv, rows, tile_heads)) != 0) return rc;

    // The dynamic shared-memory limit is set on every call (it allocates nothing): another entry
    // point, or another library object sharing these kernels, may have set a different one since.
    auto kern = p.page_split > 1 ? (p.heads_per_warp <= 8 ? paged_decode_kernel<1, 128, true> : paged_decode_kernel<2, 128, true>)
                                 : (p.heads_per_warp <= 8 ? paged_decode_kernel<1, 128, false> : paged_decode_kernel<2, 128, false>);
    GB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, setup->smem_optin));
    decode_plan_kernel<<<1, 1024, 0, st>>>(p);
    kern<<<p.n_ctas, kDecodeThreads, smem_bytes, st>>>(kmap, vmap, p);
    if (!p.fused_merge) decode_merge_kernel<<<dim3(p.batch, p.num_heads), kMergeThreads, 0, st>>>(p);
    GB_CUDA_TRY(cudaGetLastError());
    return GRANITE_CUDA_SUCCESS;
}
