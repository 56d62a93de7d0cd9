// Internal state behind the opaque granite_cuda_compute_t handle: device, stream, the device
// status word, cached TMA tensor maps and the scratch arena that the split-KV decode and the
// tensor-core kernels carve their partials from.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <string>
#include <tuple>
#include <vector>

#include "../../include/granite_cuda.h"

namespace gb200 {

// Bits of the device status word.
enum : int {
    kStatusTimeout = 1,      // a bounded device-side wait ran out
    kStatusBadTable = 2,     // a block-table entry outside [0, num_blocks)
    kStatusBadSeqLen = 4,    // a sequence length outside [0, max_blocks*block_size]
    kStatusBadParent = 8,    // a tree parent index outside [-1, num_nodes)
    kStatusLayout = 16,      // a kernel found its shared-memory window smaller than its layout
};

// The status word and, 256 bytes behind it, the arrival counters of the one-launch decode (one per (sequence,
// KV head) pair) share one small allocation.
constexpr int kMaxDirectPairs = 192;
constexpr size_t kStatusBlockBytes = 256 + kMaxDirectPairs * sizeof(unsigned);

void set_error(const std::string& msg);
int fail(int code, const std::string& msg);

#define GB_CUDA_TRY(expr)                                                                  \
    do {                                                                                   \
        cudaError_t _e = (expr);                                                           \
        if (_e != cudaSuccess)                                                             \
            return ::gb200::fail(_e == cudaErrorMemoryAllocation ? GRANITE_CUDA_OUT_OF_MEMORY \
                                                                 : GRANITE_CUDA_EXECUTION_FAILED, \
                                 std::string(#expr) + ": " + cudaGetErrorString(_e));      \
    } while (0)

struct TensorMapKey {
    const void* base;
    uint64_t dim0, dim1, dim2;
    uint64_t stride1, stride2;
    uint32_t box0, box1, box2;
    int swizzle;
    int rank;
    uint64_t dim3 = 0, stride3 = 0;  // rank 4 only
    uint32_t box3 = 0;
    bool operator<(const TensorMapKey& o) const {
        return std::tie(base, dim0, dim1, dim2, dim3, stride1, stride2, stride3, box0, box1, box2, box3, swizzle, rank) <
               std::tie(o.base, o.dim0, o.dim1, o.dim2, o.dim3, o.stride1, o.stride2, o.stride3, o.box0, o.box1,
                        o.box2, o.box3, o.swizzle, o.rank);
    }
};

}  // namespace gb200

struct granite_cuda_compute {
    int device = 0;
    int sm_count = 0;
    int smem_optin = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int* d_status = nullptr;  // device status word
    int* d_pages_done = nullptr;        // page counters of the decode without a plan kernel: zero between launches
    size_t pages_done_count = 0;
    int ensure_page_counters(size_t count);
    unsigned* d_direct_done = nullptr;  // arrival counters of the one-launch decode (same allocation, 256 bytes further)
    int* h_status = nullptr;  // pinned mirror
    uint64_t dispatches = 0;
    uint64_t syncs = 0;
    // scratch arena (grown on demand, never shrunk)
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    // Cached TMA descriptors, keyed by (buffer, shape).  Bounded: once kMaxTensorMaps entries exist,
    // everything but the kKeepRecent most recently used ones is dropped (encode_map), so a pointer
    // returned by encode_map stays valid for at least the next kKeepRecent - 1 calls to it.
    struct CachedTensorMap { CUtensorMap map; uint64_t last_use; };
    static constexpr size_t kMaxTensorMaps = 256;
    static constexpr uint64_t kKeepRecent = 32;
    std::map<gb200::TensorMapKey, CachedTensorMap> tensor_maps;
    uint64_t tensor_map_tick = 0;

    // per-kernel GPU timing (MetalCompute::enable_kernel_timing, metal_compute.h:54-60)
    struct TimedLaunch { const char* name; cudaEvent_t begin, end; };
    struct KernelStat { double ms = 0.0; uint64_t dispatches = 0; };
    bool kernel_timing = false;
    std::vector<TimedLaunch> pending_timings;
    std::vector<cudaEvent_t> event_pool;
    std::map<std::string, KernelStat> kernel_stats;
    cudaEvent_t take_event();
    void resolve_timings();  // call only after the stream has drained

    int ensure_scratch(size_t bytes);
    // fp16 tensor maps; returns nullptr (and sets the error message) on failure.
    const CUtensorMap* tensor_map_2d(const void* base, uint64_t dim0, uint64_t dim1,
                                     uint64_t stride1_bytes, uint32_t box0, uint32_t box1,
                                     int swizzle_bytes);
    const CUtensorMap* tensor_map_3d(const void* base, uint64_t dim0, uint64_t dim1, uint64_t dim2,
                                     uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t box0,
                                     uint32_t box1, uint32_t box2, int swizzle_bytes);
    // One K (or V) page of a tile of KV heads as a single box: dims {64 halfs, rows, 64-wide chunks
    // of a head, heads}, box {64, 16 rows, all chunks, tile_heads}; lands in shared memory as
    // [head][chunk][row][64] under the 128-byte swizzle.
    const CUtensorMap* tensor_map_pages(const void* base, uint32_t head_dim, uint64_t rows, uint64_t row_stride_bytes,
                                        uint64_t heads, uint64_t head_stride_bytes, uint32_t rows_per_box,
                                        uint32_t tile_heads);
    // The pool [rows, width halfs] (width = Hkv * head_dim) seen in groups of 8 rows: dims {width,
    // 8 rows, 64-wide chunks of a head, rows / 8}, box {64, 8, all chunks, 2} = one 16-row page of one
    // head, landing as [row group][chunk][8 rows][64]; x selects the head (x = head * head_dim).
    const CUtensorMap* tensor_map_page_groups(const void* base, uint64_t width, uint64_t rows, uint32_t head_dim);
    const CUtensorMap* encode_map(const gb200::TensorMapKey& key);
};

namespace gb200 {
// Brackets one kernel launch with events when kernel timing is on; counts the dispatch always.
struct LaunchScope {
    granite_cuda_compute* c;
    cudaEvent_t end = nullptr;
    LaunchScope(granite_cuda_compute* c_, const char* name) : c(c_) {
        c->dispatches++;
        if (c->kernel_timing) {
            cudaEvent_t b = c->take_event();
            end = c->take_event();
            cudaEventRecord(b, c->stream);
            c->pending_timings.push_back({name, b, end});
        }
    }
    ~LaunchScope() {
        if (end) cudaEventRecord(end, c->stream);
    }
};
// Optional gather of the decode output: every final row also goes to dst[r] (row row_offset + sequence).
struct DecodeGather {
    void* const* dst;
    uint32_t n_dst;
    uint64_t row_offset;
    uint32_t dst_heads = 0;    // query heads per destination row; 0: this call's num_heads
    uint32_t head_offset = 0;  // first destination head of this call's heads
};
int launch_paged_decode(granite_cuda_compute* c, const GraniteCudaPagedDecodeArgs& a, bool contiguous,
                        uint32_t max_seq, const DecodeGather* gather = nullptr);
int launch_prefill(granite_cuda_compute* c, const GraniteCudaAttentionArgs& a);
int launch_tree_verify(granite_cuda_compute* c, const GraniteCudaTreeAttentionArgs& a);
int launch_kv_cache_append(granite_cuda_compute* c, const GraniteCudaKvAppendArgs& a);
int launch_paged_kv_cache_append(granite_cuda_compute* c, const GraniteCudaPagedKvAppendArgs& a);
int launch_sdpa_operator(granite_cuda_compute* c, const GraniteCudaSdpaArgs& a);
int launch_tree_mask(granite_cuda_compute* c, const int32_t* parents, uint64_t* masks, uint32_t batch, uint32_t n);
int launch_rope_multihead(granite_cuda_compute* c, float* q, float* k, uint32_t hq, uint32_t hk, uint32_t seq_len,
                          uint32_t head_dim, uint32_t start_pos, const float* cos_t, const float* sin_t, uint32_t table_len);
int launch_rope_paged_append(granite_cuda_compute* c, const GraniteCudaRopeAppendArgs& a);
int launch_tree_commit(granite_cuda_compute* c, const GraniteCudaTreeCommitArgs& a);
int launch_paged_prefill(granite_cuda_compute* c, const GraniteCudaPagedPrefillArgs& a);
// plain fp32 kernel for head dims, page sizes and head counts outside the tuned kernels' shapes
int launch_generic_decode(granite_cuda_compute* c, const GraniteCudaPagedDecodeArgs& a, bool contiguous, uint32_t max_seq);
int launch_generic_prefill(granite_cuda_compute* c, const GraniteCudaAttentionArgs& a);
int launch_generic_paged_prefill(granite_cuda_compute* c, const GraniteCudaPagedPrefillArgs& a);
int launch_generic_tree(granite_cuda_compute* c, const GraniteCudaTreeAttentionArgs& a);
int launch_bounded_wait_selftest(granite_cuda_compute* c, uint64_t limit_cycles, int* released_early_dev);
int launch_push_rows(granite_cuda_compute* c, cudaStream_t stream, const void* src, void* const* dst_ptrs, uint32_t n_dst,
                     uint64_t dst_offset_bytes, uint64_t bytes);
}  // namespace gb200
