/*
 * granite_cuda.h - C ABI of the B200 (sm_100a) attention backend for Granite.
 *
 * This is the drop-in boundary: a CUDA compute class / backend / operator inside Granite binds
 * exactly these entry points (the integration notes shipped beside this header show the binding a maintainer adds).  Plain
 * pointers and sizes only; no C++ or torch types cross it.
 *
 * Conventions (following the reference):
 *   - every function returns an int equal to a granite::ErrorCode value
 *     (include/granite/error.h:16-57); 0 is Success;
 *   - work is enqueued asynchronously on the compute object's single in-order stream; only
 *     granite_cuda_sync() blocks (include/granite/metal_compute.h:36-40,
 *     src/backend/metal/metal_compute.mm:2721-2745 for the one-object-one-queue model);
 *   - device-side problems (a wait that ran out, a block-table entry outside the pool) never
 *     trap: kernels clamp, raise a status word and return; granite_cuda_sync() reports it;
 *   - there is no CPU fallback: on a machine without a usable GPU every compute call fails
 *     with GRANITE_CUDA_BACKEND_NOT_INITIALIZED.
 */
#ifndef GRANITE_CUDA_H
#define GRANITE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Values of granite::ErrorCode (include/granite/error.h:16-57), by position. */
enum {
    GRANITE_CUDA_SUCCESS = 0,
    GRANITE_CUDA_OUT_OF_MEMORY = 4,
    GRANITE_CUDA_ALLOCATION_FAILED = 5,
    GRANITE_CUDA_BUFFER_TOO_SMALL = 6,
    GRANITE_CUDA_BACKEND_NOT_SUPPORTED = 7,
    GRANITE_CUDA_BACKEND_NOT_INITIALIZED = 8,
    GRANITE_CUDA_OPERATOR_NOT_IMPLEMENTED = 9,
    GRANITE_CUDA_EXECUTION_FAILED = 11,
    GRANITE_CUDA_TIMEOUT = 12,
    GRANITE_CUDA_INVALID_SHAPE = 13,
    GRANITE_CUDA_INVALID_ARGUMENT = 16,
    GRANITE_CUDA_NULL_POINTER = 17,
    GRANITE_CUDA_INVALID_STATE = 20,
    GRANITE_CUDA_INTERNAL_ERROR = 24,
    GRANITE_CUDA_NOT_IMPLEMENTED = 25
};

/* Opaque compute object: one device, one stream, cached tensor maps and scratch memory.
 * Replaces the MetalCompute singleton (include/granite/metal_compute.h:20-66); one per GPU. */
typedef struct granite_cuda_compute granite_cuda_compute_t;

/* Message of the last failing call on this thread (never NULL). */
const char* granite_cuda_last_error_message(void);

/* Number of visible CUDA devices (0 when there is no driver/GPU). */
int granite_cuda_device_count(void);

/* MetalCompute::initialize (metal_compute.h:30).  `stream` may be NULL (the object creates its
 * own non-blocking stream) or an existing cudaStream_t to enqueue on; to name the default
 * stream pass cudaStreamLegacy or cudaStreamPerThread, since its plain handle is NULL. */
int granite_cuda_compute_create(int device, void* stream, granite_cuda_compute_t** out);
/* MetalCompute::shutdown (metal_compute.h:31). */
void granite_cuda_compute_destroy(granite_cuda_compute_t* c);
/* The cudaStream_t the object enqueues on. */
void* granite_cuda_compute_stream(granite_cuda_compute_t* c);
/* Number of SMs of the object's device. */
int granite_cuda_compute_sm_count(granite_cuda_compute_t* c);
/* MetalCompute::sync (metal_compute.h:36): blocks until the stream drains, then maps the device
 * status word to Timeout / InvalidArgument / ExecutionFailed and clears it. */
int granite_cuda_sync(granite_cuda_compute_t* c);
/* MetalCompute::get_profiling_stats (metal_compute.h:48-52): kernels launched and syncs so far. */
void granite_cuda_get_profiling_stats(granite_cuda_compute_t* c, uint64_t* dispatches,
                                      uint64_t* syncs);

/* MetalCompute::enable_kernel_timing / reset_kernel_timing / get_kernel_timing_stats
 * (metal_compute.h:54-60): when enabled every kernel launch is bracketed by CUDA events on the
 * object's stream; the getter drains the stream and returns one row per kernel name (the number
 * of rows available; at most `capacity` are written). */
typedef struct {
    char name[64];
    double gpu_time_ms;
    uint64_t dispatches;
} GraniteCudaKernelTiming;
void granite_cuda_enable_kernel_timing(granite_cuda_compute_t* c, int enable);
void granite_cuda_reset_kernel_timing(granite_cuda_compute_t* c);
int granite_cuda_get_kernel_timing_stats(granite_cuda_compute_t* c, GraniteCudaKernelTiming* out,
                                         int capacity);

/* ---- raw buffers: MetalCompute::create_buffer (metal_compute.h:944) and the
 * IComputeBackend buffer calls (include/granite/backend.h:62-115) ------------------------- */
int granite_cuda_malloc(granite_cuda_compute_t* c, size_t bytes, void** dev_ptr);
int granite_cuda_free(granite_cuda_compute_t* c, void* dev_ptr);
int granite_cuda_malloc_host(size_t bytes, void** host_ptr); /* pinned */
int granite_cuda_free_host(void* host_ptr);
/* Asynchronous on the object's stream; pair with granite_cuda_sync(). */
int granite_cuda_write_buffer(granite_cuda_compute_t* c, void* dev_dst, const void* host_src,
                              size_t bytes);
int granite_cuda_read_buffer(granite_cuda_compute_t* c, void* host_dst, const void* dev_src,
                             size_t bytes);
int granite_cuda_copy_buffer(granite_cuda_compute_t* c, void* dev_dst, const void* dev_src,
                             size_t bytes);
int granite_cuda_memset(granite_cuda_compute_t* c, void* dev_dst, int byte, size_t bytes);

/* ---- paged decode attention ---------------------------------------------------------------
 * MetalCompute::batched_paged_attention_decode (metal_compute.h:906-920,
 * metal_compute.mm:2658-2696) and, with batch_size 1 and seq_lens NULL,
 * MetalCompute::paged_attention_decode (metal_compute.h:869-881, metal_compute.mm:2535-2621).
 * Addressing rule (metal_compute.h:853-861): token pos of a sequence lives at pool row
 * block_table[pos / block_size] * block_size + pos % block_size.
 * Tuned kernel: head_dim 128 or 64, block_size 16, any num_kv_heads (tiles of 8, 4, 2 or 1 heads); other
 * head dims (multiples of 8 up to 256) and page sizes run on a plain fp32 kernel;
 * num_heads % num_kv_heads != 0 or a head_dim outside that range returns InvalidArgument as the
 * reference does for an unsupported head_dim (metal_compute.mm:2556-2559).  A sequence of length 0
 * gets a zero row. */
typedef struct {
    const float* q;              /* [batch, num_heads, head_dim] fp32, device */
    const void* k_cache;         /* [num_blocks*block_size, num_kv_heads, head_dim] fp16, device */
    const void* v_cache;         /* same layout */
    const int32_t* block_tables; /* [batch, max_blocks_per_seq] int32, device */
    const int32_t* seq_lens;     /* [batch] int32, device; NULL: every sequence has seq_len */
    float* output;               /* [batch, num_heads, head_dim] fp32, device */
    uint32_t batch_size;
    uint32_t num_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t block_size;
    uint32_t max_blocks_per_seq;
    uint32_t num_blocks; /* capacity of the pool in blocks (the MTL::Buffer length upstream) */
    uint32_t seq_len;    /* used only when seq_lens is NULL */
    float scale;
} GraniteCudaPagedDecodeArgs;

int granite_cuda_batched_paged_attention_decode(granite_cuda_compute_t* c,
                                                const GraniteCudaPagedDecodeArgs* args);

/* The same decode with the gather that follows it on several GPUs fused in: when sequences are
 * sharded across GPUs, every rank needs all output rows.  Each final row (sequence b, all heads) is
 * stored by the attention kernel itself to args->output and to dst_ptrs[r] + (dst_row_offset + b) rows,
 * r < n_dst (<= 16) - buffers [total sequences, num_heads, head_dim] fp32 that may live on other GPUs
 * (peer-mapped, e.g. symmetric memory), on this one, or in pinned host memory (the rows then reach the host
 * while the kernel runs, without a device-to-host copy behind it).  Plain stores over NVLink from the kernel that
 * produced the row: no extra launch, no multicast, no waiting on another GPU.  Ordering towards a
 * reader on another GPU is the caller's (stream completion plus its own signal between ranks).
 * No reference counterpart (the reference runs on one GPU). */
int granite_cuda_batched_paged_attention_decode_gather(granite_cuda_compute_t* c,
                                                       const GraniteCudaPagedDecodeArgs* args,
                                                       void* const* dst_ptrs, uint32_t n_dst,
                                                       uint64_t dst_row_offset);

/* The fused gather for KV-head sharding.  When every GPU holds ALL sequences but only a slice of the KV
 * heads (pool shard [num_blocks * block_size, num_kv_heads / ranks, head_dim], block tables replicated -
 * they index tokens, not heads), args describes the local slice (num_heads and num_kv_heads are the
 * local counts) and a destination row holds dst_num_heads query heads, of which this call writes heads
 * [dst_head_offset, dst_head_offset + args->num_heads): element (b, h, d) goes to
 * dst + (((dst_row_offset + b) * dst_num_heads + dst_head_offset + h) * head_dim + d).
 * dst_num_heads == 0 means args->num_heads (the by-sequence form above).  Needs the shapes of the
 * tuned decode kernel (head_dim 128 or 64, 16-token pages).
 * No reference counterpart; the addressing rule inside the pool shard is the reference's
 * (include/granite/metal_compute.h:853-861) with the local head count. */
int granite_cuda_batched_paged_attention_decode_gather_heads(granite_cuda_compute_t* c,
                                                             const GraniteCudaPagedDecodeArgs* args,
                                                             void* const* dst_ptrs, uint32_t n_dst,
                                                             uint64_t dst_row_offset, uint32_t dst_num_heads,
                                                             uint32_t dst_head_offset);

/* Allocation-free batched paged decode.  This entry point has no counterpart in the reference.
 * It exists for hosts that cannot let a plug-in allocate device memory: a serving process whose
 * own arena already owns the GPU's memory, or a latency-critical loop that cannot afford the
 * device-wide synchronisation hidden in cudaMalloc/cudaFree.  Same arguments, layouts and results
 * as granite_cuda_batched_paged_attention_decode, but it needs no compute object and
 * calls no cudaMalloc, cudaFree or other allocating routine: its scratch (prefix sums and the
 * partials of sequences split across SMs) is a fixed ~13.8 MB array that every GPU which loads
 * this library holds until the process exits.
 *   - Shapes: narrower than the regular entry point, which falls back to other kernels.  Here
 *     head_dim must be 128, block_size 16, num_kv_heads 1, 2, 4 or a multiple of 8, and at most
 *     16 query heads may share one consumer warp (num_heads / num_kv_heads <= 16 when there are
 *     eight or more KV heads); anything else returns GRANITE_CUDA_INVALID_ARGUMENT.
 *   - Limits: batch_size <= 4096, num_heads <= 64, at most 192 SMs; beyond them the call returns
 *     GRANITE_CUDA_BUFFER_TOO_SMALL and launches nothing.
 *   - Runs on the CURRENT device, on `stream` (a cudaStream_t; NULL is the default stream),
 *     asynchronously.
 *   - The first call on each device also does a one-time set-up (it resolves the array's device
 *     address and reads the device's limits), so make that first call before any stream capture
 *     begins.
 *   - All calls share the one array and it keeps the previous call's contents; the call clears
 *     the only part that must start at zero.  Two calls that overlap on the same GPU (different
 *     streams, or different threads) race on it: serialise them.
 *   - device_status: optional device int32 that receives the status bits (2 = block-table entry
 *     outside the pool, 4 = bad sequence length, 1 = a bounded wait ran out); the caller zeroes
 *     and reads it.  NULL: the bits go to a word inside the array and are not reported. */
int granite_cuda_batched_paged_attention_decode_static(const GraniteCudaPagedDecodeArgs* args,
                                                       void* stream, int32_t* device_status);

/* ---- contiguous-cache attention -------------------------------------------------------------
 * MetalCompute::multihead_attention (metal_compute.h:804-816, metal_compute.mm:2253-2378).
 * seq_q == 1: decode. q/out [num_heads, head_dim] fp32; k/v [num_kv_heads, max_seq, head_dim]
 *             fp16 of which the first seq_kv rows per head are live.
 * seq_q  > 1: causal prefill (metal_compute.mm:2333-2375). q/out [seq_q, num_heads, head_dim];
 *             k/v [num_kv_heads, max_seq, head_dim] fp16, keys [0, seq_kv) live.
 *             q_dtype / out_dtype: 0 = fp32 (the reference's layout), 1 = fp16.  fp32 Q reaches
 *             the tensor cores as an fp16 hi + lo pair, so nothing of it is rounded away;
 *             accumulation is fp32.
 * max_seq == 0 means seq_kv, as in the reference (metal_compute.mm:2260).
 * batch_size > 1 (beyond the reference, which handles one sequence per call): a leading batch
 * dimension on every buffer - q/out [batch, seq_q, num_heads, head_dim] (decode: [batch, num_heads,
 * head_dim]), k/v [batch, num_kv_heads, max_seq, head_dim] - with the same seq_q, seq_kv and
 * start_pos for every sequence. */
typedef struct {
    const void* q;
    const void* k;
    const void* v;
    void* output;
    uint32_t num_heads;
    uint32_t num_kv_heads;
    uint32_t seq_q;
    uint32_t seq_kv;
    uint32_t head_dim;
    uint32_t max_seq;
    uint32_t q_dtype;   /* 0 fp32, 1 fp16 (prefill only) */
    uint32_t out_dtype; /* 0 fp32, 1 fp16 (prefill only) */
    float scale;
    uint32_t start_pos; /* prefill only: query i sits at position start_pos + i and sees keys
                           <= that position (chunked prefill, src/llm/transformer.mm:3682-3692);
                           the reference wrapper passes 0 */
    uint32_t batch_size; /* 0 or 1: one sequence */
} GraniteCudaAttentionArgs;

int granite_cuda_multihead_attention(granite_cuda_compute_t* c,
                                     const GraniteCudaAttentionArgs* args);

/* ---- operator-level attention -----------------------------------------------------------------
 * The computation behind OpType::ScaledDotProductAttention (include/granite/operators.h:71):
 * out = softmax(scale * Q K^T) V for one head, any head_dim; q/out [seq_q, head_dim],
 * v [seq_kv, head_dim].  k_transposed = 1: k is [head_dim, seq_kv] (the Vulkan operator,
 * src/operators/vulkan/vulkan_operators.cpp:345-434); 0: k is [seq_kv, head_dim].  causal = 1
 * limits row i to keys < i + start_pos + 1 (the Metal operator,
 * src/operators/metal/metal_operators.mm:619-690).  dtype 0 = fp32, 1 = fp16 (all four buffers). */
typedef struct {
    const void* q;
    const void* k;
    const void* v;
    void* output;
    uint32_t seq_q;
    uint32_t seq_kv;
    uint32_t head_dim;
    uint32_t dtype;
    uint32_t k_transposed;
    uint32_t causal;
    uint32_t start_pos;
    float scale;
} GraniteCudaSdpaArgs;

int granite_cuda_sdpa(granite_cuda_compute_t* c, const GraniteCudaSdpaArgs* args);

/* ---- K/V cache writes ---------------------------------------------------------------------------
 * MetalCompute::kv_cache_append (metal_compute.h:787-797; kernel kv_cache_append_f16,
 * metal_shaders_attention.h:102-132): new_k/new_v [new_len, num_kv_heads, head_dim] fp32 are
 * written at rows [current_len, current_len + new_len) of cache_k/cache_v
 * [num_kv_heads, max_seq_len, head_dim] fp16.  Overflow is InvalidArgument as in
 * KVCache::append (src/llm/kv_cache.cpp:60-64).
 * fp32 -> fp16 follows Granite's CPU path bit for bit (truncation, src/llm/math_ops.cpp:45-54). */
typedef struct {
    void* cache_k;
    void* cache_v;
    const void* new_k;
    const void* new_v;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t current_len;
    uint32_t new_len;
    uint32_t max_seq_len;
} GraniteCudaKvAppendArgs;

int granite_cuda_kv_cache_append(granite_cuda_compute_t* c, const GraniteCudaKvAppendArgs* args);

/* MetalCompute::paged_kv_cache_append (metal_compute.h:887-898; kernel
 * metal_shaders_attention.h:2142-2176): new_k/new_v [num_kv_heads, new_len, head_dim] fp32 go to
 * positions [start_pos, start_pos + new_len) of one sequence through block_table
 * [table_len] int32.  With `positions` non-NULL it is the batched decode-step form instead:
 * new_k/new_v [batch_size, num_kv_heads, head_dim], token b goes to position positions[b] of
 * sequence b through row b of block_table [batch_size, table_len]. */
typedef struct {
    const void* new_k;
    const void* new_v;
    void* k_cache;               /* pool [num_blocks*block_size, num_kv_heads, head_dim] fp16 */
    void* v_cache;
    const int32_t* block_table;  /* device */
    const int32_t* positions;    /* device [batch_size] or NULL */
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t start_pos;
    uint32_t new_len;
    uint32_t block_size;
    uint32_t num_blocks;
    uint32_t table_len;          /* entries per block-table row */
    uint32_t batch_size;         /* used only with positions */
} GraniteCudaPagedKvAppendArgs;

int granite_cuda_paged_kv_cache_append(granite_cuda_compute_t* c, const GraniteCudaPagedKvAppendArgs* args);

/* ---- tree attention for speculative-decoding verification -----------------------------------
 * MetalCompute::attention_tree (metal_compute.h:830-844, metal_compute.mm:2463-2529): every tree
 * node attends to the whole committed prefix and, among the tree nodes, to itself and its
 * ancestors (mask rule of src/llm/transformer.mm:823-840; parents must lie in [-1, num_nodes),
 * :806-813 - a parent outside that range is treated as "no parent" and reported by sync as
 * InvalidArgument).  With batch_size 1, block_tables NULL, cache_lens NULL and cache_stride 0
 * the layouts are exactly the reference's:
 *   q, output      [num_heads, num_nodes, head_dim] fp32
 *   k_cache/v_cache [num_kv_heads, cache_len, head_dim] fp16 (row stride cache_len)
 *   k_tree/v_tree  [num_kv_heads, num_nodes, head_dim] fp16, parent_indices [num_nodes] int32
 * Extensions for the batched configurations: a leading batch dimension on every buffer,
 * per-sequence prefix lengths (cache_lens, device), a contiguous cache whose row stride exceeds
 * the live length (cache_stride), and a prefix that lives in the paged pool (block_tables
 * non-NULL: k_cache/v_cache are then the pools [num_blocks*block_size, num_kv_heads, head_dim]).
 * q_dtype 1 takes fp16 queries (no hi/lo split needed).  num_nodes <= 64 (the reference caps the
 * tree at 64 nodes, src/llm/speculative_runner.cpp:579); head_dim 128; block_size 16. */
typedef struct {
    const void* q;                 /* [batch, num_heads, num_nodes, head_dim] fp32 (or fp16) */
    const void* k_cache;           /* may be NULL when there is no prefix */
    const void* v_cache;
    const void* k_tree;            /* [batch, num_kv_heads, num_nodes, head_dim] fp16 */
    const void* v_tree;
    const int32_t* parent_indices; /* [batch, num_nodes] int32, device */
    const int32_t* block_tables;   /* [batch, max_blocks_per_seq] or NULL (contiguous cache) */
    const int32_t* cache_lens;     /* [batch] int32, device, or NULL (use cache_len) */
    float* output;                 /* [batch, num_heads, num_nodes, head_dim] fp32 */
    uint32_t batch_size;
    uint32_t num_heads;
    uint32_t num_kv_heads;
    uint32_t num_nodes;
    uint32_t cache_len;
    uint32_t head_dim;
    uint32_t cache_stride;         /* contiguous cache: rows per (sequence, KV head); 0 = cache_len */
    uint32_t block_size;
    uint32_t max_blocks_per_seq;
    uint32_t num_blocks;
    uint32_t q_dtype;              /* 0 fp32, 1 fp16 */
    float scale;
} GraniteCudaTreeAttentionArgs;

int granite_cuda_attention_tree(granite_cuda_compute_t* c, const GraniteCudaTreeAttentionArgs* args);

/* The ancestor mask on its own (src/llm/transformer.mm:823-840): masks[b*num_nodes + i] gets a
 * 64-bit word whose bit j is set when node i of sequence b may attend to tree node j. */
int granite_cuda_build_tree_mask(granite_cuda_compute_t* c, const int32_t* parent_indices,
                                 uint64_t* masks, uint32_t batch_size, uint32_t num_nodes);

/* ---- RoPE and the fused RoPE + paged cache write ---------------------------------------------
 * The step immediately before attention (src/llm/transformer.mm:2975-2986: rope_multihead, then
 * paged_kv_cache_append, then the attention kernel).  The rotation follows the CPU path the
 * results are checked against: RoPECache (src/llm/rope.cpp:5-92) - cos/sin tables
 * [table_len, head_dim/2] built once on the host with the reference's own float formula,
 * adjacent pairs (2i, 2i+1), both products rounded separately - so rotated values are
 * bit-identical to Granite's CPU arithmetic.  (MetalCompute::rope_multihead,
 * include/granite/metal_compute.h:730-739, recomputes cos/sin per element on the device instead;
 * it takes freq_base where these calls take the tables.) */

/* Builds the tables on the host (rope.cpp:5-22) and uploads them; the two device arrays are
 * released with granite_cuda_free. */
int granite_cuda_rope_table_create(granite_cuda_compute_t* c, uint32_t max_seq_len, uint32_t head_dim,
                                   float theta, float** cos_table, float** sin_table);

/* MetalCompute::rope_multihead: q [seq_len, num_heads_q, head_dim] and k [seq_len, num_heads_k,
 * head_dim] fp32, rotated in place for positions start_pos .. start_pos + seq_len - 1
 * (kernel indexing of metal_shaders_util.h:596-635).  k may be NULL. */
int granite_cuda_rope_multihead(granite_cuda_compute_t* c, float* q, float* k, uint32_t num_heads_q,
                                uint32_t num_heads_k, uint32_t seq_len, uint32_t head_dim,
                                uint32_t start_pos, const float* cos_table, const float* sin_table,
                                uint32_t table_len);

/* One launch for rope_multihead + paged_kv_cache_append of a batch of sequences: q is rotated in
 * place; k is rotated, narrowed with the truncating cast (src/llm/math_ops.cpp:45-54) and
 * stored, v is narrowed and stored, at positions positions[b] .. positions[b] + new_len - 1 of
 * sequence b through row b of block_tables (addressing rule metal_compute.h:853-861).  k and v
 * are not modified.  A position outside the RoPE table or the block table, or a table entry
 * outside the pool, skips that token and is reported by granite_cuda_sync as InvalidArgument. */
typedef struct {
    float* q;                    /* [batch_size, new_len, num_heads, head_dim] fp32 or NULL */
    const float* k;              /* [batch_size, new_len, num_kv_heads, head_dim] fp32 */
    const float* v;
    const float* cos_table;      /* [table_len, head_dim/2] */
    const float* sin_table;
    void* k_cache;               /* pool [num_blocks*block_size, num_kv_heads, head_dim] fp16 */
    void* v_cache;
    const int32_t* block_tables; /* device [batch_size, max_blocks_per_seq] */
    const int32_t* positions;    /* device [batch_size] first new position per sequence; NULL: start_pos */
    uint32_t batch_size;
    uint32_t new_len;
    uint32_t num_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t block_size;
    uint32_t max_blocks_per_seq;
    uint32_t num_blocks;
    uint32_t table_len;
    uint32_t start_pos;
} GraniteCudaRopeAppendArgs;

int granite_cuda_rope_paged_kv_cache_append(granite_cuda_compute_t* c, const GraniteCudaRopeAppendArgs* args);

/* ---- tree commit ---------------------------------------------------------------------------------
 * After verification the accepted path's K/V rows are kept instead of being recomputed: row
 * accepted[b][j] of the tree K/V of sequence b is copied to position cache_lens[b] + j of its
 * paged cache, j < num_accepted[b]; the host then truncates the sequence to that length
 * (the reference truncates the contiguous cache after verification,
 * src/llm/speculative_runner.cpp:871-882).  Pure byte moves: bit-exact. */
typedef struct {
    const void* k_tree;          /* [batch_size, num_kv_heads, num_nodes, head_dim] fp16 */
    const void* v_tree;
    void* k_cache;               /* pool */
    void* v_cache;
    const int32_t* block_tables; /* device [batch_size, max_blocks_per_seq] */
    const int32_t* cache_lens;   /* device [batch_size] committed length before the tree */
    const int32_t* accepted;     /* device [batch_size, max_accepted] node indices, root first */
    const int32_t* num_accepted; /* device [batch_size] */
    uint32_t batch_size;
    uint32_t num_nodes;
    uint32_t max_accepted;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t block_size;
    uint32_t max_blocks_per_seq;
    uint32_t num_blocks;
} GraniteCudaTreeCommitArgs;

int granite_cuda_tree_commit(granite_cuda_compute_t* c, const GraniteCudaTreeCommitArgs* args);

/* ---- chunked prefill over the paged cache --------------------------------------------------------
 * Causal attention of a chunk of seq_q new tokens at positions start_pos .. start_pos + seq_q - 1
 * against the sequence's paged cache, which already holds those tokens' K/V (the start_pos =
 * chunk_start form of forward_prefill_raw, src/llm/transformer.mm:3467-3476, :3682-3692, with
 * K/V read through the block table instead of a contiguous cache).  Same arithmetic and
 * dtypes as granite_cuda_multihead_attention's prefill. */
typedef struct {
    const void* q;               /* [seq_q, num_heads, head_dim] */
    const void* k_cache;         /* pool [num_blocks*block_size, num_kv_heads, head_dim] fp16 */
    const void* v_cache;
    const int32_t* block_table;  /* device [max_blocks_per_seq] of this sequence */
    void* output;                /* [seq_q, num_heads, head_dim] */
    uint32_t num_heads;
    uint32_t num_kv_heads;
    uint32_t seq_q;
    uint32_t start_pos;
    uint32_t head_dim;           /* 128 */
    uint32_t block_size;         /* 16 */
    uint32_t max_blocks_per_seq;
    uint32_t num_blocks;
    uint32_t q_dtype;            /* 0 fp32, 1 fp16 */
    uint32_t out_dtype;
    float scale;
} GraniteCudaPagedPrefillArgs;

int granite_cuda_paged_prefill_attention(granite_cuda_compute_t* c, const GraniteCudaPagedPrefillArgs* args);

/* ---- output gather over NVLink peer memory ---------------------------------------------------------
 * Sequences are sharded across GPUs with no exchange inside attention; what follows the path is a
 * gather of the per-GPU output rows.  This call pushes `bytes` bytes from `src` (this GPU) to
 * dst_ptrs[r] + dst_offset_bytes for every r < n_dst with plain 16-byte stores - the destinations are
 * peer-mapped buffers of the other GPUs of the box (symmetric memory, CUDA IPC or cuMemMap; one of
 * them may be local).  No collective library, no multicast, nothing waits on another GPU: ordering
 * towards a consumer on the destination GPU is the caller's (an event, a flag, a barrier).
 * stream NULL = the compute object's stream; any other stream lets the push overlap the next step.
 * src, every destination and bytes must be 16-byte aligned; n_dst <= 16.  No reference counterpart
 * (the reference runs on one GPU). */
int granite_cuda_push_rows(granite_cuda_compute_t* c, void* stream, const void* src, void* const* dst_ptrs,
                           uint32_t n_dst, uint64_t dst_offset_bytes, uint64_t bytes);

/* ---- self-test of the bounded device waits -------------------------------------------------------
 * Every wait inside the kernels (on an mbarrier fed by TMA, by the tensor pipe or by another role)
 * gives up after a cycle limit, raises the status word and releases the other roles through an
 * abort flag, so that a lost signal ends as an error code and never as a hung GPU.  This call runs
 * that mechanism on purpose: one thread waits on a barrier nothing arrives at and expires after
 * limit_cycles (<= 2e8, about 0.1 s); a second waiter must leave early through the abort flag
 * (*released_early, device int, is set to 1).  The next granite_cuda_sync returns Timeout and clears
 * the status; the compute object stays usable.  No reference counterpart. */
int granite_cuda_selftest_bounded_wait(granite_cuda_compute_t* c, uint64_t limit_cycles, int32_t* released_early);

#ifdef __cplusplus
}
#endif
#endif /* GRANITE_CUDA_H */
