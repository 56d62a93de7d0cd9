// C++ host faces above the C ABI (include/granite_cuda.h), shaped like the Granite interfaces
// they plug into, so that they can be dropped into Granite's tree next to its Metal and Vulkan
// backends.  Only the parts of the vocabulary that the attention path touches are restated here
// (in Granite itself these come from include/granite/{error,types,backend,tensor,operators,llm}.h).
//
//   CudaBackend      : IComputeBackend                 (include/granite/backend.h:30-183)
//   CudaAttentionOp  : IOperator, register_cuda_operators()
//                                                      (include/granite/operators.h:196-291)
//   CudaCompute      : attention group of MetalCompute (include/granite/metal_compute.h:749-920)
//   BlockManager / PagedKVCache / PagedKVPool / KVCache with their pages in HBM
//                                                      (include/granite/llm.h:117-167, 888-1035)
//   SpeculationTree                                    (include/granite/llm.h:293-356)
// Every device operation goes through the extern "C" entry points; nothing here launches a
// kernel or touches the CUDA runtime directly, and nothing falls back to the CPU.
#pragma once
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <unordered_map>
#include <utility>
#include <variant>
#include <vector>

#include "../../../include/granite_cuda.h"

// Built inside Granite's tree (or against its headers: -DGRANITE_WITH_REFERENCE_HEADERS with
// include/ of the checkout on the include path) the vocabulary below IS Granite's: every class
// of this file then derives from the real interfaces with `override`, Tensor / Error /
// OperatorRegistry are Granite's own objects, and only the enumerator for this backend is missing
// upstream (a maintainer adds `CUDA` to BackendType, include/granite/types.h:93-98; until then the
// next free value is used).  Built alone, the restatement below stands in for those headers.
#ifdef GRANITE_WITH_REFERENCE_HEADERS
#include "granite/backend.h"
#include "granite/error.h"
#include "granite/operators.h"
#include "granite/tensor.h"
#include "granite/types.h"
namespace granite {
inline constexpr BackendType kCudaBackendType = static_cast<BackendType>(static_cast<uint8_t>(BackendType::Talos) + 1);
}
#else
namespace granite {

// ------------------------------------------------------------------ errors (error.h:16-226)
enum class ErrorCode {
    Success = 0, FileNotFound, InvalidFormat, IOError, OutOfMemory, AllocationFailed, BufferTooSmall,
    BackendNotSupported, BackendNotInitialized, OperatorNotImplemented, ShaderCompilationFailed,
    ExecutionFailed, Timeout, InvalidShape, ShapeMismatch, DTypeMismatch, InvalidArgument, NullPointer,
    InvalidGraph, CycleDetected, InvalidState, UnsupportedModel, CorruptedWeights, MissingOperator,
    InternalError, NotImplemented,
};

class Error {
public:
    Error(ErrorCode code, std::string message) : code_(code), message_(std::move(message)) {}
    ErrorCode code() const { return code_; }
    const std::string& message() const { return message_; }
private:
    ErrorCode code_;
    std::string message_;
};

template <typename T>
class Result {
public:
    Result(T value) : v_(std::move(value)) {}
    Result(Error error) : v_(std::move(error)) {}
    bool ok() const { return std::holds_alternative<T>(v_); }
    T& value() { return std::get<T>(v_); }
    const T& value() const { return std::get<T>(v_); }
    T take() && { return std::move(std::get<T>(v_)); }
    const Error& error() const { return std::get<Error>(v_); }
private:
    std::variant<T, Error> v_;
};

template <>
class Result<void> {
public:
    Result() = default;
    Result(Error error) : e_(std::make_shared<Error>(std::move(error))) {}
    bool ok() const { return !e_; }
    const Error& error() const { return *e_; }
private:
    std::shared_ptr<Error> e_;
};

// ------------------------------------------------------------------ types (types.h:20-169)
enum class DataType : uint8_t { FP32, FP16, INT32, INT64, UINT8 };
constexpr size_t dtype_size(DataType t) {
    return t == DataType::FP32 || t == DataType::INT32 ? 4 : t == DataType::FP16 ? 2 : t == DataType::INT64 ? 8 : 1;
}
enum class BackendType : uint8_t { CPU, Metal, Vulkan, Talos, CUDA };
constexpr const char* backend_name(BackendType t) {
    switch (t) {
        case BackendType::CPU: return "CPU";
        case BackendType::Metal: return "Metal";
        case BackendType::Vulkan: return "Vulkan";
        case BackendType::Talos: return "Talos";
        case BackendType::CUDA: return "CUDA";
    }
    return "unknown";
}
struct BufferHandle { uint64_t id = 0; bool valid() const { return id != 0; } };
struct PipelineHandle { uint64_t id = 0; bool valid() const { return id != 0; } };
struct FenceHandle { uint64_t id = 0; bool valid() const { return id != 0; } };
enum class MemoryType : uint8_t { Device, Shared, Managed };
struct BufferDesc {
    size_t size = 0;
    MemoryType memory_type = MemoryType::Device;
    bool allow_aliasing = false;
    static BufferDesc device(size_t n) { return {n, MemoryType::Device, false}; }
    static BufferDesc shared(size_t n) { return {n, MemoryType::Shared, false}; }
    static BufferDesc managed(size_t n) { return {n, MemoryType::Managed, false}; }
};
struct DeviceCapabilities {
    const char* name = nullptr;
    size_t max_buffer_size = 0, max_threadgroup_size = 0, shared_memory_size = 0;
    uint32_t simd_width = 0;
    bool supports_fp16 = false, supports_bf16 = false, supports_int8 = false, supports_int4 = false,
         supports_simd_groups = false;
};
struct PipelineDesc {
    std::string shader_source, entry_point = "main";
    uint32_t threadgroup_size_x = 0, threadgroup_size_y = 0, threadgroup_size_z = 0;
};

// ------------------------------------------------------------------ backend (backend.h:30-183)
class IComputeBackend {
public:
    virtual ~IComputeBackend() = default;
    virtual Result<void> initialize() = 0;
    virtual void shutdown() = 0;
    virtual bool is_initialized() const = 0;
    virtual DeviceCapabilities get_capabilities() const = 0;
    virtual BackendType get_type() const = 0;
    virtual Result<BufferHandle> create_buffer(const BufferDesc& desc) = 0;
    virtual Result<BufferHandle> create_buffer_from_host(const void* data, const BufferDesc& desc);
    virtual void destroy_buffer(BufferHandle handle) = 0;
    virtual Result<void*> map_buffer(BufferHandle handle) = 0;
    virtual void unmap_buffer(BufferHandle handle) = 0;
    virtual Result<void> write_buffer(BufferHandle handle, const void* data, size_t size, size_t offset = 0) = 0;
    virtual Result<void> read_buffer(BufferHandle handle, void* data, size_t size, size_t offset = 0) = 0;
    virtual Result<void> copy_buffer(BufferHandle src, BufferHandle dst, size_t size, size_t src_offset = 0,
                                     size_t dst_offset = 0) = 0;
    virtual void* get_native_buffer(BufferHandle) { return nullptr; }
    virtual void* get_native_device() { return nullptr; }
    virtual void* get_native_queue() { return nullptr; }
    virtual Result<PipelineHandle> create_pipeline(const PipelineDesc& desc) = 0;
    virtual void destroy_pipeline(PipelineHandle handle) = 0;
    virtual Result<void> begin_commands() = 0;
    virtual Result<void> bind_pipeline(PipelineHandle pipeline) = 0;
    virtual Result<void> bind_buffer(uint32_t index, BufferHandle buffer, size_t offset = 0) = 0;
    virtual Result<void> set_push_constants(const void* data, size_t size) = 0;
    virtual Result<void> dispatch(uint32_t groups_x, uint32_t groups_y = 1, uint32_t groups_z = 1) = 0;
    virtual Result<void> end_commands() = 0;
    virtual Result<void> submit() = 0;
    virtual Result<void> wait_for_completion() = 0;
    virtual Result<FenceHandle> create_fence() = 0;
    virtual Result<void> wait_fence(FenceHandle fence, uint64_t timeout_ns = UINT64_MAX) = 0;
    virtual void destroy_fence(FenceHandle fence) = 0;
};

// ------------------------------------------------------------------ tensor (tensor.h:19-178)
// Non-owning view: the buffer lives until destroy_buffer or backend shutdown.
class Tensor {
public:
    Tensor() = default;
    static Result<Tensor> allocate(const std::vector<int64_t>& shape, DataType dtype, IComputeBackend* backend);
    static Tensor from_buffer(BufferHandle buffer, const std::vector<int64_t>& shape, DataType dtype,
                              IComputeBackend* backend);
    const std::vector<int64_t>& shape() const { return shape_; }
    DataType dtype() const { return dtype_; }
    size_t ndim() const { return shape_.size(); }
    int64_t size(int dim) const { return shape_[dim < 0 ? shape_.size() + dim : dim]; }
    size_t numel() const;
    size_t size_bytes() const { return numel() * dtype_size(dtype_); }
    bool valid() const { return buffer_.valid(); }
    BufferHandle buffer() const { return buffer_; }
    IComputeBackend* backend() const { return backend_; }
private:
    BufferHandle buffer_;
    std::vector<int64_t> shape_;
    DataType dtype_ = DataType::FP32;
    IComputeBackend* backend_ = nullptr;
};

// ------------------------------------------------------------------ operators (operators.h:140-291)
enum class OpType : uint32_t { ScaledDotProductAttention = 35, MultiHeadAttention = 36 };
using AttrValue = std::variant<int64_t, double, bool, std::string, std::vector<int64_t>, std::vector<double>>;
class Attributes {
public:
    void set(const std::string& key, AttrValue value) { attrs_[key] = std::move(value); }
    template <typename T>
    T get(const std::string& key, T fallback = T{}) const {
        auto it = attrs_.find(key);
        if (it == attrs_.end()) return fallback;
        if (auto* v = std::get_if<T>(&it->second)) return *v;
        return fallback;
    }
    bool has(const std::string& key) const { return attrs_.count(key) != 0; }
private:
    std::unordered_map<std::string, AttrValue> attrs_;
};
struct OpContext {
    IComputeBackend* backend = nullptr;
    std::vector<Tensor> inputs, outputs;
    Attributes attrs;
    size_t num_inputs() const { return inputs.size(); }
    size_t num_outputs() const { return outputs.size(); }
};
class IOperator {
public:
    virtual ~IOperator() = default;
    virtual OpType type() const = 0;
    virtual Result<void> validate(const OpContext& ctx) const = 0;
    virtual Result<std::vector<std::vector<int64_t>>> infer_shapes(const OpContext& ctx) const = 0;
    virtual Result<void> execute(OpContext& ctx) = 0;
};
using OperatorFactory = std::function<std::unique_ptr<IOperator>()>;
class OperatorRegistry {
public:
    static OperatorRegistry& instance();
    void register_op(OpType op, BackendType backend, OperatorFactory factory);
    // Unlike the reference (src/core/operator_registry.cpp:26-35) a miss is a miss: there is no
    // silent fallback to a CPU operator.
    std::unique_ptr<IOperator> create(OpType op, BackendType backend) const;
    bool has_implementation(OpType op, BackendType backend) const;
private:
    std::unordered_map<uint64_t, OperatorFactory> factories_;
};
inline constexpr BackendType kCudaBackendType = BackendType::CUDA;
}  // namespace granite
#endif

namespace granite {

// Error of the last failing C-ABI call, as a Granite error value.
Error cuda_error(int code);
inline Result<void> cuda_result(int code) {
    if (code == 0) return {};
    return cuda_error(code);
}

// Factory, wired like the out-of-tree Talos backend (src/core/backend_factory.cpp:29-31,62-68).
std::unique_ptr<IComputeBackend> create_cuda_backend(int device = 0);

void register_cuda_operators();

// ------------------------------------------------------------------ compute class
// One per GPU (the reference's get_metal_compute() singleton becomes per device).
class CudaCompute {
public:
    CudaCompute() = default;
    ~CudaCompute();
    CudaCompute(const CudaCompute&) = delete;
    CudaCompute& operator=(const CudaCompute&) = delete;
    Result<void> initialize(int device, void* stream = nullptr);
    void shutdown();
    void sync();
    Result<void> sync_checked();
    void commit() {}
    bool is_initialized() const { return h_ != nullptr; }
    granite_cuda_compute_t* handle() const { return h_; }
    void get_profiling_stats(uint64_t& dispatches, uint64_t& syncs) const;
    void enable_kernel_timing(bool enable);

    void* create_buffer(size_t size);
    void destroy_buffer(void* ptr);
    std::pair<void*, void*> create_kv_cache(uint32_t num_kv_heads, uint32_t max_seq_len, uint32_t head_dim);

    Result<void> kv_cache_append(void* cache_k, void* cache_v, const void* new_k, const void* new_v,
                                 uint32_t num_kv_heads, uint32_t head_dim, uint32_t current_len, uint32_t new_len,
                                 uint32_t max_seq_len);
    Result<void> multihead_attention(const void* Q, const void* K, const void* V, void* output, uint32_t num_heads,
                                     uint32_t num_kv_heads, uint32_t seq_q, uint32_t seq_kv, uint32_t head_dim,
                                     float scale, uint32_t max_seq = 0);
    Result<void> attention_tree(const void* Q, const void* K_cache, const void* V_cache, const void* K_tree,
                                const void* V_tree, const int32_t* parent_indices, float* output,
                                uint32_t num_heads, uint32_t num_kv_heads, uint32_t num_nodes, uint32_t cache_len,
                                uint32_t head_dim, float scale);
    Result<void> paged_attention_decode(const float* Q, const void* K_cache, const void* V_cache,
                                        const int32_t* block_table, float* output, uint32_t num_heads,
                                        uint32_t num_kv_heads, uint32_t seq_len, uint32_t head_dim,
                                        uint32_t block_size, float scale, uint32_t num_blocks);
    Result<void> paged_kv_cache_append(const void* new_k, const void* new_v, void* K_cache, void* V_cache,
                                       const int32_t* block_table, uint32_t num_kv_heads, uint32_t head_dim,
                                       uint32_t start_pos, uint32_t new_len, uint32_t block_size,
                                       uint32_t num_blocks, uint32_t table_len);
    Result<void> batched_paged_attention_decode(const float* Q, const void* K_cache, const void* V_cache,
                                                const int32_t* block_tables, const int32_t* seq_lens,
                                                float* output, uint32_t batch_size, uint32_t num_heads,
                                                uint32_t num_kv_heads, uint32_t head_dim, uint32_t block_size,
                                                uint32_t max_blocks_per_seq, float scale, uint32_t num_blocks);
    // Several GPUs, sequences sharded: the same decode, whose kernels also store every final row into the
    // ranks' gathered buffers (gather_dst[r], n_dst <= 16, row gather_row_offset + sequence).  No counterpart
    // upstream (one GPU).
    Result<void> batched_paged_attention_decode_gather(const GraniteCudaPagedDecodeArgs& args, void* const* gather_dst,
                                                       uint32_t n_dst, uint64_t gather_row_offset);
    // Several GPUs, KV heads sharded (every rank holds all sequences, num_kv_heads / ranks heads): args describes
    // the local head slice; a destination row holds dst_num_heads query heads, this call's start at dst_head_offset.
    Result<void> batched_paged_attention_decode_gather_heads(const GraniteCudaPagedDecodeArgs& args, void* const* gather_dst,
                                                             uint32_t n_dst, uint64_t gather_row_offset,
                                                             uint32_t dst_num_heads, uint32_t dst_head_offset);
    // The step before attention and the ones after verification (the "next" tier of the path):
    // RoPE with host-built tables, RoPE fused with the paged cache write, the tree commit copy and
    // chunked prefill over the paged cache.  Argument meaning as in granite_cuda.h.
    Result<void> rope_multihead(float* q, float* k, uint32_t num_heads_q, uint32_t num_heads_k, uint32_t seq_len,
                                uint32_t head_dim, uint32_t start_pos, const float* cos_table, const float* sin_table,
                                uint32_t table_len);
    Result<void> rope_paged_kv_cache_append(const GraniteCudaRopeAppendArgs& args);
    Result<void> tree_commit(const GraniteCudaTreeCommitArgs& args);
    Result<void> paged_prefill_attention(const GraniteCudaPagedPrefillArgs& args);
private:
    granite_cuda_compute_t* h_ = nullptr;
};
CudaCompute* get_cuda_compute(int device = 0);

// ------------------------------------------------------------------ RoPE tables (llm.h:173-197)
class RoPECache {
public:
    RoPECache() = default;
    ~RoPECache();
    RoPECache(const RoPECache&) = delete;
    RoPECache& operator=(const RoPECache&) = delete;
    // cos/sin [max_seq_len, head_dim/2] on the host, in the reference's float arithmetic (src/llm/rope.cpp:5-22)
    void initialize(int max_seq_len, int head_dim, float theta = 10000.0f);
    // q [batch, seq_len, num_heads, head_dim], k [batch, seq_len, num_kv_heads, head_dim] fp32 device
    // tensors of the CUDA backend, rotated in place (src/llm/rope.cpp:24-92; batch 1 as there)
    Result<void> apply(Tensor& q, Tensor& k, int start_pos, IComputeBackend* backend);
    const std::vector<float>& cos_cache() const { return cos_; }
    const std::vector<float>& sin_cache() const { return sin_; }
    bool is_initialized() const { return !cos_.empty(); }
    int max_seq_len() const { return max_seq_len_; }
    int head_dim() const { return head_dim_; }
    // device copies of the tables, uploaded on first use through `compute`
    Result<void> upload(granite_cuda_compute_t* compute);
    const float* device_cos() const { return d_cos_; }
    const float* device_sin() const { return d_sin_; }
private:
    std::vector<float> cos_, sin_;
    int max_seq_len_ = 0, head_dim_ = 0;
    float *d_cos_ = nullptr, *d_sin_ = nullptr;
    granite_cuda_compute_t* owner_ = nullptr;
};

// ------------------------------------------------------------------ KV caches (llm.h:117-167, 888-1035)
struct ModelConfig {
    int num_layers = 0, num_heads = 0, num_kv_heads = 0, head_dim = 0;
};

class KVCache {
public:
    static Result<KVCache> allocate(const ModelConfig& config, int max_seq_len, IComputeBackend* backend);
    // keys/values: [1, num_kv_heads, new_len, head_dim] fp16 device tensors
    Result<void> append(int layer, const Tensor& keys, const Tensor& values);
    std::pair<Tensor, Tensor> get(int layer) const;
    int seq_len() const { return current_len_; }
    int max_seq_len() const { return max_seq_len_; }
    void clear() { current_len_ = 0; }
    void increment_seq_len(int delta = 1) { current_len_ += delta; }
    void set_seq_len(int len) { current_len_ = len; }
    void truncate(int new_len) { if (new_len >= 0 && new_len < current_len_) current_len_ = new_len; }
    size_t memory_bytes() const;
    bool is_allocated() const { return !layers_.empty(); }
private:
    struct LayerCache { Tensor keys, values; };
    std::vector<LayerCache> layers_;
    int max_seq_len_ = 0, current_len_ = 0, num_kv_heads_ = 0, head_dim_ = 0;
    IComputeBackend* backend_ = nullptr;
};

struct PagedKVConfig {
    int block_size = 16, num_blocks = 256, num_layers = 0, num_kv_heads = 0, head_dim = 0;
};

class BlockManager {
public:
    Result<void> initialize(const PagedKVConfig& config, IComputeBackend* backend);
    int allocate_block();
    void free_block(int block_idx);
    int num_free_blocks() const { return num_free_; }
    int num_total_blocks() const { return num_blocks_; }
    int block_size() const { return block_size_; }
    Tensor& k_cache(int layer) { return k_blocks_[layer]; }
    Tensor& v_cache(int layer) { return v_blocks_[layer]; }
    bool is_initialized() const { return initialized_; }
    const PagedKVConfig& config() const { return config_; }
    // diagnostics: the reference only logs these (src/llm/paged_kv_cache.cpp:84-98)
    int rejected_frees() const { return rejected_frees_; }
private:
    PagedKVConfig config_;
    int num_blocks_ = 0, block_size_ = 0, num_free_ = 0, rejected_frees_ = 0;
    bool initialized_ = false;
    std::vector<int> free_list_;
    std::vector<bool> block_allocated_;
    std::vector<Tensor> k_blocks_, v_blocks_;
    IComputeBackend* backend_ = nullptr;
};

class PagedKVCache {
public:
    PagedKVCache() = default;
    explicit PagedKVCache(BlockManager* bm) : block_manager_(bm) {}
    void release();
    bool append_tokens(int num_tokens);
    int seq_len() const { return seq_len_; }
    int num_blocks() const { return static_cast<int>(block_table_.size()); }
    const std::vector<int>& block_table() const { return block_table_; }
    int get_physical_block(int token_pos) const;
    int get_block_offset(int token_pos) const;
    void clear() { release(); }
    void truncate(int new_len);
    BlockManager* block_manager() { return block_manager_; }
private:
    BlockManager* block_manager_ = nullptr;
    std::vector<int> block_table_;
    int seq_len_ = 0;
};

class PagedKVPool {
public:
    Result<void> initialize(const ModelConfig& config, int max_sequences, int max_total_tokens, int block_size,
                            IComputeBackend* backend);
    int acquire_slot();
    void release_slot(int slot);
    PagedKVCache& get_cache(int slot) { return caches_[slot]; }
    BlockManager& block_manager() { return block_manager_; }
    int num_free_slots() const;
    int num_free_blocks() const { return block_manager_.num_free_blocks(); }
    int num_slots() const { return static_cast<int>(caches_.size()); }
    bool is_initialized() const { return block_manager_.is_initialized(); }
    // Mirrors the tables of `slots` to the device as [n, max_blocks] int32 (-1 padded) plus
    // [n] lengths: the batched form of TransformerModel::sync_block_table_to_gpu
    // (src/llm/transformer.mm:2798-2816).  Asynchronous on the compute object's stream.
    Result<void> sync_block_tables_to_gpu(CudaCompute* compute, const std::vector<int>& slots,
                                          int32_t* d_tables, int max_blocks, int32_t* d_seq_lens);
private:
    BlockManager block_manager_;
    std::vector<PagedKVCache> caches_;
    std::vector<bool> slot_in_use_;
    std::vector<int32_t> staging_;
};

// ------------------------------------------------------------------ speculation tree (llm.h:293-356)
class SpeculationTree {
public:
    struct Node {
        int32_t token;
        int parent_idx;
        int depth;
        float log_prob;
        std::vector<int> children;
    };
    int add_node(int32_t token, int parent_idx, float log_prob = 0.0f);
    std::vector<int> get_leaves() const;
    std::vector<int> get_path(int node_idx) const;
    std::vector<int> get_parent_indices() const;
    std::vector<int32_t> flatten_tokens() const;
    size_t size() const { return nodes_.size(); }
    const Node& node(int idx) const { return nodes_[idx]; }
    const Node* get_node(int idx) const {
        return idx < 0 || idx >= static_cast<int>(nodes_.size()) ? nullptr : &nodes_[idx];
    }
    int max_depth() const;
    void clear() { nodes_.clear(); }
    std::vector<int32_t> find_accepted_path(const std::vector<int32_t>& target_choices) const;
    // The node indices behind find_accepted_path's tokens, root first (the target's own closing
    // token has no node): what the tree commit copies into the cache.
    std::vector<int> find_accepted_nodes(const std::vector<int32_t>& target_choices) const;
private:
    std::vector<Node> nodes_;
};

// ------------------------------------------------------------------ batched paged decode step
// One decode step for every active request in one set of launches: what
// BatchScheduler::process_batch_paged (src/llm/batch_scheduler.cpp:391-452) leaves as a TODO after
// it has grown each request's PagedKVCache by one token.  Block tables, lengths and positions of
// the batch live on the device; a step copies the two length arrays and only the table rows that
// gained a block.
class PagedDecodeBatch {
public:
    ~PagedDecodeBatch();
    Result<void> initialize(PagedKVPool* pool, CudaCompute* compute, RoPECache* rope, const ModelConfig& config,
                            int max_batch, int max_blocks_per_seq);
    // rows of the batch are kept dense; returns the row, or -1 when full / already present
    int add_request(int slot);
    void remove_request(int slot);
    int batch_size() const { return static_cast<int>(slots_.size()); }
    const std::vector<int>& slots() const { return slots_; }
    // Grows every active sequence by one token (PagedKVCache::append_tokens(1)) and brings the
    // device arrays up to date.  Slots whose allocation failed are removed from the batch and
    // returned (the reference marks such a request FAILED, batch_scheduler.cpp:431-435).
    Result<std::vector<int>> begin_step();
    // One layer of the step: q [B, Hq, D] (rotated in place), k, v [B, Hkv, D] fp32 -> the new
    // token's K/V into `layer`'s pools, attention output [B, Hq, D] fp32.  Asynchronous.
    Result<void> attend(int layer, float* q, const float* k, const float* v, float* out, float scale);
    const int32_t* device_tables() const { return d_tables_; }
    const int32_t* device_seq_lens() const { return d_lens_; }
private:
    PagedKVPool* pool_ = nullptr;
    CudaCompute* compute_ = nullptr;
    RoPECache* rope_ = nullptr;
    ModelConfig config_;
    int max_batch_ = 0, max_blocks_ = 0;
    std::vector<int> slots_;            // row -> slot
    // row -> the table entries the device row holds.  A step re-sends from the first entry that
    // differs from the sequence's current table, so a table that shrank (truncate after a tree
    // commit, or a slot released and taken again) and regrew over other blocks is never left stale.
    std::vector<std::vector<int32_t>> sent_rows_;
    int32_t *d_tables_ = nullptr, *d_lens_ = nullptr, *d_positions_ = nullptr;
    int32_t* h_staging_ = nullptr;      // pinned: [max_batch] positions, [max_batch] lengths, [max_batch, max_blocks] rows
};

}  // namespace granite
