// Implementation of the C++ host faces declared in granite_host.h.  Everything here talks to the
// device through the extern "C" entry points of include/granite_cuda.h only.
#include "granite_host.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <mutex>
#include <queue>

namespace granite {

Error cuda_error(int code) {
    return Error(static_cast<ErrorCode>(code), granite_cuda_last_error_message());
}

#ifndef GRANITE_WITH_REFERENCE_HEADERS  // upstream, backend.h provides this default inline
Result<BufferHandle> IComputeBackend::create_buffer_from_host(const void* data, const BufferDesc& desc) {
    if (!data) return Error(ErrorCode::InvalidArgument, "Null host buffer");
    auto b = create_buffer(desc);
    if (!b.ok()) return b.error();
    auto w = write_buffer(b.value(), data, desc.size);
    if (!w.ok()) {
        destroy_buffer(b.value());
        return w.error();
    }
    return b;
}
#endif

// =================================================================== CudaCompute
CudaCompute::~CudaCompute() { shutdown(); }

Result<void> CudaCompute::initialize(int device, void* stream) {
    if (h_) return {};
    return cuda_result(granite_cuda_compute_create(device, stream, &h_));
}
void CudaCompute::shutdown() {
    if (h_) granite_cuda_compute_destroy(h_);
    h_ = nullptr;
}
void CudaCompute::sync() { (void)granite_cuda_sync(h_); }
Result<void> CudaCompute::sync_checked() { return cuda_result(granite_cuda_sync(h_)); }
void CudaCompute::get_profiling_stats(uint64_t& dispatches, uint64_t& syncs) const {
    granite_cuda_get_profiling_stats(h_, &dispatches, &syncs);
}
void CudaCompute::enable_kernel_timing(bool enable) { granite_cuda_enable_kernel_timing(h_, enable ? 1 : 0); }

void* CudaCompute::create_buffer(size_t size) {
    void* p = nullptr;
    return granite_cuda_malloc(h_, size, &p) == 0 ? p : nullptr;
}
void CudaCompute::destroy_buffer(void* ptr) { (void)granite_cuda_free(h_, ptr); }

std::pair<void*, void*> CudaCompute::create_kv_cache(uint32_t num_kv_heads, uint32_t max_seq_len, uint32_t head_dim) {
    // [num_kv_heads, max_seq_len, head_dim] fp16, zeroed (metal_compute.h:771-776)
    const size_t bytes = static_cast<size_t>(num_kv_heads) * max_seq_len * head_dim * 2;
    void* k = create_buffer(bytes);
    void* v = create_buffer(bytes);
    if (!k || !v) {
        destroy_buffer(k);
        destroy_buffer(v);
        return {nullptr, nullptr};
    }
    granite_cuda_memset(h_, k, 0, bytes);
    granite_cuda_memset(h_, v, 0, bytes);
    return {k, v};
}

Result<void> CudaCompute::kv_cache_append(void* cache_k, void* cache_v, const void* new_k, const void* new_v,
                                          uint32_t num_kv_heads, uint32_t head_dim, uint32_t current_len,
                                          uint32_t new_len, uint32_t max_seq_len) {
    GraniteCudaKvAppendArgs a{cache_k, cache_v, new_k, new_v, num_kv_heads, head_dim, current_len, new_len, max_seq_len};
    return cuda_result(granite_cuda_kv_cache_append(h_, &a));
}

Result<void> CudaCompute::multihead_attention(const void* Q, const void* K, const void* V, void* output,
                                              uint32_t num_heads, uint32_t num_kv_heads, uint32_t seq_q,
                                              uint32_t seq_kv, uint32_t head_dim, float scale, uint32_t max_seq) {
    GraniteCudaAttentionArgs a{Q, K, V, output, num_heads, num_kv_heads, seq_q, seq_kv, head_dim, max_seq, 0, 0, scale, 0};
    return cuda_result(granite_cuda_multihead_attention(h_, &a));
}

Result<void> CudaCompute::attention_tree(const void* Q, const void* K_cache, const void* V_cache, const void* K_tree,
                                         const void* V_tree, const int32_t* parent_indices, float* output,
                                         uint32_t num_heads, uint32_t num_kv_heads, uint32_t num_nodes,
                                         uint32_t cache_len, uint32_t head_dim, float scale) {
    GraniteCudaTreeAttentionArgs a{};
    a.q = Q; a.k_cache = K_cache; a.v_cache = V_cache; a.k_tree = K_tree; a.v_tree = V_tree;
    a.parent_indices = parent_indices; a.output = output;
    a.batch_size = 1; a.num_heads = num_heads; a.num_kv_heads = num_kv_heads; a.num_nodes = num_nodes;
    a.cache_len = cache_len; a.head_dim = head_dim; a.block_size = 16; a.scale = scale;
    return cuda_result(granite_cuda_attention_tree(h_, &a));
}

Result<void> CudaCompute::paged_attention_decode(const float* Q, const void* K_cache, const void* V_cache,
                                                 const int32_t* block_table, float* output, uint32_t num_heads,
                                                 uint32_t num_kv_heads, uint32_t seq_len, uint32_t head_dim,
                                                 uint32_t block_size, float scale, uint32_t num_blocks) {
    const uint32_t table_len = block_size ? (seq_len + block_size - 1) / block_size : 0;
    GraniteCudaPagedDecodeArgs a{Q, K_cache, V_cache, block_table, nullptr, output, 1, num_heads, num_kv_heads,
                                 head_dim, block_size, table_len ? table_len : 1, num_blocks, seq_len, scale};
    return cuda_result(granite_cuda_batched_paged_attention_decode(h_, &a));
}

Result<void> CudaCompute::paged_kv_cache_append(const void* new_k, const void* new_v, void* K_cache, void* V_cache,
                                                const int32_t* block_table, uint32_t num_kv_heads, uint32_t head_dim,
                                                uint32_t start_pos, uint32_t new_len, uint32_t block_size,
                                                uint32_t num_blocks, uint32_t table_len) {
    GraniteCudaPagedKvAppendArgs a{new_k, new_v, K_cache, V_cache, block_table, nullptr, num_kv_heads, head_dim,
                                   start_pos, new_len, block_size, num_blocks, table_len, 0};
    return cuda_result(granite_cuda_paged_kv_cache_append(h_, &a));
}

Result<void> CudaCompute::batched_paged_attention_decode(const float* Q, const void* K_cache, const void* V_cache,
                                                         const int32_t* block_tables, const int32_t* seq_lens,
                                                         float* output, uint32_t batch_size, uint32_t num_heads,
                                                         uint32_t num_kv_heads, uint32_t head_dim, uint32_t block_size,
                                                         uint32_t max_blocks_per_seq, float scale, uint32_t num_blocks) {
    GraniteCudaPagedDecodeArgs a{Q, K_cache, V_cache, block_tables, seq_lens, output, batch_size, num_heads,
                                 num_kv_heads, head_dim, block_size, max_blocks_per_seq, num_blocks, 0, scale};
    return cuda_result(granite_cuda_batched_paged_attention_decode(h_, &a));
}

Result<void> CudaCompute::batched_paged_attention_decode_gather(const GraniteCudaPagedDecodeArgs& args,
                                                                void* const* gather_dst, uint32_t n_dst,
                                                                uint64_t gather_row_offset) {
    return cuda_result(granite_cuda_batched_paged_attention_decode_gather(h_, &args, gather_dst, n_dst, gather_row_offset));
}

Result<void> CudaCompute::batched_paged_attention_decode_gather_heads(const GraniteCudaPagedDecodeArgs& args,
                                                                      void* const* gather_dst, uint32_t n_dst,
                                                                      uint64_t gather_row_offset, uint32_t dst_num_heads,
                                                                      uint32_t dst_head_offset) {
    return cuda_result(granite_cuda_batched_paged_attention_decode_gather_heads(h_, &args, gather_dst, n_dst, gather_row_offset,
                                                                                dst_num_heads, dst_head_offset));
}

Result<void> CudaCompute::rope_multihead(float* q, float* k, uint32_t num_heads_q, uint32_t num_heads_k,
                                         uint32_t seq_len, uint32_t head_dim, uint32_t start_pos,
                                         const float* cos_table, const float* sin_table, uint32_t table_len) {
    return cuda_result(granite_cuda_rope_multihead(h_, q, k, num_heads_q, num_heads_k, seq_len, head_dim, start_pos,
                                                   cos_table, sin_table, table_len));
}

Result<void> CudaCompute::rope_paged_kv_cache_append(const GraniteCudaRopeAppendArgs& args) {
    return cuda_result(granite_cuda_rope_paged_kv_cache_append(h_, &args));
}

Result<void> CudaCompute::tree_commit(const GraniteCudaTreeCommitArgs& args) {
    return cuda_result(granite_cuda_tree_commit(h_, &args));
}

Result<void> CudaCompute::paged_prefill_attention(const GraniteCudaPagedPrefillArgs& args) {
    return cuda_result(granite_cuda_paged_prefill_attention(h_, &args));
}

// =================================================================== RoPECache (src/llm/rope.cpp)
void RoPECache::initialize(int max_seq_len, int head_dim, float theta) {
    max_seq_len_ = max_seq_len;
    head_dim_ = head_dim;
    const int half_dim = head_dim / 2;
    cos_.assign(static_cast<size_t>(max_seq_len) * half_dim, 0.0f);
    sin_.assign(cos_.size(), 0.0f);
    // float arithmetic throughout, one pow per (position, pair) as the reference computes it
    // (rope.cpp:13-20): the tables are part of the bit-exact contract of the rotation
    for (int pos = 0; pos < max_seq_len; pos++)
        for (int i = 0; i < half_dim; i++) {
            const float freq = 1.0f / std::pow(theta, static_cast<float>(2 * i) / head_dim);
            const float angle = static_cast<float>(pos) * freq;
            cos_[static_cast<size_t>(pos) * half_dim + i] = std::cos(angle);
            sin_[static_cast<size_t>(pos) * half_dim + i] = std::sin(angle);
        }
    if (d_cos_ && owner_) {  // re-initialised: the device copies are stale
        granite_cuda_free(owner_, d_cos_);
        granite_cuda_free(owner_, d_sin_);
        d_cos_ = d_sin_ = nullptr;
    }
}

RoPECache::~RoPECache() {
    if (owner_ && d_cos_) {
        granite_cuda_free(owner_, d_cos_);
        granite_cuda_free(owner_, d_sin_);
    }
}

Result<void> RoPECache::upload(granite_cuda_compute_t* compute) {
    if (!is_initialized()) return Error(ErrorCode::InvalidState, "RoPE cache not initialized");
    if (d_cos_ && owner_ == compute) return {};
    if (!compute) return Error(ErrorCode::NullPointer, "RoPECache::upload: null compute object");
    void *c = nullptr, *s = nullptr;
    const size_t bytes = cos_.size() * sizeof(float);
    int rc = granite_cuda_malloc(compute, bytes, &c);
    if (!rc) rc = granite_cuda_malloc(compute, bytes, &s);
    if (!rc) rc = granite_cuda_write_buffer(compute, c, cos_.data(), bytes);
    if (!rc) rc = granite_cuda_write_buffer(compute, s, sin_.data(), bytes);
    if (!rc) rc = granite_cuda_sync(compute);
    if (rc) {
        if (c) granite_cuda_free(compute, c);
        if (s) granite_cuda_free(compute, s);
        return cuda_error(rc);
    }
    d_cos_ = static_cast<float*>(c);
    d_sin_ = static_cast<float*>(s);
    owner_ = compute;
    return {};
}

Result<void> RoPECache::apply(Tensor& q, Tensor& k, int start_pos, IComputeBackend* backend) {
    if (!is_initialized()) return Error(ErrorCode::InvalidState, "RoPE cache not initialized");
    if (!backend || backend->get_type() != kCudaBackendType)
        return Error(ErrorCode::BackendNotSupported, "RoPECache::apply needs the CUDA backend (no CPU fallback)");
    const int seq_len = static_cast<int>(q.size(1));
    const int num_heads_q = static_cast<int>(q.size(2)), num_heads_k = static_cast<int>(k.size(2));
    if (start_pos < 0 || start_pos + seq_len > max_seq_len_)
        return Error(ErrorCode::InvalidArgument, "RoPE position out of range: " + std::to_string(start_pos) + " + " +
                                                     std::to_string(seq_len) + " > " + std::to_string(max_seq_len_));
    auto* compute = static_cast<granite_cuda_compute_t*>(backend->get_native_device());
    auto up = upload(compute);
    if (!up.ok()) return up;
    int rc = granite_cuda_rope_multihead(compute, static_cast<float*>(backend->get_native_buffer(q.buffer())),
                                         static_cast<float*>(backend->get_native_buffer(k.buffer())), num_heads_q,
                                         num_heads_k, seq_len, head_dim_, start_pos, d_cos_, d_sin_, max_seq_len_);
    if (!rc) rc = granite_cuda_sync(compute);
    return cuda_result(rc);
}

CudaCompute* get_cuda_compute(int device) {
    // one lazily created object per device (the reference keeps one global MetalCompute,
    // src/backend/metal/metal_compute.mm:2721-2745)
    static std::mutex mu;
    static std::unordered_map<int, std::unique_ptr<CudaCompute>> objects;
    std::lock_guard<std::mutex> lock(mu);
    auto& slot = objects[device];
    if (!slot) {
        auto c = std::make_unique<CudaCompute>();
        if (!c->initialize(device).ok()) return nullptr;
        slot = std::move(c);
    }
    return slot.get();
}

// =================================================================== CudaBackend
namespace {

class CudaBackend final : public IComputeBackend {
public:
    explicit CudaBackend(int device) : device_(device) {}
    ~CudaBackend() override { shutdown(); }

    Result<void> initialize() override {
        if (compute_.is_initialized()) return {};
        return compute_.initialize(device_);
    }
    void shutdown() override {
        if (!compute_.is_initialized()) return;
        for (auto& kv : buffers_) release(kv.second);
        buffers_.clear();
        compute_.shutdown();
    }
    bool is_initialized() const override { return compute_.is_initialized(); }
    DeviceCapabilities get_capabilities() const override {
        DeviceCapabilities caps;
        caps.name = "NVIDIA B200 (sm_100a)";
        caps.max_buffer_size = size_t(180) << 30;
        caps.max_threadgroup_size = 1024;
        caps.shared_memory_size = 227 * 1024;
        caps.simd_width = 32;
        caps.supports_fp16 = caps.supports_bf16 = caps.supports_int8 = caps.supports_int4 = true;
        caps.supports_simd_groups = true;
        return caps;
    }
    BackendType get_type() const override { return kCudaBackendType; }

    Result<BufferHandle> create_buffer(const BufferDesc& desc) override {
        if (!is_initialized()) return Error(ErrorCode::BackendNotInitialized, "CUDA backend not initialized");
        if (desc.size == 0) return Error(ErrorCode::InvalidArgument, "Buffer size must be > 0");
        Buffer b;
        b.size = desc.size;
        b.type = desc.memory_type;
        if (desc.memory_type == MemoryType::Shared) {
            // CPU/GPU shared staging memory: pinned host memory, visible to the device
            int rc = granite_cuda_malloc_host(desc.size, &b.host);
            if (rc) return cuda_error(rc);
        } else {
            // Device and Managed both live in HBM; Managed gets a pinned shadow on first map
            int rc = granite_cuda_malloc(compute_.handle(), desc.size, &b.dev);
            if (rc) return cuda_error(rc);
        }
        BufferHandle h{next_id_++};
        buffers_[h.id] = b;
        return h;
    }
    void destroy_buffer(BufferHandle handle) override {
        auto it = buffers_.find(handle.id);
        if (it == buffers_.end()) return;
        release(it->second);
        buffers_.erase(it);
    }
    // Mapping a device-resident buffer downloads it into a pinned shadow; unmap uploads the
    // shadow again (the managed-mode didModifyRange of src/backend/metal/metal_backend.mm:247-260).
    Result<void*> map_buffer(BufferHandle handle) override {
        auto it = buffers_.find(handle.id);
        if (it == buffers_.end()) return Error(ErrorCode::InvalidArgument, "Invalid buffer handle");
        Buffer& b = it->second;
        if (b.type == MemoryType::Shared) return b.host;
        if (!b.host) {
            int rc = granite_cuda_malloc_host(b.size, &b.host);
            if (rc) return cuda_error(rc);
        }
        if (!b.mapped) {
            int rc = granite_cuda_read_buffer(compute_.handle(), b.host, b.dev, b.size);
            if (!rc) rc = granite_cuda_sync(compute_.handle());
            if (rc) return cuda_error(rc);
            b.mapped = true;
        }
        return b.host;
    }
    void unmap_buffer(BufferHandle handle) override {
        auto it = buffers_.find(handle.id);
        if (it == buffers_.end()) return;
        Buffer& b = it->second;
        if (b.type == MemoryType::Shared || !b.mapped) return;
        granite_cuda_write_buffer(compute_.handle(), b.dev, b.host, b.size);
        granite_cuda_sync(compute_.handle());
        b.mapped = false;
    }
    Result<void> write_buffer(BufferHandle handle, const void* data, size_t size, size_t offset) override {
        auto it = buffers_.find(handle.id);
        if (it == buffers_.end()) return Error(ErrorCode::InvalidArgument, "Invalid buffer handle");
        Buffer& b = it->second;
        if (offset + size > b.size) return Error(ErrorCode::BufferTooSmall, "write past the end of the buffer");
        if (b.type == MemoryType::Shared) {
            std::memcpy(static_cast<uint8_t*>(b.host) + offset, data, size);
            return {};
        }
        int rc = granite_cuda_write_buffer(compute_.handle(), static_cast<uint8_t*>(b.dev) + offset, data, size);
        if (!rc) rc = granite_cuda_sync(compute_.handle());  // `data` may be pageable and short-lived
        return cuda_result(rc);
    }
    Result<void> read_buffer(BufferHandle handle, void* data, size_t size, size_t offset) override {
        auto it = buffers_.find(handle.id);
        if (it == buffers_.end()) return Error(ErrorCode::InvalidArgument, "Invalid buffer handle");
        Buffer& b = it->second;
        if (offset + size > b.size) return Error(ErrorCode::BufferTooSmall, "read past the end of the buffer");
        if (b.type == MemoryType::Shared) {
            granite_cuda_sync(compute_.handle());
            std::memcpy(data, static_cast<uint8_t*>(b.host) + offset, size);
            return {};
        }
        int rc = granite_cuda_read_buffer(compute_.handle(), data, static_cast<uint8_t*>(b.dev) + offset, size);
        if (!rc) rc = granite_cuda_sync(compute_.handle());
        return cuda_result(rc);
    }
    Result<void> copy_buffer(BufferHandle src, BufferHandle dst, size_t size, size_t src_offset, size_t dst_offset) override {
        auto s = buffers_.find(src.id), d = buffers_.find(dst.id);
        if (s == buffers_.end() || d == buffers_.end()) return Error(ErrorCode::InvalidArgument, "Invalid buffer handle");
        if (src_offset + size > s->second.size || dst_offset + size > d->second.size)
            return Error(ErrorCode::BufferTooSmall, "copy past the end of a buffer");
        const void* sp = static_cast<uint8_t*>(native(s->second)) + src_offset;
        void* dp = static_cast<uint8_t*>(native(d->second)) + dst_offset;
        int rc;
        if (s->second.type == MemoryType::Shared && d->second.type == MemoryType::Shared) {
            std::memcpy(dp, sp, size);
            rc = 0;
        } else if (s->second.type == MemoryType::Shared) {
            rc = granite_cuda_write_buffer(compute_.handle(), dp, sp, size);
        } else if (d->second.type == MemoryType::Shared) {
            rc = granite_cuda_read_buffer(compute_.handle(), dp, sp, size);
        } else {
            rc = granite_cuda_copy_buffer(compute_.handle(), dp, sp, size);
        }
        if (!rc) rc = granite_cuda_sync(compute_.handle());
        return cuda_result(rc);
    }
    void* get_native_buffer(BufferHandle handle) override {
        auto it = buffers_.find(handle.id);
        return it == buffers_.end() ? nullptr : native(it->second);
    }
    void* get_native_device() override { return compute_.handle(); }
    void* get_native_queue() override { return granite_cuda_compute_stream(compute_.handle()); }

    // The pipeline / command-recording half of the interface is for shader back ends; like the CPU
    // backend (src/backend/cpu/cpu_backend.cpp:149-165) this one has no use for it.
    Result<PipelineHandle> create_pipeline(const PipelineDesc&) override {
        return Error(ErrorCode::NotImplemented, "CUDA backend does not compile pipelines; kernels are built in");
    }
    void destroy_pipeline(PipelineHandle) override {}
    Result<void> begin_commands() override { return {}; }
    Result<void> bind_pipeline(PipelineHandle) override { return {}; }
    Result<void> bind_buffer(uint32_t, BufferHandle, size_t) override { return {}; }
    Result<void> set_push_constants(const void*, size_t) override { return {}; }
    Result<void> dispatch(uint32_t, uint32_t, uint32_t) override {
        return Error(ErrorCode::NotImplemented, "CUDA backend has no generic dispatch; call the compute object");
    }
    Result<void> end_commands() override { return {}; }
    Result<void> submit() override { return {}; }
    Result<void> wait_for_completion() override { return compute_.sync_checked(); }
    Result<FenceHandle> create_fence() override { return FenceHandle{next_id_++}; }
    Result<void> wait_fence(FenceHandle, uint64_t) override { return compute_.sync_checked(); }
    void destroy_fence(FenceHandle) override {}

private:
    struct Buffer {
        void* dev = nullptr;
        void* host = nullptr;
        size_t size = 0;
        MemoryType type = MemoryType::Device;
        bool mapped = false;
    };
    static void* native(const Buffer& b) { return b.type == MemoryType::Shared ? b.host : b.dev; }
    void release(Buffer& b) {
        if (b.dev) granite_cuda_free(compute_.handle(), b.dev);
        if (b.host) granite_cuda_free_host(b.host);
        b.dev = b.host = nullptr;
    }
    int device_;
    CudaCompute compute_;
    uint64_t next_id_ = 1;
    std::unordered_map<uint64_t, Buffer> buffers_;
};

}  // namespace

std::unique_ptr<IComputeBackend> create_cuda_backend(int device) { return std::make_unique<CudaBackend>(device); }

#ifndef GRANITE_WITH_REFERENCE_HEADERS  // upstream: src/core/tensor.cpp and src/core/operator_registry.cpp
// =================================================================== Tensor
size_t Tensor::numel() const {
    if (shape_.empty()) return 0;
    size_t n = 1;
    for (int64_t d : shape_) n *= static_cast<size_t>(d);
    return n;
}

Result<Tensor> Tensor::allocate(const std::vector<int64_t>& shape, DataType dtype, IComputeBackend* backend) {
    if (!backend) return Error(ErrorCode::NullPointer, "Backend is null");
    if (!backend->is_initialized()) return Error(ErrorCode::BackendNotInitialized, "Backend not initialized");
    for (int64_t d : shape)
        if (d <= 0) return Error(ErrorCode::InvalidShape, "Tensor dimensions must be positive");
    Tensor t;
    t.shape_ = shape;
    t.dtype_ = dtype;
    t.backend_ = backend;
    // the reference always asks for managed memory (src/core/tensor.cpp:87)
    auto buf = backend->create_buffer(BufferDesc::managed(t.size_bytes()));
    if (!buf.ok()) return buf.error();
    t.buffer_ = buf.value();
    return t;
}

Tensor Tensor::from_buffer(BufferHandle buffer, const std::vector<int64_t>& shape, DataType dtype,
                           IComputeBackend* backend) {
    Tensor t;
    t.buffer_ = buffer;
    t.shape_ = shape;
    t.dtype_ = dtype;
    t.backend_ = backend;
    return t;
}

// =================================================================== operators
OperatorRegistry& OperatorRegistry::instance() {
    static OperatorRegistry r;
    return r;
}
static uint64_t op_key(OpType op, BackendType backend) {
    return (static_cast<uint64_t>(op) << 8) | static_cast<uint64_t>(backend);
}
void OperatorRegistry::register_op(OpType op, BackendType backend, OperatorFactory factory) {
    factories_[op_key(op, backend)] = std::move(factory);
}
std::unique_ptr<IOperator> OperatorRegistry::create(OpType op, BackendType backend) const {
    auto it = factories_.find(op_key(op, backend));
    return it == factories_.end() ? nullptr : it->second();
}
bool OperatorRegistry::has_implementation(OpType op, BackendType backend) const {
    return factories_.count(op_key(op, backend)) != 0;
}
#endif

namespace {

// OpType::ScaledDotProductAttention on the CUDA backend.  Contract of the reference operators:
// at least three inputs, output shaped like Q, attrs "scale" (double, default 1/sqrt(D)) and
// "start_pos" (int64, default 0) (src/operators/metal/metal_operators.mm:1226-1325,
// src/operators/vulkan/vulkan_operators.cpp:345-434).  fp32 inputs follow the Vulkan layout
// (K pre-transposed [D, T], no mask); fp16 inputs follow the Metal layout (K [T, D], keys limited
// to q + start_pos + 1).
class CudaAttentionOp final : public IOperator {
public:
    OpType type() const override { return OpType::ScaledDotProductAttention; }
    Result<void> validate(const OpContext& ctx) const override {
        if (ctx.num_inputs() < 3) return Error(ErrorCode::InvalidArgument, "Attention requires 3 inputs (Q, K, V)");
        return {};
    }
    Result<std::vector<std::vector<int64_t>>> infer_shapes(const OpContext& ctx) const override {
        if (ctx.num_inputs() < 1) return Error(ErrorCode::InvalidArgument, "Attention requires 3 inputs (Q, K, V)");
        const auto q_shape = ctx.inputs[0].shape();  // a vector here, a span over it upstream (tensor.h:45)
        return std::vector<std::vector<int64_t>>{std::vector<int64_t>(q_shape.begin(), q_shape.end())};
    }
    Result<void> execute(OpContext& ctx) override {
        auto ok = validate(ctx);
        if (!ok.ok()) return ok;
        if (ctx.num_outputs() < 1) return Error(ErrorCode::InvalidArgument, "Attention requires an output tensor");
        if (!ctx.backend || ctx.backend->get_type() != kCudaBackendType)
            return Error(ErrorCode::OperatorNotImplemented, "CudaAttentionOp needs the CUDA backend (no CPU fallback)");
        const Tensor &Q = ctx.inputs[0], &K = ctx.inputs[1], &V = ctx.inputs[2];
        Tensor& out = ctx.outputs[0];
        if (Q.ndim() != 2 || K.ndim() != 2 || V.ndim() != 2) return Error(ErrorCode::InvalidShape, "Attention operator takes 2-D tensors");
        if (Q.dtype() != K.dtype() || Q.dtype() != V.dtype() || Q.dtype() != out.dtype())
            return Error(ErrorCode::DTypeMismatch, "Q, K, V and output must share a dtype");
        if (Q.dtype() != DataType::FP32 && Q.dtype() != DataType::FP16)
            return Error(ErrorCode::DTypeMismatch, "Attention operator supports fp32 and fp16");
        const bool f32 = Q.dtype() == DataType::FP32;
        const uint32_t seq_q = static_cast<uint32_t>(Q.size(0)), head_dim = static_cast<uint32_t>(Q.size(1));
        const uint32_t seq_kv = static_cast<uint32_t>(V.size(0));
        const bool shapes_ok = f32 ? (K.size(0) == head_dim && K.size(1) == seq_kv) : (K.size(0) == seq_kv && K.size(1) == head_dim);
        if (!shapes_ok || V.size(1) != head_dim || out.size(0) != seq_q || out.size(1) != head_dim)
            return Error(ErrorCode::ShapeMismatch, "Attention operator: inconsistent Q/K/V/output shapes");
        GraniteCudaSdpaArgs a{};
        a.q = ctx.backend->get_native_buffer(Q.buffer());
        a.k = ctx.backend->get_native_buffer(K.buffer());
        a.v = ctx.backend->get_native_buffer(V.buffer());
        a.output = ctx.backend->get_native_buffer(out.buffer());
        a.seq_q = seq_q;
        a.seq_kv = seq_kv;
        a.head_dim = head_dim;
        a.dtype = f32 ? 0 : 1;
        a.k_transposed = f32 ? 1 : 0;
        a.causal = f32 ? 0 : 1;
        a.start_pos = static_cast<uint32_t>(ctx.attrs.get<int64_t>("start_pos", 0));
        a.scale = static_cast<float>(ctx.attrs.get<double>("scale", 1.0 / std::sqrt(static_cast<double>(head_dim))));
        auto* compute = static_cast<granite_cuda_compute_t*>(ctx.backend->get_native_device());
        int rc = granite_cuda_sdpa(compute, &a);
        if (!rc) rc = granite_cuda_sync(compute);
        return cuda_result(rc);
    }
};

}  // namespace

void register_cuda_operators() {
    OperatorRegistry::instance().register_op(OpType::ScaledDotProductAttention, kCudaBackendType,
                                             [] { return std::make_unique<CudaAttentionOp>(); });
}

// =================================================================== KVCache (src/llm/kv_cache.cpp)
Result<KVCache> KVCache::allocate(const ModelConfig& config, int max_seq_len, IComputeBackend* backend) {
    KVCache cache;
    cache.max_seq_len_ = max_seq_len;
    cache.num_kv_heads_ = config.num_kv_heads;
    cache.head_dim_ = config.head_dim;
    cache.backend_ = backend;
    const std::vector<int64_t> shape = {1, config.num_kv_heads, max_seq_len, config.head_dim};
    for (int i = 0; i < config.num_layers; i++) {
        auto k = Tensor::allocate(shape, DataType::FP16, backend);
        if (!k.ok()) return k.error();
        auto v = Tensor::allocate(shape, DataType::FP16, backend);
        if (!v.ok()) return v.error();
        cache.layers_.push_back({std::move(k).take(), std::move(v).take()});
    }
    return cache;
}

Result<void> KVCache::append(int layer, const Tensor& keys, const Tensor& values) {
    if (layer < 0 || layer >= static_cast<int>(layers_.size())) return Error(ErrorCode::InvalidArgument, "Invalid layer index");
    const int new_len = static_cast<int>(keys.size(2));
    if (current_len_ + new_len > max_seq_len_)
        return Error(ErrorCode::InvalidArgument, "KV cache overflow: " + std::to_string(current_len_) + " + " +
                                                     std::to_string(new_len) + " > " + std::to_string(max_seq_len_));
    // per head: rows [current, current + new_len) of [Hkv, max_seq, D]; device-to-device copies
    auto& lc = layers_[layer];
    const size_t row = static_cast<size_t>(head_dim_) * 2;
    for (int h = 0; h < num_kv_heads_; h++) {
        const size_t dst = (static_cast<size_t>(h) * max_seq_len_ + current_len_) * row;
        const size_t src = static_cast<size_t>(h) * new_len * row;
        auto r1 = backend_->copy_buffer(keys.buffer(), lc.keys.buffer(), new_len * row, src, dst);
        if (!r1.ok()) return r1;
        auto r2 = backend_->copy_buffer(values.buffer(), lc.values.buffer(), new_len * row, src, dst);
        if (!r2.ok()) return r2;
    }
    // the length moves only with the last layer (src/llm/kv_cache.cpp:101-104)
    if (layer == static_cast<int>(layers_.size()) - 1) current_len_ += new_len;
    return {};
}

std::pair<Tensor, Tensor> KVCache::get(int layer) const {
    if (layer < 0 || layer >= static_cast<int>(layers_.size())) return {Tensor{}, Tensor{}};
    return {layers_[layer].keys, layers_[layer].values};
}

size_t KVCache::memory_bytes() const {
    size_t total = 0;
    for (const auto& lc : layers_) total += lc.keys.size_bytes() + lc.values.size_bytes();
    return total;
}

// =================================================================== page manager (src/llm/paged_kv_cache.cpp)
Result<void> BlockManager::initialize(const PagedKVConfig& config, IComputeBackend* backend) {
    if (config.num_blocks <= 0 || config.block_size <= 0) return Error(ErrorCode::InvalidArgument, "Invalid block configuration");
    config_ = config;
    backend_ = backend;
    num_blocks_ = config.num_blocks;
    block_size_ = config.block_size;
    free_list_.resize(num_blocks_);
    block_allocated_.assign(num_blocks_, false);
    for (int i = 0; i < num_blocks_; i++) free_list_[i] = i;
    num_free_ = num_blocks_;
    rejected_frees_ = 0;
    // one K pool and one V pool per layer, [num_blocks * block_size, num_kv_heads, head_dim] fp16, in HBM
    k_blocks_.clear();
    v_blocks_.clear();
    const std::vector<int64_t> shape = {static_cast<int64_t>(num_blocks_) * block_size_, config.num_kv_heads, config.head_dim};
    for (int layer = 0; layer < config.num_layers; layer++) {
        auto k = Tensor::allocate(shape, DataType::FP16, backend);
        auto v = Tensor::allocate(shape, DataType::FP16, backend);
        if (!k.ok() || !v.ok())
            return Error(ErrorCode::AllocationFailed, "Failed to allocate paged KV blocks for layer " + std::to_string(layer));
        k_blocks_.push_back(std::move(k).take());
        v_blocks_.push_back(std::move(v).take());
    }
    initialized_ = true;
    return {};
}

int BlockManager::allocate_block() {
    if (num_free_ == 0) return -1;
    const int idx = free_list_[--num_free_];  // top of the stack: the first calls hand out the highest indices
    block_allocated_[idx] = true;
    return idx;
}

void BlockManager::free_block(int block_idx) {
    if (block_idx < 0 || block_idx >= num_blocks_ || !block_allocated_[block_idx]) {
        rejected_frees_++;  // out of range or double free: ignored, as in the reference
        return;
    }
    block_allocated_[block_idx] = false;
    free_list_[num_free_++] = block_idx;
}

void PagedKVCache::release() {
    if (!block_manager_) return;
    for (int idx : block_table_) block_manager_->free_block(idx);
    block_table_.clear();
    seq_len_ = 0;
}

bool PagedKVCache::append_tokens(int num_tokens) {
    if (!block_manager_) return false;
    const int bs = block_manager_->block_size();
    const int new_len = seq_len_ + num_tokens;
    const int needed = (new_len + bs - 1) / bs;
    int have = static_cast<int>(block_table_.size());
    while (have < needed) {
        const int blk = block_manager_->allocate_block();
        if (blk < 0) return false;  // blocks taken so far stay with the sequence; the length does not move
        block_table_.push_back(blk);
        have++;
    }
    seq_len_ = new_len;
    return true;
}

int PagedKVCache::get_physical_block(int token_pos) const {
    if (!block_manager_) return -1;
    const int logical = token_pos / block_manager_->block_size();
    if (logical >= static_cast<int>(block_table_.size())) return -1;
    return block_table_[logical];
}

int PagedKVCache::get_block_offset(int token_pos) const {
    if (!block_manager_) return 0;
    return token_pos % block_manager_->block_size();
}

void PagedKVCache::truncate(int new_len) {
    if (new_len >= seq_len_ || !block_manager_) return;
    const int bs = block_manager_->block_size();
    int needed = (new_len + bs - 1) / bs;
    if (new_len == 0) needed = 0;
    while (static_cast<int>(block_table_.size()) > needed) {
        block_manager_->free_block(block_table_.back());
        block_table_.pop_back();
    }
    seq_len_ = new_len;
}

Result<void> PagedKVPool::initialize(const ModelConfig& config, int max_sequences, int max_total_tokens,
                                     int block_size, IComputeBackend* backend) {
    PagedKVConfig pc;
    pc.block_size = block_size;
    pc.num_blocks = block_size > 0 ? (max_total_tokens + block_size - 1) / block_size : 0;
    pc.num_layers = config.num_layers;
    pc.num_kv_heads = config.num_kv_heads;
    pc.head_dim = config.head_dim;
    auto r = block_manager_.initialize(pc, backend);
    if (!r.ok()) return r;
    caches_.assign(max_sequences, PagedKVCache(&block_manager_));
    slot_in_use_.assign(max_sequences, false);
    return {};
}

int PagedKVPool::acquire_slot() {
    for (size_t i = 0; i < slot_in_use_.size(); i++) {
        if (!slot_in_use_[i]) {
            slot_in_use_[i] = true;
            caches_[i].clear();
            return static_cast<int>(i);
        }
    }
    return -1;
}

void PagedKVPool::release_slot(int slot) {
    if (slot < 0 || slot >= static_cast<int>(slot_in_use_.size())) return;
    if (slot_in_use_[slot]) {
        caches_[slot].release();
        slot_in_use_[slot] = false;
    }
}

int PagedKVPool::num_free_slots() const {
    int n = 0;
    for (bool used : slot_in_use_) n += used ? 0 : 1;
    return n;
}

Result<void> PagedKVPool::sync_block_tables_to_gpu(CudaCompute* compute, const std::vector<int>& slots,
                                                   int32_t* d_tables, int max_blocks, int32_t* d_seq_lens) {
    if (!compute || !d_tables || !d_seq_lens) return Error(ErrorCode::NullPointer, "sync_block_tables_to_gpu: null argument");
    const size_t n = slots.size();
    staging_.assign(n * max_blocks + n, -1);
    for (size_t i = 0; i < n; i++) {
        const int slot = slots[i];
        if (slot < 0 || slot >= num_slots()) return Error(ErrorCode::InvalidArgument, "sync_block_tables_to_gpu: bad slot");
        const auto& c = caches_[slot];
        if (c.num_blocks() > max_blocks) return Error(ErrorCode::BufferTooSmall, "sync_block_tables_to_gpu: table wider than max_blocks");
        std::copy(c.block_table().begin(), c.block_table().end(), staging_.begin() + i * max_blocks);
        staging_[n * max_blocks + i] = c.seq_len();
    }
    int rc = granite_cuda_write_buffer(compute->handle(), d_tables, staging_.data(), n * max_blocks * 4);
    if (!rc) rc = granite_cuda_write_buffer(compute->handle(), d_seq_lens, staging_.data() + n * max_blocks, n * 4);
    // staging_ is pageable host memory that the next call overwrites: wait for the copies
    if (!rc) rc = granite_cuda_sync(compute->handle());
    return cuda_result(rc);
}

// =================================================================== SpeculationTree (src/llm/speculation_tree.cpp)
int SpeculationTree::add_node(int32_t token, int parent_idx, float log_prob) {
    const int idx = static_cast<int>(nodes_.size());
    Node n{token, parent_idx, 0, log_prob, {}};
    if (parent_idx >= 0) {
        n.depth = nodes_[parent_idx].depth + 1;
        nodes_[parent_idx].children.push_back(idx);
    }
    nodes_.push_back(std::move(n));
    return idx;
}

std::vector<int> SpeculationTree::get_leaves() const {
    std::vector<int> leaves;
    for (size_t i = 0; i < nodes_.size(); i++)
        if (nodes_[i].children.empty()) leaves.push_back(static_cast<int>(i));
    return leaves;
}

std::vector<int> SpeculationTree::get_path(int node_idx) const {
    std::vector<int> path;
    for (int cur = node_idx; cur >= 0; cur = nodes_[cur].parent_idx) path.push_back(cur);
    std::reverse(path.begin(), path.end());
    return path;
}

std::vector<int> SpeculationTree::get_parent_indices() const {
    std::vector<int> parents;
    parents.reserve(nodes_.size());
    for (const auto& n : nodes_) parents.push_back(n.parent_idx);
    return parents;
}

std::vector<int32_t> SpeculationTree::flatten_tokens() const {
    std::vector<int32_t> tokens;
    if (nodes_.empty()) return tokens;
    std::queue<int> q;  // breadth first from node 0, so a parent always precedes its children
    q.push(0);
    while (!q.empty()) {
        const int idx = q.front();
        q.pop();
        tokens.push_back(nodes_[idx].token);
        for (int child : nodes_[idx].children) q.push(child);
    }
    return tokens;
}

int SpeculationTree::max_depth() const {
    int d = 0;
    for (const auto& n : nodes_) d = std::max(d, n.depth);
    return d;
}

std::vector<int32_t> SpeculationTree::find_accepted_path(const std::vector<int32_t>& target_choices) const {
    if (nodes_.empty() || target_choices.empty()) return {};
    std::vector<int32_t> best, cur;
    // depth-first: a node is accepted when its token equals the target's choice at its depth; at
    // the first mismatch the target's own choice closes the path (src/llm/speculation_tree.cpp:85-143)
    std::function<void(int, int)> dfs = [&](int node_idx, int pos) {
        if (node_idx < 0 || pos >= static_cast<int>(target_choices.size())) {
            if (cur.size() > best.size()) best = cur;
            return;
        }
        const Node& n = nodes_[node_idx];
        if (n.token == target_choices[pos]) {
            cur.push_back(n.token);
            if (n.children.empty()) {
                if (cur.size() > best.size()) best = cur;
            } else {
                for (int child : n.children) dfs(child, pos + 1);
            }
            cur.pop_back();
        } else {
            cur.push_back(target_choices[pos]);
            if (cur.size() > best.size()) best = cur;
            cur.pop_back();
        }
    };
    dfs(0, 0);
    return best;
}

std::vector<int> SpeculationTree::find_accepted_nodes(const std::vector<int32_t>& target_choices) const {
    if (nodes_.empty() || target_choices.empty()) return {};
    // the same walk as find_accepted_path, recording nodes; the path that wins there is the one
    // with the most tokens, and the closing token of a mismatch counts as a token but has no node
    std::vector<int> best_nodes, cur;
    size_t best_tokens = 0;
    std::function<void(int, int)> dfs = [&](int node_idx, int pos) {
        if (node_idx < 0 || pos >= static_cast<int>(target_choices.size())) {
            if (cur.size() > best_tokens) {
                best_tokens = cur.size();
                best_nodes = cur;
            }
            return;
        }
        const Node& n = nodes_[node_idx];
        if (n.token == target_choices[pos]) {
            cur.push_back(node_idx);
            if (n.children.empty()) {
                if (cur.size() > best_tokens) {
                    best_tokens = cur.size();
                    best_nodes = cur;
                }
            } else {
                for (int child : n.children) dfs(child, pos + 1);
            }
            cur.pop_back();
        } else if (cur.size() + 1 > best_tokens) {
            best_tokens = cur.size() + 1;
            best_nodes = cur;
        }
    };
    dfs(0, 0);
    return best_nodes;
}

// =================================================================== PagedDecodeBatch
PagedDecodeBatch::~PagedDecodeBatch() {
    if (compute_ && compute_->is_initialized()) {
        if (d_tables_) compute_->destroy_buffer(d_tables_);
        if (d_lens_) compute_->destroy_buffer(d_lens_);
        if (d_positions_) compute_->destroy_buffer(d_positions_);
    }
    if (h_staging_) granite_cuda_free_host(h_staging_);
}

Result<void> PagedDecodeBatch::initialize(PagedKVPool* pool, CudaCompute* compute, RoPECache* rope,
                                          const ModelConfig& config, int max_batch, int max_blocks_per_seq) {
    if (!pool || !compute || !rope) return Error(ErrorCode::NullPointer, "PagedDecodeBatch: null argument");
    if (!pool->is_initialized() || !compute->is_initialized() || !rope->is_initialized())
        return Error(ErrorCode::InvalidState, "PagedDecodeBatch: pool, compute object and RoPE tables must be initialized");
    if (max_batch <= 0 || max_blocks_per_seq <= 0) return Error(ErrorCode::InvalidArgument, "PagedDecodeBatch: empty batch shape");
    pool_ = pool;
    compute_ = compute;
    rope_ = rope;
    config_ = config;
    max_batch_ = max_batch;
    max_blocks_ = max_blocks_per_seq;
    auto up = rope->upload(compute->handle());
    if (!up.ok()) return up;
    d_tables_ = static_cast<int32_t*>(compute->create_buffer(static_cast<size_t>(max_batch) * max_blocks_per_seq * 4));
    d_lens_ = static_cast<int32_t*>(compute->create_buffer(static_cast<size_t>(max_batch) * 4));
    d_positions_ = static_cast<int32_t*>(compute->create_buffer(static_cast<size_t>(max_batch) * 4));
    void* host = nullptr;
    const size_t staging = (static_cast<size_t>(max_batch) * 2 + static_cast<size_t>(max_batch) * max_blocks_per_seq) * 4;
    if (!d_tables_ || !d_lens_ || !d_positions_ || granite_cuda_malloc_host(staging, &host) != 0)
        return Error(ErrorCode::OutOfMemory, "PagedDecodeBatch: allocation failed");
    h_staging_ = static_cast<int32_t*>(host);
    int rc = granite_cuda_memset(compute->handle(), d_tables_, 0, static_cast<size_t>(max_batch) * max_blocks_per_seq * 4);
    return cuda_result(rc);
}

int PagedDecodeBatch::add_request(int slot) {
    if (batch_size() >= max_batch_ || slot < 0 || slot >= pool_->num_slots()) return -1;
    if (std::find(slots_.begin(), slots_.end(), slot) != slots_.end()) return -1;
    slots_.push_back(slot);
    sent_rows_.emplace_back();  // the whole row goes up at the next step
    return batch_size() - 1;
}

void PagedDecodeBatch::remove_request(int slot) {
    auto it = std::find(slots_.begin(), slots_.end(), slot);
    if (it == slots_.end()) return;
    const size_t row = static_cast<size_t>(it - slots_.begin());
    // keep the rows dense: the last row moves into the hole and is re-sent whole
    slots_[row] = slots_.back();
    sent_rows_[row].clear();
    slots_.pop_back();
    sent_rows_.pop_back();
}

Result<std::vector<int>> PagedDecodeBatch::begin_step() {
    if (!pool_) return Error(ErrorCode::InvalidState, "PagedDecodeBatch not initialized");
    std::vector<int> failed;
    for (size_t row = 0; row < slots_.size();) {
        auto& cache = pool_->get_cache(slots_[row]);
        if (cache.seq_len() + 1 > rope_->max_seq_len() || (cache.seq_len() / pool_->block_manager().block_size()) >= max_blocks_ ||
            !cache.append_tokens(1)) {
            failed.push_back(slots_[row]);
            remove_request(slots_[row]);  // the row now holds another request (or none): do not advance
            continue;
        }
        row++;
    }
    const int n = batch_size();
    if (n == 0) return failed;
    // the previous step's copies out of the pinned staging area must have left it
    auto sr = compute_->sync_checked();
    if (!sr.ok()) return sr.error();
    int32_t* positions = h_staging_;
    int32_t* lens = h_staging_ + max_batch_;
    int32_t* rows = h_staging_ + 2 * static_cast<size_t>(max_batch_);
    int rc = 0;
    for (int row = 0; row < n && !rc; row++) {
        const auto& cache = pool_->get_cache(slots_[row]);
        lens[row] = cache.seq_len();
        positions[row] = cache.seq_len() - 1;
        const int have = cache.num_blocks();
        if (have > max_blocks_) return Error(ErrorCode::BufferTooSmall, "PagedDecodeBatch: block table wider than max_blocks_per_seq");
        // only the entries the device row does not hold already: everything from the first one that
        // differs from what was sent (a shrunken table drops the tail of the mirror first)
        auto& sent = sent_rows_[row];
        const auto& table = cache.block_table();
        if (static_cast<int>(sent.size()) > have) sent.resize(static_cast<size_t>(have));
        int first = 0;
        while (first < static_cast<int>(sent.size()) && sent[static_cast<size_t>(first)] == table[static_cast<size_t>(first)]) first++;
        if (first < have) {
            int32_t* stage = rows + static_cast<size_t>(row) * max_blocks_;
            std::copy(table.begin() + first, table.begin() + have, stage + first);
            rc = granite_cuda_write_buffer(compute_->handle(), d_tables_ + static_cast<size_t>(row) * max_blocks_ + first,
                                           stage + first, static_cast<size_t>(have - first) * 4);
            sent.assign(table.begin(), table.begin() + have);
        }
    }
    if (!rc) rc = granite_cuda_write_buffer(compute_->handle(), d_positions_, positions, static_cast<size_t>(n) * 4);
    if (!rc) rc = granite_cuda_write_buffer(compute_->handle(), d_lens_, lens, static_cast<size_t>(n) * 4);
    if (rc) return cuda_error(rc);
    return failed;
}

Result<void> PagedDecodeBatch::attend(int layer, float* q, const float* k, const float* v, float* out, float scale) {
    if (!pool_) return Error(ErrorCode::InvalidState, "PagedDecodeBatch not initialized");
    const int n = batch_size();
    if (n == 0) return {};
    auto& bm = pool_->block_manager();
    if (layer < 0 || layer >= bm.config().num_layers) return Error(ErrorCode::InvalidArgument, "PagedDecodeBatch: bad layer");
    void* backend_k = bm.k_cache(layer).backend()->get_native_buffer(bm.k_cache(layer).buffer());
    void* backend_v = bm.v_cache(layer).backend()->get_native_buffer(bm.v_cache(layer).buffer());
    GraniteCudaRopeAppendArgs a{};
    a.q = q;
    a.k = k;
    a.v = v;
    a.cos_table = rope_->device_cos();
    a.sin_table = rope_->device_sin();
    a.k_cache = backend_k;
    a.v_cache = backend_v;
    a.block_tables = d_tables_;
    a.positions = d_positions_;
    a.batch_size = static_cast<uint32_t>(n);
    a.new_len = 1;
    a.num_heads = static_cast<uint32_t>(config_.num_heads);
    a.num_kv_heads = static_cast<uint32_t>(config_.num_kv_heads);
    a.head_dim = static_cast<uint32_t>(config_.head_dim);
    a.block_size = static_cast<uint32_t>(bm.block_size());
    a.max_blocks_per_seq = static_cast<uint32_t>(max_blocks_);
    a.num_blocks = static_cast<uint32_t>(bm.num_total_blocks());
    a.table_len = static_cast<uint32_t>(rope_->max_seq_len());
    auto r = compute_->rope_paged_kv_cache_append(a);
    if (!r.ok()) return r;
    return compute_->batched_paged_attention_decode(q, backend_k, backend_v, d_tables_, d_lens_, out, a.batch_size,
                                                    a.num_heads, a.num_kv_heads, a.head_dim, a.block_size,
                                                    a.max_blocks_per_seq, scale, a.num_blocks);
}

}  // namespace granite
