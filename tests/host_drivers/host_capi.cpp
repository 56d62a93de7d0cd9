// extern "C" drivers of the C++ host faces (granite_host.h), so that tests written in another
// language can exercise them the way Granite's own Catch2 tests exercise its backends:
// the operator registry flow of tests/test_vulkan.cpp:353-482, page-manager scripts, the
// speculation tree, the contiguous KVCache and an end-to-end paged decode through
// PagedKVPool + CudaCompute.  TEST CODE: built into its own library beside the tests
// (tests/host_drivers/build.py), never into the product library.
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include "granite_host.h"

using namespace granite;

namespace {
int code_of(const Error& e) { return static_cast<int>(e.code()); }
thread_local std::string g_host_error;
int host_fail(const Error& e) {
    g_host_error = e.message();
    return code_of(e);
}
}  // namespace

extern "C" {

const char* granite_host_last_error(void) { return g_host_error.c_str(); }

// Replays page-manager operations on a PagedKVPool without device pools (num_layers = 0, so it
// runs anywhere).  Opcodes and outputs as in the reference harness used to make the golden files:
//   0 acquire_slot | 1 append_tokens(slot a, n b) | 2 truncate(slot a, len b) | 3 release_slot(a)
//   4 allocate_block | 5 free_block(a) | 6 get_physical_block(a, b) | 7 get_block_offset(a, b)
int granite_host_paged_pool_script(int max_sequences, int max_total_tokens, int block_size, const int32_t* ops,
                                   int n_ops, int32_t* results, int32_t* seq_lens, int32_t* table_lens,
                                   int32_t* tables, int max_blocks, int32_t* num_free, int32_t* num_total) {
    ModelConfig cfg;  // no layers: no pools are allocated
    cfg.num_kv_heads = 1;
    cfg.head_dim = 8;
    PagedKVPool pool;
    auto r = pool.initialize(cfg, max_sequences, max_total_tokens, block_size, nullptr);
    if (!r.ok()) return host_fail(r.error());
    for (int i = 0; i < n_ops; i++) {
        const int op = ops[3 * i], a = ops[3 * i + 1], b = ops[3 * i + 2];
        int32_t res = 0;
        switch (op) {
            case 0: res = pool.acquire_slot(); break;
            case 1: res = pool.get_cache(a).append_tokens(b) ? 1 : 0; break;
            case 2: pool.get_cache(a).truncate(b); res = pool.get_cache(a).seq_len(); break;
            case 3: pool.release_slot(a); break;
            case 4: res = pool.block_manager().allocate_block(); break;
            case 5: pool.block_manager().free_block(a); res = pool.num_free_blocks(); break;
            case 6: res = pool.get_cache(a).get_physical_block(b); break;
            case 7: res = pool.get_cache(a).get_block_offset(b); break;
            default: res = -999;
        }
        results[i] = res;
    }
    for (int s = 0; s < max_sequences; s++) {
        auto& c = pool.get_cache(s);
        seq_lens[s] = c.seq_len();
        table_lens[s] = c.num_blocks();
        for (int j = 0; j < max_blocks; j++) tables[s * max_blocks + j] = j < c.num_blocks() ? c.block_table()[j] : -1;
    }
    *num_free = pool.num_free_blocks();
    *num_total = pool.block_manager().num_total_blocks();
    return 0;
}

int granite_host_speculation_tree(const int32_t* parents, int n, int32_t* parents_out, int32_t* depths,
                                  int32_t* bfs_tokens, int32_t* n_bfs, int32_t* max_depth) {
    SpeculationTree tree;
    for (int i = 0; i < n; i++) tree.add_node(i, parents[i]);
    auto p = tree.get_parent_indices();
    for (int i = 0; i < n; i++) {
        parents_out[i] = p[i];
        depths[i] = tree.node(i).depth;
    }
    auto flat = tree.flatten_tokens();
    *n_bfs = static_cast<int32_t>(flat.size());
    for (size_t i = 0; i < flat.size(); i++) bfs_tokens[i] = flat[i];
    *max_depth = tree.max_depth();
    return 0;
}

int granite_host_find_accepted_path(const int32_t* parents, const int32_t* tokens, int n, const int32_t* targets,
                                    int n_targets, int32_t* out, int32_t* n_out) {
    SpeculationTree tree;
    for (int i = 0; i < n; i++) tree.add_node(tokens[i], parents[i]);
    auto path = tree.find_accepted_path(std::vector<int32_t>(targets, targets + n_targets));
    *n_out = static_cast<int32_t>(path.size());
    for (size_t i = 0; i < path.size(); i++) out[i] = path[i];
    return 0;
}

// Buffer semantics of the CUDA backend: returns 0, or the number of the first failing step.
int granite_host_backend_selftest(int device) {
    auto be = create_cuda_backend(device);
    auto init = be->initialize();
    if (!init.ok()) return host_fail(init.error());
    if (be->get_type() != kCudaBackendType || !be->is_initialized()) return 1001;
    std::vector<uint8_t> pattern(4096), back(4096, 0);
    for (size_t i = 0; i < pattern.size(); i++) pattern[i] = static_cast<uint8_t>(i * 7 + 3);
    for (MemoryType mt : {MemoryType::Device, MemoryType::Managed, MemoryType::Shared}) {
        auto h = be->create_buffer(BufferDesc{pattern.size(), mt, false});
        if (!h.ok()) return 1002;
        if (!be->write_buffer(h.value(), pattern.data(), pattern.size()).ok()) return 1003;
        std::fill(back.begin(), back.end(), 0);
        if (!be->read_buffer(h.value(), back.data(), back.size()).ok() || back != pattern) return 1004;
        auto m = be->map_buffer(h.value());  // map sees the device contents
        if (!m.ok() || std::memcmp(m.value(), pattern.data(), pattern.size()) != 0) return 1005;
        static_cast<uint8_t*>(m.value())[5] = 0xAB;  // unmap publishes host writes
        be->unmap_buffer(h.value());
        if (!be->read_buffer(h.value(), back.data(), 16).ok() || back[5] != 0xAB) return 1006;
        if (be->write_buffer(h.value(), pattern.data(), 8, pattern.size()).ok()) return 1007;  // past the end
        if (!be->get_native_buffer(h.value())) return 1008;
        auto h2 = be->create_buffer(BufferDesc::device(pattern.size()));
        if (!h2.ok() || !be->copy_buffer(h.value(), h2.value(), 1024, 16, 32).ok()) return 1009;
        if (!be->read_buffer(h2.value(), back.data(), 1024, 32).ok() || back[0] != pattern[16]) return 1010;
        be->destroy_buffer(h.value());
        be->destroy_buffer(h2.value());
        if (be->map_buffer(h.value()).ok()) return 1011;  // destroyed handle
    }
    if (be->create_buffer(BufferDesc::device(0)).ok()) return 1012;
    auto pipe = be->create_pipeline(PipelineDesc{});
    if (pipe.ok() || pipe.error().code() != ErrorCode::NotImplemented) return 1013;
    if (!be->wait_for_completion().ok()) return 1014;
    be->shutdown();
    if (be->is_initialized()) return 1015;
    return 0;
}

// The operator flow of the reference's attention test: tensors allocated through the backend,
// filled through map/unmap, the operator created from the registry, shapes inferred, executed,
// output read through map.  dtype 0: fp32 with K given as [D, T]; 1: fp16 bits with K as [T, D].
int granite_host_operator_attention(int device, int dtype, const void* q, const void* k, const void* v, void* out,
                                    int seq_q, int seq_kv, int head_dim, int has_scale, double scale,
                                    int64_t start_pos) {
    auto be = create_cuda_backend(device);
    auto init = be->initialize();
    if (!init.ok()) return host_fail(init.error());
    register_cuda_operators();
    if (OperatorRegistry::instance().create(OpType::ScaledDotProductAttention, BackendType::CPU))
        return 2001;  // nothing must be registered for the CPU: there is no fallback
    const DataType dt = dtype == 0 ? DataType::FP32 : DataType::FP16;
    const std::vector<int64_t> shape_q = {seq_q, head_dim};
    const std::vector<int64_t> shape_k = dtype == 0 ? std::vector<int64_t>{head_dim, seq_kv} : std::vector<int64_t>{seq_kv, head_dim};
    const std::vector<int64_t> shape_v = {seq_kv, head_dim};
    auto tq = Tensor::allocate(shape_q, dt, be.get());
    auto tk = Tensor::allocate(shape_k, dt, be.get());
    auto tv = Tensor::allocate(shape_v, dt, be.get());
    if (!tq.ok() || !tk.ok() || !tv.ok()) return 2002;
    const void* srcs[3] = {q, k, v};
    Tensor ts[3] = {tq.value(), tk.value(), tv.value()};
    for (int i = 0; i < 3; i++) {
        auto m = be->map_buffer(ts[i].buffer());
        if (!m.ok()) return 2003;
        std::memcpy(m.value(), srcs[i], ts[i].size_bytes());
        be->unmap_buffer(ts[i].buffer());
    }
    auto op = OperatorRegistry::instance().create(OpType::ScaledDotProductAttention, kCudaBackendType);
    if (!op) return 2004;
    OpContext ctx;
    ctx.backend = be.get();
    ctx.inputs = {ts[0], ts[1], ts[2]};
    if (has_scale) ctx.attrs.set("scale", scale);
    if (start_pos) ctx.attrs.set("start_pos", start_pos);
    auto shapes = op->infer_shapes(ctx);
    if (!shapes.ok() || shapes.value()[0] != shape_q) return 2005;
    auto to = Tensor::allocate(shapes.value()[0], dt, be.get());
    if (!to.ok()) return 2006;
    ctx.outputs = {to.value()};
    auto ex = op->execute(ctx);
    if (!ex.ok()) return host_fail(ex.error());
    auto mo = be->map_buffer(ctx.outputs[0].buffer());
    if (!mo.ok()) return 2007;
    std::memcpy(out, mo.value(), ctx.outputs[0].size_bytes());
    be->unmap_buffer(ctx.outputs[0].buffer());
    OpContext too_few;  // fewer than three inputs is InvalidArgument
    too_few.backend = be.get();
    too_few.inputs = {ts[0]};
    auto bad = op->validate(too_few);
    if (bad.ok() || bad.error().code() != ErrorCode::InvalidArgument) return 2008;
    be->shutdown();
    return 0;
}

// Contiguous KVCache on the device: appends fp16 chunks ([1, Hkv, len, D] each) and returns layer
// 0's K and V buffers ([Hkv, max_seq, D]); fills *final_len and *overflow_code (the error code of
// one extra append that must overflow).
int granite_host_kvcache_append(int device, int num_kv_heads, int head_dim, int max_seq, const int32_t* step_lens,
                                int n_steps, const uint16_t* k_chunks, const uint16_t* v_chunks, uint16_t* k_out,
                                uint16_t* v_out, int32_t* final_len, int32_t* overflow_code) {
    auto be = create_cuda_backend(device);
    auto init = be->initialize();
    if (!init.ok()) return host_fail(init.error());
    ModelConfig cfg;
    cfg.num_layers = 2;
    cfg.num_kv_heads = num_kv_heads;
    cfg.head_dim = head_dim;
    auto cr = KVCache::allocate(cfg, max_seq, be.get());
    if (!cr.ok()) return host_fail(cr.error());
    KVCache cache = std::move(cr).take();
    std::vector<uint8_t> zeros(static_cast<size_t>(num_kv_heads) * max_seq * head_dim * 2, 0);
    for (int layer = 0; layer < 2; layer++) {
        auto kv = cache.get(layer);
        be->write_buffer(kv.first.buffer(), zeros.data(), zeros.size());
        be->write_buffer(kv.second.buffer(), zeros.data(), zeros.size());
    }
    size_t off = 0;
    for (int i = 0; i < n_steps; i++) {
        const std::vector<int64_t> shape = {1, num_kv_heads, step_lens[i], head_dim};
        auto kt = Tensor::allocate(shape, DataType::FP16, be.get());
        auto vt = Tensor::allocate(shape, DataType::FP16, be.get());
        if (!kt.ok() || !vt.ok()) return 3001;
        const size_t n = static_cast<size_t>(num_kv_heads) * step_lens[i] * head_dim;
        be->write_buffer(kt.value().buffer(), k_chunks + off, n * 2);
        be->write_buffer(vt.value().buffer(), v_chunks + off, n * 2);
        off += n;
        for (int layer = 0; layer < 2; layer++) {  // the length only moves with the last layer
            if (layer == 1 && cache.seq_len() + step_lens[i] > max_seq) break;
            auto ar = cache.append(layer, kt.value(), vt.value());
            if (!ar.ok()) return host_fail(ar.error());
        }
        be->destroy_buffer(kt.value().buffer());
        be->destroy_buffer(vt.value().buffer());
    }
    *final_len = cache.seq_len();
    {
        const std::vector<int64_t> shape = {1, num_kv_heads, max_seq - cache.seq_len() + 1, head_dim};
        auto kt = Tensor::allocate(shape, DataType::FP16, be.get());
        auto ar = cache.append(0, kt.value(), kt.value());
        *overflow_code = ar.ok() ? 0 : code_of(ar.error());
    }
    auto kv = cache.get(0);
    be->read_buffer(kv.first.buffer(), k_out, zeros.size());
    be->read_buffer(kv.second.buffer(), v_out, zeros.size());
    cache.truncate(1);
    if (cache.seq_len() != (*final_len > 1 ? 1 : *final_len)) return 3002;
    be->shutdown();
    return 0;
}

// End to end through the page manager in HBM: a PagedKVPool on the CUDA backend, one slot per
// sequence, tokens appended in ragged steps (block tables grow through BlockManager), fp32 K/V
// written into the pool with paged_kv_cache_append, tables mirrored to the device, then one
// batched paged decode.  Returns the outputs, the tables and layer 0's pools.
//   k_src/v_src: [batch][Hkv, len_b, D] fp32 concatenated; q [batch, Hq, D]; lens [batch]
int granite_host_paged_flow(int device, int batch, const int32_t* lens, int num_heads, int num_kv_heads, int head_dim,
                            int block_size, int num_blocks, const float* k_src, const float* v_src, const float* q,
                            float* out, int32_t* tables_out, int max_blocks, uint16_t* k_pool_out,
                            uint16_t* v_pool_out, int step) {
    auto be = create_cuda_backend(device);
    auto init = be->initialize();
    if (!init.ok()) return host_fail(init.error());
    auto* compute_handle = static_cast<granite_cuda_compute_t*>(be->get_native_device());
    // a CudaCompute that shares the backend's stream, so ordering between the two is trivial
    CudaCompute compute;
    auto ci = compute.initialize(device, be->get_native_queue());
    if (!ci.ok()) return host_fail(ci.error());
    (void)compute_handle;
    ModelConfig cfg;
    cfg.num_layers = 1;
    cfg.num_heads = num_heads;
    cfg.num_kv_heads = num_kv_heads;
    cfg.head_dim = head_dim;
    PagedKVPool pool;
    auto pr = pool.initialize(cfg, batch, num_blocks * block_size, block_size, be.get());
    if (!pr.ok()) return host_fail(pr.error());
    void* kpool = be->get_native_buffer(pool.block_manager().k_cache(0).buffer());
    void* vpool = be->get_native_buffer(pool.block_manager().v_cache(0).buffer());
    const size_t pool_bytes = pool.block_manager().k_cache(0).size_bytes();
    granite_cuda_memset(compute.handle(), kpool, 0, pool_bytes);
    granite_cuda_memset(compute.handle(), vpool, 0, pool_bytes);

    std::vector<int> slots(batch);
    for (int b = 0; b < batch; b++) {
        slots[b] = pool.acquire_slot();
        if (slots[b] < 0) return 4001;
    }
    auto d_table = static_cast<int32_t*>(compute.create_buffer(static_cast<size_t>(max_blocks) * 4));
    size_t src_off = 0;
    // interleave the sequences' growth so that their pages end up interleaved in the pool
    std::vector<int> done(batch, 0);
    bool more = true;
    while (more) {
        more = false;
        for (int b = 0; b < batch; b++) {
            if (done[b] >= lens[b]) continue;
            const int n = std::min(step, lens[b] - done[b]);
            auto& cache = pool.get_cache(slots[b]);
            if (!cache.append_tokens(n)) return static_cast<int>(ErrorCode::OutOfMemory);
            // the rows of this step as a contiguous [Hkv, n, D] block
            std::vector<float> kb(static_cast<size_t>(num_kv_heads) * n * head_dim), vb(kb.size());
            size_t seq_off = 0;
            for (int bb = 0; bb < b; bb++) seq_off += static_cast<size_t>(num_kv_heads) * lens[bb] * head_dim;
            for (int h = 0; h < num_kv_heads; h++)
                for (int s = 0; s < n; s++)
                    for (int d = 0; d < head_dim; d++) {
                        const size_t src = seq_off + (static_cast<size_t>(h) * lens[b] + done[b] + s) * head_dim + d;
                        const size_t dst = (static_cast<size_t>(h) * n + s) * head_dim + d;
                        kb[dst] = k_src[src];
                        vb[dst] = v_src[src];
                    }
            auto* d_k = static_cast<float*>(compute.create_buffer(kb.size() * 4));
            auto* d_v = static_cast<float*>(compute.create_buffer(vb.size() * 4));
            granite_cuda_write_buffer(compute.handle(), d_k, kb.data(), kb.size() * 4);
            granite_cuda_write_buffer(compute.handle(), d_v, vb.data(), vb.size() * 4);
            granite_cuda_write_buffer(compute.handle(), d_table, cache.block_table().data(), cache.block_table().size() * 4);
            auto ar = compute.paged_kv_cache_append(d_k, d_v, kpool, vpool, d_table, num_kv_heads, head_dim, done[b], n,
                                                    block_size, pool.block_manager().num_total_blocks(),
                                                    static_cast<uint32_t>(cache.block_table().size()));
            if (!ar.ok()) return host_fail(ar.error());
            auto sr = compute.sync_checked();
            if (!sr.ok()) return host_fail(sr.error());
            compute.destroy_buffer(d_k);
            compute.destroy_buffer(d_v);
            done[b] += n;
            if (done[b] < lens[b]) more = true;
        }
    }
    (void)src_off;
    auto* d_tables = static_cast<int32_t*>(compute.create_buffer(static_cast<size_t>(batch) * max_blocks * 4));
    auto* d_lens = static_cast<int32_t*>(compute.create_buffer(static_cast<size_t>(batch) * 4));
    auto* d_q = static_cast<float*>(compute.create_buffer(static_cast<size_t>(batch) * num_heads * head_dim * 4));
    auto* d_out = static_cast<float*>(compute.create_buffer(static_cast<size_t>(batch) * num_heads * head_dim * 4));
    auto sy = pool.sync_block_tables_to_gpu(&compute, slots, d_tables, max_blocks, d_lens);
    if (!sy.ok()) return host_fail(sy.error());
    granite_cuda_write_buffer(compute.handle(), d_q, q, static_cast<size_t>(batch) * num_heads * head_dim * 4);
    auto dr = compute.batched_paged_attention_decode(d_q, kpool, vpool, d_tables, d_lens, d_out, batch, num_heads,
                                                     num_kv_heads, head_dim, block_size, max_blocks,
                                                     1.0f / std::sqrt(static_cast<float>(head_dim)),
                                                     pool.block_manager().num_total_blocks());
    if (!dr.ok()) return host_fail(dr.error());
    granite_cuda_read_buffer(compute.handle(), out, d_out, static_cast<size_t>(batch) * num_heads * head_dim * 4);
    granite_cuda_read_buffer(compute.handle(), tables_out, d_tables, static_cast<size_t>(batch) * max_blocks * 4);
    granite_cuda_read_buffer(compute.handle(), k_pool_out, kpool, pool_bytes);
    granite_cuda_read_buffer(compute.handle(), v_pool_out, vpool, pool_bytes);
    auto fin = compute.sync_checked();
    if (!fin.ok()) return host_fail(fin.error());
    // releasing every slot returns every block
    for (int s : slots) pool.release_slot(s);
    if (pool.num_free_blocks() != pool.block_manager().num_total_blocks()) return 4002;
    for (void* p : {static_cast<void*>(d_table), static_cast<void*>(d_tables), static_cast<void*>(d_lens),
                    static_cast<void*>(d_q), static_cast<void*>(d_out)})
        compute.destroy_buffer(p);
    compute.shutdown();
    be->shutdown();
    return 0;
}

// SpeculationTree::find_accepted_nodes on a tree built from (token, parent) pairs.
int granite_host_find_accepted_nodes(const int32_t* parents, const int32_t* tokens, int n, const int32_t* targets,
                                     int n_targets, int32_t* out, int32_t* n_out) {
    SpeculationTree tree;
    for (int i = 0; i < n; i++) tree.add_node(tokens[i], parents[i]);
    auto nodes = tree.find_accepted_nodes(std::vector<int32_t>(targets, targets + n_targets));
    *n_out = static_cast<int32_t>(nodes.size());
    for (size_t i = 0; i < nodes.size(); i++) out[i] = nodes[i];
    return 0;
}

// RoPECache::initialize on the host (runs anywhere): the tables [max_seq, head_dim/2].
int granite_host_rope_table(int max_seq, int head_dim, float theta, float* cos_out, float* sin_out) {
    RoPECache rope;
    rope.initialize(max_seq, head_dim, theta);
    std::memcpy(cos_out, rope.cos_cache().data(), rope.cos_cache().size() * sizeof(float));
    std::memcpy(sin_out, rope.sin_cache().data(), rope.sin_cache().size() * sizeof(float));
    return rope.is_initialized() ? 0 : 1;
}

// RoPECache::apply through the CUDA backend's tensors: q [1, seq, Hq, D], k [1, seq, Hk, D] in place.
int granite_host_rope_apply(int device, float* q, float* k, int seq_len, int num_heads_q, int num_heads_k,
                            int head_dim, int start_pos, int max_seq, float theta) {
    auto be = create_cuda_backend(device);
    auto init = be->initialize();
    if (!init.ok()) return host_fail(init.error());
    RoPECache rope;
    Tensor none_q, none_k;
    if (rope.apply(none_q, none_k, 0, be.get()).ok()) return 5001;  // not initialized yet: InvalidState
    rope.initialize(max_seq, head_dim, theta);
    const std::vector<int64_t> q_shape = {1, seq_len, num_heads_q, head_dim}, k_shape = {1, seq_len, num_heads_k, head_dim};
    auto qt = Tensor::allocate(q_shape, DataType::FP32, be.get());
    auto kt = Tensor::allocate(k_shape, DataType::FP32, be.get());
    if (!qt.ok() || !kt.ok()) return 5002;
    Tensor tq = std::move(qt).take(), tk = std::move(kt).take();
    if (!be->write_buffer(tq.buffer(), q, tq.size_bytes()).ok()) return 5003;
    if (!be->write_buffer(tk.buffer(), k, tk.size_bytes()).ok()) return 5003;
    auto r = rope.apply(tq, tk, start_pos, be.get());
    int rc = 0;
    if (!r.ok()) {
        rc = host_fail(r.error());
    } else {
        if (!be->read_buffer(tq.buffer(), q, tq.size_bytes()).ok()) rc = 5004;
        if (!be->read_buffer(tk.buffer(), k, tk.size_bytes()).ok()) rc = 5004;
    }
    be->destroy_buffer(tq.buffer());
    be->destroy_buffer(tk.buffer());
    return rc;
}

// A serving loop in miniature over PagedKVPool + RoPECache + PagedDecodeBatch: `batch` requests
// (slot i = request i) are prefilled with lens0[i] prompt tokens, then decode together for
// n_steps steps; request `remove_slot` leaves before step `remove_at` (its pages go back to the
// pool and are handed out again).  Per step and slot the driver returns the attention output,
// the rotated query, the block table and the length, and at the end both pools, so that the
// caller can replay the whole run on the CPU checker.  Inputs per step are indexed by slot.
int granite_host_decode_batch_flow(int device, int batch, const int32_t* lens0, int n_steps, int remove_slot,
                                   int remove_at, int num_heads, int num_kv_heads, int head_dim, int block_size,
                                   int num_blocks, int max_blocks, int max_seq, const float* prompt_k,
                                   const float* prompt_v, const float* step_q, const float* step_k,
                                   const float* step_v, float* out, float* q_rot_out, int32_t* tables_out,
                                   int32_t* lens_out, uint16_t* k_pool_out, uint16_t* v_pool_out) {
    auto be = create_cuda_backend(device);
    auto init = be->initialize();
    if (!init.ok()) return host_fail(init.error());
    CudaCompute compute;
    auto ci = compute.initialize(device, be->get_native_queue());
    if (!ci.ok()) return host_fail(ci.error());
    ModelConfig cfg;
    cfg.num_layers = 1;
    cfg.num_heads = num_heads;
    cfg.num_kv_heads = num_kv_heads;
    cfg.head_dim = head_dim;
    PagedKVPool pool;
    auto pr = pool.initialize(cfg, batch, num_blocks * block_size, block_size, be.get());
    if (!pr.ok()) return host_fail(pr.error());
    void* kpool = be->get_native_buffer(pool.block_manager().k_cache(0).buffer());
    void* vpool = be->get_native_buffer(pool.block_manager().v_cache(0).buffer());
    const size_t pool_bytes = pool.block_manager().k_cache(0).size_bytes();
    granite_cuda_memset(compute.handle(), kpool, 0, pool_bytes);
    granite_cuda_memset(compute.handle(), vpool, 0, pool_bytes);
    RoPECache rope;
    rope.initialize(max_seq, head_dim);
    auto up = rope.upload(compute.handle());
    if (!up.ok()) return host_fail(up.error());

    const size_t q_row = static_cast<size_t>(num_heads) * head_dim, kv_row = static_cast<size_t>(num_kv_heads) * head_dim;
    auto* d_q = static_cast<float*>(compute.create_buffer(batch * q_row * 4));
    auto* d_out = static_cast<float*>(compute.create_buffer(batch * q_row * 4));
    auto* d_table = static_cast<int32_t*>(compute.create_buffer(static_cast<size_t>(max_blocks) * 4));

    // prefill: each prompt's K/V goes through the fused RoPE + paged write, one sequence per call
    size_t off = 0;
    for (int b = 0; b < batch; b++) {
        if (pool.acquire_slot() != b) return 6001;
        auto& cache = pool.get_cache(b);
        if (lens0[b] == 0) continue;
        if (!cache.append_tokens(lens0[b])) return static_cast<int>(ErrorCode::OutOfMemory);
        auto* d_k = static_cast<float*>(compute.create_buffer(lens0[b] * kv_row * 4));
        auto* d_v = static_cast<float*>(compute.create_buffer(lens0[b] * kv_row * 4));
        granite_cuda_write_buffer(compute.handle(), d_k, prompt_k + off * kv_row, lens0[b] * kv_row * 4);
        granite_cuda_write_buffer(compute.handle(), d_v, prompt_v + off * kv_row, lens0[b] * kv_row * 4);
        granite_cuda_write_buffer(compute.handle(), d_table, cache.block_table().data(), cache.block_table().size() * 4);
        GraniteCudaRopeAppendArgs a{};
        a.k = d_k;
        a.v = d_v;
        a.cos_table = rope.device_cos();
        a.sin_table = rope.device_sin();
        a.k_cache = kpool;
        a.v_cache = vpool;
        a.block_tables = d_table;
        a.batch_size = 1;
        a.new_len = static_cast<uint32_t>(lens0[b]);
        a.num_kv_heads = static_cast<uint32_t>(num_kv_heads);
        a.head_dim = static_cast<uint32_t>(head_dim);
        a.block_size = static_cast<uint32_t>(block_size);
        a.max_blocks_per_seq = static_cast<uint32_t>(cache.block_table().size());
        a.num_blocks = static_cast<uint32_t>(pool.block_manager().num_total_blocks());
        a.table_len = static_cast<uint32_t>(max_seq);
        a.start_pos = 0;
        auto ar = compute.rope_paged_kv_cache_append(a);
        if (!ar.ok()) return host_fail(ar.error());
        auto sr = compute.sync_checked();
        if (!sr.ok()) return host_fail(sr.error());
        compute.destroy_buffer(d_k);
        compute.destroy_buffer(d_v);
        off += lens0[b];
    }

    PagedDecodeBatch decode;
    auto di = decode.initialize(&pool, &compute, &rope, cfg, batch, max_blocks);
    if (!di.ok()) return host_fail(di.error());
    for (int b = 0; b < batch; b++)
        if (decode.add_request(b) != b) return 6002;
    if (decode.add_request(0) != -1) return 6003;  // already present

    std::vector<float> q_rows(batch * q_row), k_rows(batch * kv_row), v_rows(batch * kv_row), o_rows(batch * q_row);
    auto* d_k1 = static_cast<float*>(compute.create_buffer(batch * kv_row * 4));
    auto* d_v1 = static_cast<float*>(compute.create_buffer(batch * kv_row * 4));
    const float scale = 1.0f / std::sqrt(static_cast<float>(head_dim));
    for (int step = 0; step < n_steps; step++) {
        if (step == remove_at && remove_slot >= 0) {
            decode.remove_request(remove_slot);
            pool.release_slot(remove_slot);
        }
        auto bs = decode.begin_step();
        if (!bs.ok()) return host_fail(bs.error());
        if (!bs.value().empty()) return static_cast<int>(ErrorCode::OutOfMemory);
        const int n = decode.batch_size();
        const auto& slots = decode.slots();
        for (int row = 0; row < n; row++) {
            const size_t src = static_cast<size_t>(step) * batch + slots[row];
            std::memcpy(&q_rows[row * q_row], step_q + src * q_row, q_row * 4);
            std::memcpy(&k_rows[row * kv_row], step_k + src * kv_row, kv_row * 4);
            std::memcpy(&v_rows[row * kv_row], step_v + src * kv_row, kv_row * 4);
        }
        granite_cuda_write_buffer(compute.handle(), d_q, q_rows.data(), n * q_row * 4);
        granite_cuda_write_buffer(compute.handle(), d_k1, k_rows.data(), n * kv_row * 4);
        granite_cuda_write_buffer(compute.handle(), d_v1, v_rows.data(), n * kv_row * 4);
        auto at = decode.attend(0, d_q, d_k1, d_v1, d_out, scale);
        if (!at.ok()) return host_fail(at.error());
        granite_cuda_read_buffer(compute.handle(), o_rows.data(), d_out, n * q_row * 4);
        granite_cuda_read_buffer(compute.handle(), q_rows.data(), d_q, n * q_row * 4);
        auto sr = compute.sync_checked();
        if (!sr.ok()) return host_fail(sr.error());
        for (int b = 0; b < batch; b++) {
            lens_out[static_cast<size_t>(step) * batch + b] = -1;
            for (int j = 0; j < max_blocks; j++) tables_out[(static_cast<size_t>(step) * batch + b) * max_blocks + j] = -1;
        }
        for (int row = 0; row < n; row++) {
            const size_t dst = static_cast<size_t>(step) * batch + slots[row];
            std::memcpy(out + dst * q_row, &o_rows[row * q_row], q_row * 4);
            std::memcpy(q_rot_out + dst * q_row, &q_rows[row * q_row], q_row * 4);
            const auto& cache = pool.get_cache(slots[row]);
            lens_out[dst] = cache.seq_len();
            std::copy(cache.block_table().begin(), cache.block_table().end(), tables_out + dst * max_blocks);
        }
    }
    granite_cuda_read_buffer(compute.handle(), k_pool_out, kpool, pool_bytes);
    granite_cuda_read_buffer(compute.handle(), v_pool_out, vpool, pool_bytes);
    auto fin = compute.sync_checked();
    if (!fin.ok()) return host_fail(fin.error());
    for (void* p : {static_cast<void*>(d_q), static_cast<void*>(d_out), static_cast<void*>(d_table),
                    static_cast<void*>(d_k1), static_cast<void*>(d_v1)})
        compute.destroy_buffer(p);
    return 0;
}

// The device block-table rows of PagedDecodeBatch after a sequence's table shrank and regrew
// over different blocks: request 0 grows across a block boundary and is synced; it is truncated
// back across the boundary (its tail block returns to the pool), request 1 grows and is handed
// that block, request 0 regrows over another one.  After the next begin_step the device row of
// each request must equal its PagedKVCache table.  Returns rows as [2, max_blocks] each.
int granite_host_decode_batch_regrow(int device, int block_size, int max_blocks, int32_t* device_rows,
                                     int32_t* host_rows, int32_t* lens_out) {
    auto be = create_cuda_backend(device);
    auto init = be->initialize();
    if (!init.ok()) return host_fail(init.error());
    CudaCompute compute;
    auto ci = compute.initialize(device, be->get_native_queue());
    if (!ci.ok()) return host_fail(ci.error());
    ModelConfig cfg;
    cfg.num_layers = 1;
    cfg.num_heads = 8;
    cfg.num_kv_heads = 2;
    cfg.head_dim = 128;
    PagedKVPool pool;
    auto pr = pool.initialize(cfg, 2, 2 * max_blocks * block_size, block_size, be.get());
    if (!pr.ok()) return host_fail(pr.error());
    RoPECache rope;
    rope.initialize(max_blocks * block_size, cfg.head_dim);
    auto up = rope.upload(compute.handle());
    if (!up.ok()) return host_fail(up.error());
    if (pool.acquire_slot() != 0 || pool.acquire_slot() != 1) return 6101;
    PagedDecodeBatch decode;
    auto di = decode.initialize(&pool, &compute, &rope, cfg, 2, max_blocks);
    if (!di.ok()) return host_fail(di.error());
    if (decode.add_request(0) != 0 || decode.add_request(1) != 1) return 6102;
    // request 0: two full blocks and one token of a third; request 1: half a block
    if (!pool.get_cache(0).append_tokens(2 * block_size) || !pool.get_cache(1).append_tokens(block_size / 2)) return 6103;
    auto s1 = decode.begin_step();  // both grow by one token; rows go up
    if (!s1.ok()) return host_fail(s1.error());
    const int third_before = pool.get_cache(0).block_table()[2];
    pool.get_cache(0).truncate(2 * block_size - 3);                 // frees the third block
    if (!pool.get_cache(1).append_tokens(block_size)) return 6104;  // request 1 takes it
    if (pool.get_cache(1).block_table()[1] != third_before) return 6105;
    if (!pool.get_cache(0).append_tokens(3)) return 6106;           // back to two full blocks
    auto s2 = decode.begin_step();                                  // request 0 crosses the boundary again
    if (!s2.ok()) return host_fail(s2.error());
    if (pool.get_cache(0).block_table()[2] == third_before) return 6107;
    granite_cuda_read_buffer(compute.handle(), device_rows, decode.device_tables(), static_cast<size_t>(2) * max_blocks * 4);
    granite_cuda_read_buffer(compute.handle(), lens_out, decode.device_seq_lens(), 2 * 4);
    auto sr = compute.sync_checked();
    if (!sr.ok()) return host_fail(sr.error());
    for (int b = 0; b < 2; b++) {
        const auto& table = pool.get_cache(b).block_table();
        for (int j = 0; j < max_blocks; j++)
            host_rows[b * max_blocks + j] = j < static_cast<int>(table.size()) ? table[static_cast<size_t>(j)] : -1;
        lens_out[2 + b] = pool.get_cache(b).seq_len();
    }
    return 0;
}

}  // extern "C"
