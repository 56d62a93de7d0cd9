// TEST INFRASTRUCTURE ONLY - never linked into, imported by or called from the product.
//
// C-ABI glue over the Granite reference's OWN, unmodified sources (compiled where they lie in
// the reference checkout by oracle/Makefile into oracle/_ref/libgranite_ref.so). It exposes the
// reference behaviours that the attention path depends on, so that the CPU restatement in
// granite_attention_oracle.c and the HBM page manager of the product can be checked against the
// real thing:
//   * fp16 <-> fp32 conversion           (src/llm/math_ops.cpp:18-54)
//   * BlockManager / PagedKVCache / PagedKVPool block numbering
//                                        (src/llm/paged_kv_cache.cpp:17-258)
//   * KVCache append layout              (src/llm/kv_cache.cpp:52-107)
//   * SpeculationTree parent arrays      (src/llm/speculation_tree.cpp:13-84)
//   * parallel_for / get_num_threads     (src/llm/math_ops.h:41-69, math_ops.cpp:56-58)
// Only this glue file is ours; nothing of the reference is copied into the repository.

#include "granite/backend.h"
#include "granite/llm.h"
#include "granite/tensor.h"

#include "math_ops.h"  // reference src/llm/math_ops.h (on the include path)

#include <cstdint>
#include <cstring>
#include <memory>
#include <vector>

namespace granite {
std::unique_ptr<IComputeBackend> create_cpu_backend();
}

using namespace granite;

namespace {
IComputeBackend* cpu_backend() {
    static std::unique_ptr<IComputeBackend> be = [] {
        auto b = create_cpu_backend();
        if (b) {
            auto r = b->initialize();
            (void)r;
        }
        return b;
    }();
    return be.get();
}
}  // namespace

extern "C" {

float ref_fp16_to_fp32(uint16_t h) { return fp16_to_fp32(h); }
uint16_t ref_fp32_to_fp16(float f) { return fp32_to_fp16(f); }
// Bit patterns of fp16_to_fp32 for n codes (keeps NaN payloads, which a float return would quiet).
void ref_fp16_to_fp32_bits(const uint16_t* h, uint32_t* bits, size_t n) {
    for (size_t i = 0; i < n; i++) {
        float f = fp16_to_fp32(h[i]);
        std::memcpy(&bits[i], &f, 4);
    }
}
int ref_num_threads(void) { return static_cast<int>(get_num_threads()); }

// Runs `fn(i, user)` for i in [0, n) through the reference's parallel_for with its own thread
// count, so a timed CPU baseline uses the reference's threading policy.
void ref_parallel_for(size_t n, void (*fn)(size_t, void*), void* user) {
    parallel_for(n, get_num_threads(), [&](size_t i) { fn(i, user); });
}

// Replays a script of page-manager operations on the reference PagedKVPool.
// ops: n_ops triples (opcode, a, b):
//   0 acquire_slot()                  -> result = slot or -1
//   1 append_tokens(slot=a, n=b)      -> result = 1/0
//   2 truncate(slot=a, new_len=b)     -> result = seq_len after
//   3 release_slot(slot=a)            -> result = 0
//   4 block_manager.allocate_block()  -> result = block or -1
//   5 block_manager.free_block(a)     -> result = num_free after
//   6 get_physical_block(slot=a,pos=b)-> result
//   7 get_block_offset(slot=a,pos=b)  -> result
// results[n_ops]; then the final state is dumped: seq_lens[max_sequences],
// table_lens[max_sequences], tables[max_sequences*max_blocks] (-1 padded), *num_free.
// Returns 0, or -1 if the pool failed to initialise.
int ref_paged_pool_script(int max_sequences, int max_total_tokens, int block_size,
                          const int32_t* ops, int n_ops, int32_t* results,
                          int32_t* seq_lens, int32_t* table_lens, int32_t* tables,
                          int max_blocks, int32_t* num_free, int32_t* num_total) {
    ModelConfig cfg;
    cfg.num_layers = 1;
    cfg.num_kv_heads = 1;
    cfg.head_dim = 8;
    PagedKVPool pool;
    auto r = pool.initialize(cfg, max_sequences, max_total_tokens, block_size, cpu_backend());
    if (!r.ok()) return -1;
    for (int i = 0; i < n_ops; i++) {
        int op = ops[3 * i], a = ops[3 * i + 1], b = ops[3 * i + 2];
        int32_t res = 0;
        switch (op) {
            case 0: res = pool.acquire_slot(); break;
            case 1: res = pool.get_cache(a).append_tokens(b) ? 1 : 0; break;
            case 2: pool.get_cache(a).truncate(b); res = pool.get_cache(a).seq_len(); break;
            case 3: pool.release_slot(a); res = 0; break;
            case 4: res = pool.block_manager().allocate_block(); break;
            case 5: pool.block_manager().free_block(a); res = pool.num_free_blocks(); break;
            case 6: res = pool.get_cache(a).get_physical_block(b); break;
            case 7: res = pool.get_cache(a).get_block_offset(b); break;
            default: res = -999;
        }
        results[i] = res;
    }
    for (int s = 0; s < max_sequences; s++) {
        const auto& c = pool.get_cache(s);
        seq_lens[s] = c.seq_len();
        table_lens[s] = c.num_blocks();
        for (int j = 0; j < max_blocks; j++) {
            tables[s * max_blocks + j] = j < c.num_blocks() ? c.block_table()[j] : -1;
        }
    }
    *num_free = pool.num_free_blocks();
    *num_total = pool.block_manager().num_total_blocks();
    return 0;
}

// Appends `n_steps` chunks of fp16 K rows through the reference KVCache and dumps layer 0's K
// buffer ([1,Hkv,max_seq,D] fp16). chunk i holds step_lens[i] tokens laid out [1,Hkv,len,D].
int ref_kvcache_append(int num_kv_heads, int head_dim, int max_seq, const int32_t* step_lens,
                       int n_steps, const uint16_t* k_chunks, const uint16_t* v_chunks,
                       uint16_t* k_out, uint16_t* v_out, int32_t* final_len) {
    ModelConfig cfg;
    cfg.num_layers = 1;
    cfg.num_kv_heads = num_kv_heads;
    cfg.head_dim = head_dim;
    auto* be = cpu_backend();
    auto cr = KVCache::allocate(cfg, max_seq, be);
    if (!cr.ok()) return -1;
    KVCache cache = std::move(cr).take();
    {
        auto [k0, v0] = cache.get(0);
        auto mk = be->map_buffer(k0.buffer());
        auto mv = be->map_buffer(v0.buffer());
        std::memset(mk.value(), 0, k0.size_bytes());
        std::memset(mv.value(), 0, v0.size_bytes());
    }
    size_t off = 0;
    for (int i = 0; i < n_steps; i++) {
        std::vector<int64_t> shape = {1, num_kv_heads, step_lens[i], head_dim};
        auto kt = Tensor::allocate(shape, DataType::FP16, be);
        auto vt = Tensor::allocate(shape, DataType::FP16, be);
        if (!kt.ok() || !vt.ok()) return -2;
        Tensor k = std::move(kt).take(), v = std::move(vt).take();
        size_t n = static_cast<size_t>(num_kv_heads) * step_lens[i] * head_dim;
        std::memcpy(be->map_buffer(k.buffer()).value(), k_chunks + off, n * 2);
        std::memcpy(be->map_buffer(v.buffer()).value(), v_chunks + off, n * 2);
        off += n;
        auto ar = cache.append(0, k, v);
        if (!ar.ok()) return -3;
        be->destroy_buffer(k.buffer());
        be->destroy_buffer(v.buffer());
    }
    auto [kc, vc] = cache.get(0);
    std::memcpy(k_out, be->map_buffer(kc.buffer()).value(), kc.size_bytes());
    std::memcpy(v_out, be->map_buffer(vc.buffer()).value(), vc.size_bytes());
    *final_len = cache.seq_len();
    return 0;
}

// RoPECache::initialize (src/llm/rope.cpp:5-22): the cos / sin tables [max_seq, head_dim/2].
int ref_rope_table(int max_seq, int head_dim, float theta, float* cos_out, float* sin_out) {
    RoPECache rope;
    rope.initialize(max_seq, head_dim, theta);
    std::memcpy(cos_out, rope.cos_cache().data(), rope.cos_cache().size() * sizeof(float));
    std::memcpy(sin_out, rope.sin_cache().data(), rope.sin_cache().size() * sizeof(float));
    return 0;
}

// RoPECache::apply (src/llm/rope.cpp:24-92) on q [1, seq, Hq, D] and k [1, seq, Hk, D], in place.
int ref_rope_apply(float* q, float* k, int seq_len, int num_heads_q, int num_heads_k, int head_dim,
                   int start_pos, int max_seq, float theta) {
    auto* be = cpu_backend();
    RoPECache rope;
    rope.initialize(max_seq, head_dim, theta);
    std::vector<int64_t> qs = {1, seq_len, num_heads_q, head_dim}, ks = {1, seq_len, num_heads_k, head_dim};
    auto qt = Tensor::allocate(qs, DataType::FP32, be);
    auto kt = Tensor::allocate(ks, DataType::FP32, be);
    if (!qt.ok() || !kt.ok()) return -1;
    Tensor tq = std::move(qt).take(), tk = std::move(kt).take();
    std::memcpy(be->map_buffer(tq.buffer()).value(), q, tq.size_bytes());
    std::memcpy(be->map_buffer(tk.buffer()).value(), k, tk.size_bytes());
    auto r = rope.apply(tq, tk, start_pos, be);
    int rc = r.ok() ? 0 : static_cast<int>(r.error().code());
    if (rc == 0) {
        std::memcpy(q, be->map_buffer(tq.buffer()).value(), tq.size_bytes());
        std::memcpy(k, be->map_buffer(tk.buffer()).value(), tk.size_bytes());
    }
    be->destroy_buffer(tq.buffer());
    be->destroy_buffer(tk.buffer());
    return rc;
}

// Builds a SpeculationTree by add_node(token=i, parent=parents[i]) and returns its parent
// array, node depths and BFS-flattened tokens.
int ref_speculation_tree(const int32_t* parents, int n, int32_t* parents_out, int32_t* depths,
                         int32_t* bfs_tokens, int32_t* n_bfs, int32_t* max_depth) {
    SpeculationTree tree;
    for (int i = 0; i < n; i++) tree.add_node(i, parents[i], 0.0f);
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

// SpeculationTree::find_accepted_path (src/llm/speculation_tree.cpp:85-143) on a tree built from
// (token, parent) pairs.
int ref_find_accepted_path(const int32_t* parents, const int32_t* tokens, int n, const int32_t* targets,
                           int n_targets, int32_t* out, int32_t* n_out) {
    SpeculationTree tree;
    for (int i = 0; i < n; i++) tree.add_node(tokens[i], parents[i], 0.0f);
    auto path = tree.find_accepted_path(std::vector<int32_t>(targets, targets + n_targets));
    *n_out = static_cast<int32_t>(path.size());
    for (size_t i = 0; i < path.size(); i++) out[i] = path[i];
    return 0;
}

}  // extern "C"
