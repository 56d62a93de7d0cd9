// TEST INFRASTRUCTURE ONLY - never linked into, imported by or called from the product.
//
// The reference's OWN attention statements, compiled.  TransformerModel::attention() and
// attention_tree() (src/llm/transformer.mm) cannot be called with injected Q/K/V - they project
// from model weights - and transformer.mm does not compile without Metal.  Their arithmetic,
// however, sits in blocks that only use local variables.  oracle/slice_reference.py cuts those
// blocks out of the checkout into oracle/_ref/*.inc at build time (generated, git-ignored), and
// each function below is nothing but a parameter list that carries the names the block uses,
// the #include of the block, and a copy of its result:
//   attention_loop.inc         transformer.mm:1779-1840  scores, causal test, softmax, P.V
//   attention_cache_widen.inc  transformer.mm:1753-1765  fp16 cache -> fp32 [total_seq, Hkv, D]
//   tree_loop.inc              transformer.mm:2044-2126  prefix + masked tree attention
//   tree_mask.inc              transformer.mm:822-841    ancestor mask from the parent array
// parallel_for, get_num_threads and fp16_to_fp32 are the reference's (src/llm/math_ops.{h,cpp}).
// Built with -ffp-contract=off like the rest of the checker, so the float sums keep the order and
// rounding the statements spell out.

#include "math_ops.h"  // reference src/llm/math_ops.h (on the include path)

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

using namespace granite;

namespace {
// what the widening block asks of the cache object it reads
struct CacheGeometry {
    int max_seq;
    int max_seq_len() const { return max_seq; }
};
}  // namespace

extern "C" {

// q_data [batch, seq_len, num_heads, head_dim]; k_all, v_all [total_seq, num_kv_heads, head_dim];
// out [batch, seq_len, num_heads, head_dim] receives the block's `context`.
void ref_attention_loop(float* q_data, const float* k_all, const float* v_all, float* out, int batch, int seq_len,
                        int total_seq, int num_heads, int num_kv_heads, int head_dim, int start_pos, float scale) {
#include "_ref/attention_loop.inc"
    std::memcpy(out, context.data(), context.size() * sizeof(float));
}

// ck, cv [num_kv_heads, max_seq, head_dim] fp16 bits -> k_out, v_out [total_seq, num_kv_heads, head_dim] fp32.
void ref_attention_cache_widen(const uint16_t* ck, const uint16_t* cv, float* k_out, float* v_out, int num_kv_heads,
                               int max_seq, int total_seq, int head_dim) {
    const CacheGeometry geometry{max_seq};
    const CacheGeometry* kv_cache = &geometry;
    std::vector<float> k_buffer(static_cast<size_t>(total_seq) * num_kv_heads * head_dim);
    std::vector<float> v_buffer(k_buffer.size());
#include "_ref/attention_cache_widen.inc"
    std::memcpy(k_out, k_buffer.data(), k_buffer.size() * sizeof(float));
    std::memcpy(v_out, v_buffer.data(), v_buffer.size() * sizeof(float));
}

// mask_out [num_nodes, num_nodes] bytes, 1 = node i may attend to node j.
void ref_tree_mask(const int32_t* parents, int num_nodes, uint8_t* mask_out) {
    const std::vector<int> parent_indices(parents, parents + num_nodes);
    const bool use_gpu = false;
#include "_ref/tree_mask.inc"
    for (int i = 0; i < num_nodes; i++)
        for (int j = 0; j < num_nodes; j++) mask_out[i * num_nodes + j] = tree_mask[i][j] ? 1 : 0;
}

// q_data [batch, num_nodes, num_heads, head_dim]; k_cached, v_cached [cached_len, num_kv_heads, head_dim];
// k_data, v_data [batch, num_nodes, num_kv_heads, head_dim]; the mask is built by the reference's own
// block from `parents`; out [batch, num_nodes, num_heads, head_dim] receives `context`.
void ref_attention_tree_loop(float* q_data, const float* k_cached, const float* v_cached, float* k_data, float* v_data,
                             const int32_t* parents, float* out, int batch, int num_nodes, int cached_len, int num_heads,
                             int num_kv_heads, int head_dim, float scale) {
    const std::vector<int> parent_indices(parents, parents + num_nodes);
    const bool use_gpu = false;
#include "_ref/tree_mask.inc"
    const int total_kv = cached_len + num_nodes;
#include "_ref/tree_loop.inc"
    std::memcpy(out, context.data(), context.size() * sizeof(float));
}

}  // extern "C"
