/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement of Granite's attention arithmetic, used as the
 * parity checker by tests/, by the smoke check and by the cpu_baseline leg of the benchmark.
 * The product never imports, links or calls anything in this directory.
 *
 * Why a restatement: the reference loops sit inside TransformerModel::attention /
 * attention_tree, fused with weight projections and RoPE, and cannot be fed Q/K/V directly
 * (they need a GGUF model).  Each function below follows the cited reference lines statement
 * for statement, including the order of every floating-point sum.
 *
 * Pinning: the conversion helpers and page/tree index rules are checked against the reference's
 * own compiled sources (oracle/_ref, see ref_harness.cpp); the softmax-attention arithmetic is
 * checked against the one known-answer case the reference holds (tests/test_vulkan.cpp:353-482,
 * 2x3x4 operator test).  For attention()/attention_tree() themselves the reference has no
 * golden vectors: parity unpinned by reference tests beyond that case.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- fp16 <-> fp32 : src/llm/math_ops.cpp:18-54 ------------------------------------------ */

float gro_fp16_to_fp32(uint16_t h) {
    uint32_t sign = (uint32_t)(h >> 15) & 1u;
    uint32_t exp = (uint32_t)(h >> 10) & 0x1Fu;
    uint32_t mant = (uint32_t)h & 0x3FFu;
    uint32_t bits;
    float out;
    if (exp == 0) {
        if (mant == 0) {
            bits = sign << 31;
            memcpy(&out, &bits, 4);
            return out;
        }
        /* denormal: normalise (math_ops.cpp:31-32) */
        while ((mant & 0x400u) == 0) {
            mant <<= 1;
            exp--;
        }
        exp++;
        mant &= 0x3FFu;
    } else if (exp == 31) {
        bits = (sign << 31) | 0x7F800000u | (mant << 13);
        memcpy(&out, &bits, 4);
        return out;
    }
    bits = (sign << 31) | ((exp + 112u) << 23) | (mant << 13);
    memcpy(&out, &bits, 4);
    return out;
}

/* Truncating narrow; flushes exp<=0 to signed zero, clamps exp>=31 to inf (math_ops.cpp:45-54). */
uint16_t gro_fp32_to_fp16(float f) {
    uint32_t bits;
    memcpy(&bits, &f, 4);
    uint32_t sign = (bits >> 16) & 0x8000u;
    int32_t exp = (int32_t)((bits >> 23) & 0xFFu) - 127 + 15;
    uint32_t mant = (bits >> 13) & 0x3FFu;
    if (exp <= 0) return (uint16_t)sign;
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
    return (uint16_t)(sign | ((uint32_t)exp << 10) | mant);
}

/* ---- parallel_for : src/llm/math_ops.h:41-69 ---------------------------------------------
 * Same policy: serial when threads<=1 or n<threads; otherwise one freshly created thread per
 * contiguous chunk of ceil(n/threads) items, joined before return. */
typedef void (*gro_body_fn)(size_t idx, void* user);
typedef struct {
    gro_body_fn fn;
    void* user;
    size_t begin, end;
} gro_chunk;

static void* gro_chunk_main(void* p) {
    gro_chunk* c = (gro_chunk*)p;
    for (size_t i = c->begin; i < c->end; i++) c->fn(i, c->user);
    return NULL;
}

static void gro_parallel_for(size_t n, size_t num_threads, gro_body_fn fn, void* user) {
    if (num_threads <= 1 || n < num_threads) {
        for (size_t i = 0; i < n; i++) fn(i, user);
        return;
    }
    pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * num_threads);
    gro_chunk* ch = (gro_chunk*)malloc(sizeof(gro_chunk) * num_threads);
    size_t chunk = (n + num_threads - 1) / num_threads, started = 0;
    for (size_t t = 0; t < num_threads; t++) {
        size_t b = t * chunk, e = b + chunk < n ? b + chunk : n;
        if (b >= n) break;
        ch[t].fn = fn;
        ch[t].user = user;
        ch[t].begin = b;
        ch[t].end = e;
        pthread_create(&th[t], NULL, gro_chunk_main, &ch[t]);
        started++;
    }
    for (size_t t = 0; t < started; t++) pthread_join(th[t], NULL);
    free(th);
    free(ch);
}

/* ---- cache -> fp32 [seq,Hkv,D] : src/llm/transformer.mm:1753-1763 ------------------------ */
void gro_cache_to_fp32(const uint16_t* cache /*[Hkv,max_seq,D]*/, float* out /*[total_seq,Hkv,D]*/,
                       int num_kv_heads, int max_seq, int total_seq, int head_dim) {
    for (int h = 0; h < num_kv_heads; h++)
        for (int s = 0; s < total_seq; s++)
            for (int d = 0; d < head_dim; d++) {
                size_t src = (size_t)h * max_seq * head_dim + (size_t)s * head_dim + d;
                size_t dst = (size_t)s * num_kv_heads * head_dim + (size_t)h * head_dim + d;
                out[dst] = gro_fp16_to_fp32(cache[src]);
            }
}

/* ---- paged addressing : include/granite/metal_compute.h:853-861,
 *      tools/test_paged_flash_attention.mm:41-49 ------------------------------------------
 * Gathers the fp16 rows of one sequence out of the pool [num_blocks*block_size, Hkv, D] in
 * logical order.  Returns the number of table entries that were out of [0,num_blocks). */
int gro_paged_gather_f16(const uint16_t* pool, const int32_t* block_table, int seq_len,
                         int block_size, int num_blocks, int num_kv_heads, int head_dim,
                         uint16_t* out /*[seq_len,Hkv,D]*/) {
    int bad = 0;
    size_t row = (size_t)num_kv_heads * head_dim;
    for (int pos = 0; pos < seq_len; pos++) {
        int logical = pos / block_size, off = pos % block_size;
        int32_t phys = block_table[logical];
        if (phys < 0 || phys >= num_blocks) {
            bad++;
            memset(out + (size_t)pos * row, 0, row * 2);
            continue;
        }
        size_t phys_pos = (size_t)phys * block_size + off;
        memcpy(out + (size_t)pos * row, pool + phys_pos * row, row * 2);
    }
    return bad;
}

void gro_f16_to_f32_array(const uint16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = gro_fp16_to_fp32(src[i]);
}

/* ---- attention core loop : src/llm/transformer.mm:1779-1840 ------------------------------ */
typedef struct {
    const float *q, *k_all, *v_all;
    float* ctx;
    int batch, seq_len, total_seq, num_heads, num_kv_heads, head_dim, start_pos;
    float scale;
} gro_attn_args;

static void gro_attn_body(size_t work_idx_u, void* user) {
    const gro_attn_args* a = (const gro_attn_args*)user;
    int work_idx = (int)work_idx_u;
    int num_heads = a->num_heads, seq_len = a->seq_len, head_dim = a->head_dim;
    int total_seq = a->total_seq, num_kv_heads = a->num_kv_heads;
    int heads_per_kv = num_heads / num_kv_heads;
    int b = work_idx / (num_heads * seq_len);
    int rem = work_idx % (num_heads * seq_len);
    int h = rem / seq_len;
    int q_pos = rem % seq_len;
    int kv_h = h / heads_per_kv;           /* :1796 */
    int abs_pos = a->start_pos + q_pos;    /* :1797 */

    float* scores = (float*)malloc(sizeof(float) * (size_t)total_seq);
    const float* q_vec = a->q + ((size_t)b * seq_len + q_pos) * num_heads * head_dim + (size_t)h * head_dim;

    for (int k_pos = 0; k_pos < total_seq; k_pos++) {  /* :1804-1815 */
        if (k_pos > abs_pos) {
            scores[k_pos] = -INFINITY;
        } else {
            const float* k_vec = a->k_all + (size_t)k_pos * num_kv_heads * head_dim + (size_t)kv_h * head_dim;
            float dot = 0;
            for (int d = 0; d < head_dim; d++) dot += q_vec[d] * k_vec[d];
            scores[k_pos] = dot * a->scale;
        }
    }
    float max_score = scores[0];  /* std::max_element, :1818 */
    for (int i = 1; i < total_seq; i++)
        if (scores[i] > max_score) max_score = scores[i];
    float sum = 0;
    for (int i = 0; i < total_seq; i++) {  /* :1820-1823 */
        scores[i] = expf(scores[i] - max_score);
        sum += scores[i];
    }
    float inv_sum = 1.0f / sum;
    for (int i = 0; i < total_seq; i++) scores[i] *= inv_sum;  /* :1825-1827 */

    float* ctx = a->ctx + ((size_t)b * seq_len + q_pos) * num_heads * head_dim + (size_t)h * head_dim;
    for (int d = 0; d < head_dim; d++) ctx[d] = 0.0f;
    for (int v_pos = 0; v_pos < total_seq; v_pos++) {  /* :1833-1839 */
        const float* v_vec = a->v_all + (size_t)v_pos * num_kv_heads * head_dim + (size_t)kv_h * head_dim;
        float w = scores[v_pos];
        for (int d = 0; d < head_dim; d++) ctx[d] += w * v_vec[d];
    }
    free(scores);
}

/* q, ctx: [batch, seq_len, Hq, D] fp32; k_all, v_all: [total_seq, Hkv, D] fp32.
 * scale <= 0 means the reference's 1/sqrt(head_dim) (:1705). */
void gro_attention(const float* q, const float* k_all, const float* v_all, float* ctx, int batch,
                   int seq_len, int total_seq, int num_heads, int num_kv_heads, int head_dim,
                   int start_pos, float scale, int num_threads) {
    gro_attn_args a = {q, k_all, v_all, ctx, batch, seq_len, total_seq, num_heads, num_kv_heads,
                       head_dim, start_pos, scale > 0 ? scale : 1.0f / sqrtf((float)head_dim)};
    gro_parallel_for((size_t)batch * num_heads * seq_len, (size_t)num_threads, gro_attn_body, &a);
}

/* ---- tree mask : src/llm/transformer.mm:823-840 ------------------------------------------
 * mask[i*n+j]=1 when node i may attend node j (self or ancestor).  The reference walks the
 * parent chain with no cycle guard; here the walk stops after n hops, which is identical for
 * every acyclic parent array (the only inputs the reference terminates on). */
void gro_tree_mask(const int32_t* parents, int n, uint8_t* mask) {
    memset(mask, 0, (size_t)n * n);
    for (int i = 0; i < n; i++) {
        mask[(size_t)i * n + i] = 1;
        int cur = parents[i];
        int hops = 0;
        while (cur >= 0 && cur < n && hops++ < n) {
            mask[(size_t)i * n + cur] = 1;
            cur = parents[cur];
        }
    }
}

/* parent range check of forward_tree (:806-813): returns 0 if every parent is in [-1,n). */
int gro_tree_validate(const int32_t* parents, int n) {
    for (int i = 0; i < n; i++)
        if (parents[i] < -1 || parents[i] >= n) return -1;
    return 0;
}

/* ---- tree attention core loop : src/llm/transformer.mm:2044-2126 ------------------------- */
typedef struct {
    const float *q, *k_cached, *v_cached, *k_tree, *v_tree;
    const uint8_t* mask;
    float* ctx;
    int batch, num_nodes, cached_len, num_heads, num_kv_heads, head_dim;
    float scale;
} gro_tree_args;

static void gro_tree_body(size_t work_idx_u, void* user) {
    const gro_tree_args* a = (const gro_tree_args*)user;
    int work_idx = (int)work_idx_u;
    int num_heads = a->num_heads, num_nodes = a->num_nodes, head_dim = a->head_dim;
    int num_kv_heads = a->num_kv_heads, cached_len = a->cached_len;
    int total_kv = cached_len + num_nodes;
    int heads_per_kv = num_heads / num_kv_heads;
    int b = work_idx / (num_heads * num_nodes);
    int rem = work_idx % (num_heads * num_nodes);
    int h = rem / num_nodes;
    int q_node = rem % num_nodes;
    int kv_h = h / heads_per_kv;

    float* scores = (float*)malloc(sizeof(float) * (size_t)total_kv);
    const float* q_vec = a->q + ((size_t)b * num_nodes + q_node) * num_heads * head_dim + (size_t)h * head_dim;

    for (int k_pos = 0; k_pos < cached_len; k_pos++) {  /* :2066-2073 */
        const float* k_vec = a->k_cached + (size_t)k_pos * num_kv_heads * head_dim + (size_t)kv_h * head_dim;
        float dot = 0;
        for (int d = 0; d < head_dim; d++) dot += q_vec[d] * k_vec[d];
        scores[k_pos] = dot * a->scale;
    }
    for (int k_node = 0; k_node < num_nodes; k_node++) {  /* :2076-2090 */
        int k_pos_in_total = cached_len + k_node;
        if (a->mask[(size_t)q_node * num_nodes + k_node]) {
            const float* k_vec = a->k_tree + ((size_t)b * num_nodes + k_node) * num_kv_heads * head_dim + (size_t)kv_h * head_dim;
            float dot = 0;
            for (int d = 0; d < head_dim; d++) dot += q_vec[d] * k_vec[d];
            scores[k_pos_in_total] = dot * a->scale;
        } else {
            scores[k_pos_in_total] = -INFINITY;
        }
    }
    float max_score = scores[0];
    for (int i = 1; i < total_kv; i++)
        if (scores[i] > max_score) max_score = scores[i];
    float sum = 0;
    for (int i = 0; i < total_kv; i++) {
        scores[i] = expf(scores[i] - max_score);
        sum += scores[i];
    }
    float inv_sum = 1.0f / sum;
    for (int i = 0; i < total_kv; i++) scores[i] *= inv_sum;

    float* ctx = a->ctx + ((size_t)b * num_nodes + q_node) * num_heads * head_dim + (size_t)h * head_dim;
    for (int d = 0; d < head_dim; d++) ctx[d] = 0.0f;
    for (int v_pos = 0; v_pos < cached_len; v_pos++) {  /* :2109-2115 */
        const float* v_vec = a->v_cached + (size_t)v_pos * num_kv_heads * head_dim + (size_t)kv_h * head_dim;
        float w = scores[v_pos];
        for (int d = 0; d < head_dim; d++) ctx[d] += w * v_vec[d];
    }
    for (int v_node = 0; v_node < num_nodes; v_node++) {  /* :2118-2125 */
        const float* v_vec = a->v_tree + ((size_t)b * num_nodes + v_node) * num_kv_heads * head_dim + (size_t)kv_h * head_dim;
        float w = scores[cached_len + v_node];
        for (int d = 0; d < head_dim; d++) ctx[d] += w * v_vec[d];
    }
    free(scores);
}

/* q, ctx: [batch, N, Hq, D]; k_cached, v_cached: [cached_len, Hkv, D] (shared by the batch, as in
 * the reference, which verifies one sequence at a time); k_tree, v_tree: [batch, N, Hkv, D];
 * mask: [N, N] bytes from gro_tree_mask. */
void gro_attention_tree(const float* q, const float* k_cached, const float* v_cached,
                        const float* k_tree, const float* v_tree, const uint8_t* mask, float* ctx,
                        int batch, int num_nodes, int cached_len, int num_heads, int num_kv_heads,
                        int head_dim, float scale, int num_threads) {
    gro_tree_args a = {q, k_cached, v_cached, k_tree, v_tree, mask, ctx, batch, num_nodes,
                       cached_len, num_heads, num_kv_heads, head_dim,
                       scale > 0 ? scale : 1.0f / sqrtf((float)head_dim)};
    gro_parallel_for((size_t)batch * num_heads * num_nodes, (size_t)num_threads, gro_tree_body, &a);
}

/* ---- batched paged decode = per sequence: gather pages -> fp32 -> attention(seq_q=1) -------
 * The reference has no CPU paged attention in the library; its batch scheduler decodes request
 * by request (src/llm/batch_scheduler.cpp:391-452).  Each sequence therefore runs the a1 loop
 * on rows fetched by the a9 addressing rule, with start_pos = len-1 so nothing is masked.
 * q, out: [B, Hq, D] fp32; pools: [num_blocks*bs, Hkv, D] fp16; tables: [B, max_blocks] int32.
 * Sequences with seq_len <= 0 get a zero output (metal_shaders_attention.h:2186 early return
 * leaves the output untouched; zero is this build's defined value).
 * stride>1 computes only sequences 0, stride, 2*stride... (bounded CPU-baseline sample). */
int gro_paged_decode_batch(const float* q, const uint16_t* k_pool, const uint16_t* v_pool,
                           const int32_t* tables, const int32_t* seq_lens, float* out, int batch,
                           int num_heads, int num_kv_heads, int head_dim, int block_size,
                           int max_blocks, int num_blocks, float scale, int num_threads,
                           int stride) {
    int bad = 0;
    size_t row = (size_t)num_kv_heads * head_dim;
    if (stride < 1) stride = 1;
    for (int b = 0; b < batch; b += stride) {
        int len = seq_lens[b];
        float* o = out + (size_t)b * num_heads * head_dim;
        if (len <= 0) {
            memset(o, 0, sizeof(float) * (size_t)num_heads * head_dim);
            continue;
        }
        uint16_t* kh = (uint16_t*)malloc(row * 2 * (size_t)len);
        uint16_t* vh = (uint16_t*)malloc(row * 2 * (size_t)len);
        float* kf = (float*)malloc(row * 4 * (size_t)len);
        float* vf = (float*)malloc(row * 4 * (size_t)len);
        const int32_t* tbl = tables + (size_t)b * max_blocks;
        bad += gro_paged_gather_f16(k_pool, tbl, len, block_size, num_blocks, num_kv_heads, head_dim, kh);
        bad += gro_paged_gather_f16(v_pool, tbl, len, block_size, num_blocks, num_kv_heads, head_dim, vh);
        gro_f16_to_f32_array(kh, kf, row * (size_t)len);
        gro_f16_to_f32_array(vh, vf, row * (size_t)len);
        gro_attention(q + (size_t)b * num_heads * head_dim, kf, vf, o, 1, 1, len, num_heads,
                      num_kv_heads, head_dim, len - 1, scale, num_threads);
        free(kh);
        free(vh);
        free(kf);
        free(vf);
    }
    return bad;
}

/* ---- operator-level SDPA : src/operators/vulkan/vulkan_operators.cpp:345-434 --------------
 * out = softmax(scale * Q Kt) V with Q [S,D], Kt [D,T] (pre-transposed), V [T,D], all fp32,
 * optional causal limit k <= q + start_pos (src/operators/metal/metal_operators.mm:1252-1253;
 * causal < 0 disables it).  Arithmetic order follows the known-answer reference in
 * tests/test_vulkan.cpp:436-474. */
void gro_sdpa_kt(const float* q, const float* kt, const float* v, float* out, int seq_q,
                 int seq_kv, int head_dim, float scale, int causal_start_pos) {
    float* scores = (float*)malloc(sizeof(float) * (size_t)seq_kv);
    for (int i = 0; i < seq_q; i++) {
        for (int j = 0; j < seq_kv; j++) {
            if (causal_start_pos >= 0 && j > i + causal_start_pos) {
                scores[j] = -INFINITY;
                continue;
            }
            float sum = 0.0f;
            for (int d = 0; d < head_dim; d++) sum += q[i * head_dim + d] * kt[d * seq_kv + j];
            scores[j] = sum * scale;
        }
        float max_val = scores[0];
        for (int j = 1; j < seq_kv; j++) max_val = scores[j] > max_val ? scores[j] : max_val;
        float sum_exp = 0.0f;
        for (int j = 0; j < seq_kv; j++) {
            scores[j] = expf(scores[j] - max_val);
            sum_exp += scores[j];
        }
        float inv_sum = 1.0f / sum_exp;
        for (int j = 0; j < seq_kv; j++) scores[j] *= inv_sum;
        for (int d = 0; d < head_dim; d++) {
            float sum = 0.0f;
            for (int j = 0; j < seq_kv; j++) sum += scores[j] * v[j * head_dim + d];
            out[i * head_dim + d] = sum;
        }
    }
    free(scores);
}

/* ---- RoPE tables : src/llm/rope.cpp:5-22 -----------------------------------------------------
 * cos/sin [max_seq, head_dim/2] in float arithmetic throughout: freq = 1 / pow(theta, 2i/head_dim),
 * angle = pos * freq.  The reference calls the float overloads of std::pow / std::cos / std::sin. */
void gro_rope_table(int max_seq, int head_dim, float theta, float* cos_out, float* sin_out) {
    int half_dim = head_dim / 2;
    for (int pos = 0; pos < max_seq; pos++)
        for (int i = 0; i < half_dim; i++) {
            float freq = 1.0f / powf(theta, (float)(2 * i) / head_dim);
            float angle = (float)pos * freq;
            cos_out[(size_t)pos * half_dim + i] = cosf(angle);
            sin_out[(size_t)pos * half_dim + i] = sinf(angle);
        }
}

/* ---- RoPE rotation : src/llm/rope.cpp:52-86 --------------------------------------------------
 * x [seq_len, num_heads, head_dim] rotated in place: adjacent pairs (2i, 2i+1), position
 * start_pos + s, products rounded separately (no fused multiply-add).  Returns -1 when a
 * position falls outside the table (rope.cpp:34-38 rejects the call). */
int gro_rope_apply(float* x, int seq_len, int num_heads, int head_dim, int start_pos,
                   const float* cos_t, const float* sin_t, int table_len) {
    int half_dim = head_dim / 2;
    if (start_pos < 0 || start_pos + seq_len > table_len) return -1;
    for (int s = 0; s < seq_len; s++) {
        int pos = start_pos + s;
        for (int h = 0; h < num_heads; h++) {
            float* p = x + ((size_t)s * num_heads + h) * head_dim;
            for (int i = 0; i < half_dim; i++) {
                float c = cos_t[(size_t)pos * half_dim + i], sn = sin_t[(size_t)pos * half_dim + i];
                float x0 = p[2 * i], x1 = p[2 * i + 1];
                p[2 * i] = x0 * c - x1 * sn;
                p[2 * i + 1] = x0 * sn + x1 * c;
            }
        }
    }
    return 0;
}

/* ---- RoPE + cache write of a batch of new tokens ----------------------------------------------
 * The step before attention in the paged decode / prefill flow (src/llm/transformer.mm:2975-2986):
 * rotate Q and K (rope.cpp:52-86), narrow K and V to fp16 with the truncating cast
 * (transformer.mm:1681-1691 -> math_ops.cpp:45-54) and store them at the new positions through
 * the block table (metal_compute.h:853-861).  q [batch, new_len, Hq, D] is rotated in place;
 * k, v [batch, new_len, Hkv, D] are left untouched; sequence b's tokens take positions
 * positions[b] .. positions[b] + new_len - 1.  Returns the number of tokens that could not be
 * written (position outside the RoPE table, table entry outside the pool). */
int gro_rope_paged_append(float* q, const float* k, const float* v, const float* cos_t,
                          const float* sin_t, int table_len, uint16_t* k_pool, uint16_t* v_pool,
                          const int32_t* block_tables, const int32_t* positions, int batch,
                          int new_len, int num_heads, int num_kv_heads, int head_dim,
                          int block_size, int max_blocks, int num_blocks) {
    int bad = 0;
    size_t krow = (size_t)num_kv_heads * head_dim;
    float* kr = (float*)malloc(krow * sizeof(float));
    for (int b = 0; b < batch; b++)
        for (int s = 0; s < new_len; s++) {
            int pos = positions[b] + s;
            size_t row = (size_t)b * new_len + s;
            int logical = pos / block_size;
            if (pos < 0 || pos >= table_len || logical >= max_blocks) { bad++; continue; }
            int32_t phys = block_tables[(size_t)b * max_blocks + logical];
            if (phys < 0 || phys >= num_blocks) { bad++; continue; }
            if (q) gro_rope_apply(q + row * num_heads * head_dim, 1, num_heads, head_dim, pos, cos_t, sin_t, table_len);
            memcpy(kr, k + row * krow, krow * sizeof(float));
            gro_rope_apply(kr, 1, num_kv_heads, head_dim, pos, cos_t, sin_t, table_len);
            size_t dst = ((size_t)phys * block_size + pos % block_size) * krow;
            for (size_t i = 0; i < krow; i++) {
                k_pool[dst + i] = gro_fp32_to_fp16(kr[i]);
                v_pool[dst + i] = gro_fp32_to_fp16(v[row * krow + i]);
            }
        }
    free(kr);
    return bad;
}

/* ---- tree commit ---------------------------------------------------------------------------------
 * Keeps the accepted path of a verified tree: row accepted[b][j] of tree K/V
 * [batch, Hkv, num_nodes, D] (fp16 bits) goes to position cache_lens[b] + j of sequence b's paged
 * cache (addressing rule metal_compute.h:853-861); the caller then truncates the sequence to
 * cache_lens[b] + num_accepted[b] as src/llm/speculative_runner.cpp:871-882 does for the
 * contiguous cache.  Returns the number of rows that could not be written. */
int gro_tree_commit(const uint16_t* k_tree, const uint16_t* v_tree, uint16_t* k_pool,
                    uint16_t* v_pool, const int32_t* block_tables, const int32_t* cache_lens,
                    const int32_t* accepted, const int32_t* num_accepted, int batch, int num_nodes,
                    int max_accepted, int num_kv_heads, int head_dim, int block_size,
                    int max_blocks, int num_blocks) {
    int bad = 0;
    for (int b = 0; b < batch; b++) {
        int n_acc = num_accepted[b];
        if (n_acc < 0 || n_acc > max_accepted) { bad++; continue; }
        for (int j = 0; j < n_acc; j++) {
            int node = accepted[(size_t)b * max_accepted + j];
            int pos = cache_lens[b] + j;
            int logical = pos / block_size;
            if (node < 0 || node >= num_nodes || pos < 0 || logical >= max_blocks) { bad++; continue; }
            int32_t phys = block_tables[(size_t)b * max_blocks + logical];
            if (phys < 0 || phys >= num_blocks) { bad++; continue; }
            for (int h = 0; h < num_kv_heads; h++) {
                size_t src = (((size_t)b * num_kv_heads + h) * num_nodes + node) * head_dim;
                size_t dst = (((size_t)phys * block_size + pos % block_size) * num_kv_heads + h) * head_dim;
                memcpy(k_pool + dst, k_tree + src, (size_t)head_dim * 2);
                memcpy(v_pool + dst, v_tree + src, (size_t)head_dim * 2);
            }
        }
    }
    return bad;
}
