/*
 * vvb_ops.c -- C11 host layer of libvvb200: the exported entry points.
 *
 * Each entry validates its arguments the way the reference's launchers do
 * (NULL tensors -> VV_ERR_NULL_PTR: src/cuda/rmsnorm.cu:86, rope.cu:93,
 * swiglu.cu:83, embedding.cu:63; a failed launch -> VV_ERR_CUDA_LAUNCH), adds
 * the checks the reference leaves to luck (negative sizes, products that
 * overflow), and hands the work to the CUDA translation units through the
 * launch interface in csrc/vvb_launch.h. No CUDA call is made here except
 * through that interface; there is no CPU implementation of any op in this
 * library.
 */
#include "vvb200.h"
#include "../csrc/vvb_launch.h"

#include <limits.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>

#define VVB_VERSION "0.1.0"

static vv_status_t from_cuda(int err) { return err == 0 ? VV_OK : VV_ERR_CUDA_LAUNCH; }

/* ------------------------------------------------------------------ group 1 */

vv_status_t vv_embedding_dev(const void* table, const int32_t* ids, void* output,
                             int seq_len, int hidden_size, void* stream) {
    if (!table || !ids || !output) return VV_ERR_NULL_PTR;
    if (seq_len < 0 || hidden_size < 0) return VV_ERR_INVALID_ARG;
    if (seq_len == 0 || hidden_size == 0) return VV_OK;
    return from_cuda(vvbk_row_norm(table, NULL, ids, 0, output, NULL, NULL,
                                   seq_len, hidden_size, 0.0f, stream));
}

vv_status_t vv_rmsnorm_dev(const void* input, const void* weight, void* output,
                           int seq_len, int hidden_size, float eps, void* stream) {
    if (!input || !weight || !output) return VV_ERR_NULL_PTR;
    if (seq_len < 0 || hidden_size < 0) return VV_ERR_INVALID_ARG;
    if (seq_len == 0 || hidden_size == 0) return VV_OK;
    return from_cuda(vvbk_row_norm(input, NULL, NULL, 0, NULL, weight, output,
                                   seq_len, hidden_size, eps, stream));
}

/* freq_i = powf(theta, -2i/head_dim): the very expression of the reference's
 * CPU kernel (src/cpu/cpu_kernels.c:1468), evaluated by the host libm so the
 * device sees the same 32-bit values the CPU path uses. */
static void fill_inv_freq(float* out, int head_dim, float theta) {
    for (int i = 0; i < head_dim / 2; i++)
        out[i] = powf(theta, -2.0f * (float)i / (float)head_dim);
}

vv_status_t vvb_rope_qk_dev(void* q, void* k, int rows, int n_q_heads, int n_kv_heads,
                            int head_dim, int position_offset, const int* d_position,
                            float theta, void* stream) {
    if (rows < 0 || n_q_heads < 0 || n_kv_heads < 0 || head_dim < 0) return VV_ERR_INVALID_ARG;
    if ((n_q_heads > 0 && !q) || (n_kv_heads > 0 && !k)) return VV_ERR_NULL_PTR;
    if (rows == 0 || n_q_heads + n_kv_heads == 0 || head_dim < 2) return VV_OK;
    if (head_dim / 2 > VVB_ROPE_MAX_HALF) return VV_ERR_UNSUPPORTED;
    float inv_freq[VVB_ROPE_MAX_HALF];
    fill_inv_freq(inv_freq, head_dim, theta);
    return from_cuda(vvbk_rope(q, k, rows, n_q_heads, n_kv_heads, head_dim,
                               position_offset, d_position, inv_freq, stream));
}

static vv_status_t kv_rotate_common(void* x, int n_heads, int head_dim, int rows, int inverse, void* stream) {
    if (!x) return VV_ERR_NULL_PTR;
    if (n_heads < 0 || rows < 0 || head_dim <= 0) return VV_ERR_INVALID_ARG;
    if (head_dim != 128) return VV_ERR_UNSUPPORTED;       /* as the reference (src/cuda/kv_quant.cu:477) */
    if (((uintptr_t)x & 1u) != 0) return VV_ERR_INVALID_ARG;
    const size_t nvec = (size_t)rows * (size_t)n_heads;
    if (nvec == 0) return VV_OK;
    return from_cuda(vvbk_kv_rotate(x, nvec, inverse, stream));
}

vv_status_t vvb_kv_rotate_dev(void* x, int n_heads, int head_dim, int rows, void* stream) {
    return kv_rotate_common(x, n_heads, head_dim, rows, 0, stream);
}

vv_status_t vvb_kv_unrotate_dev(void* x, int n_heads, int head_dim, int rows, void* stream) {
    return kv_rotate_common(x, n_heads, head_dim, rows, 1, stream);
}

vv_status_t vvb_kv_append_dev(const vvb_kv_append_t* a, void* stream) {
    if (!a) return VV_ERR_NULL_PTR;
    if (!a->q || !a->k || !a->v || !a->k_store || !a->v_store) return VV_ERR_NULL_PTR;
    if (a->rows < 0 || a->n_q_heads <= 0 || a->n_kv_heads <= 0 || a->head_dim <= 0 || a->cache_offset < 0)
        return VV_ERR_INVALID_ARG;
    /* the reference's vv_kv_format_t: 0 FP16, 1 FP8 E4M3, 2 FP8 E5M2 (its own
     * FP8 store takes head_dim 128 only, src/cuda/kv_quant.cu:527; the byte
     * layout is defined for any head_dim and this kernel takes multiples of
     * 16); 3..6 the TurboQuant formats, defined for head_dim 128. */
    if (a->kv_format < VVB_KV_FP16 || a->kv_format > VVB_KV_TQ1_5) return VV_ERR_UNSUPPORTED;
    const int tq = a->kv_format >= VVB_KV_TQ4;
    if (tq && (!a->k_meta || !a->v_meta)) return VV_ERR_NULL_PTR;
    if (tq && a->head_dim != 128) return VV_ERR_UNSUPPORTED;       /* as the reference's store: src/cuda/kv_quant.cu:527 */
    if (a->rows == 0) return VV_OK;
    if (a->head_dim / 2 > VVB_ROPE_MAX_HALF) return VV_ERR_UNSUPPORTED;
    float inv_freq[VVB_ROPE_MAX_HALF];
    fill_inv_freq(inv_freq, a->head_dim, a->theta);
    const int err = vvbk_rope_append(a->q, a->k, a->v, a->q_bias, a->k_bias, a->v_bias, a->k_store, a->v_store,
                                     a->rows, a->n_q_heads, a->n_kv_heads, a->head_dim, a->position_offset,
                                     a->cache_offset, a->d_position, inv_freq, a->keep_k, a->kv_format,
                                     a->kv_format == VVB_KV_FP16 ? NULL : a->k_ref, a->page_table,
                                     tq ? a->k_meta : NULL, tq ? a->v_meta : NULL, stream);
    if (err == 801) return VV_ERR_UNSUPPORTED;   /* cudaErrorNotSupported: not vectorisable */
    return from_cuda(err);
}

static vv_status_t rope_qk_append(void* q, void* k, const void* v,
                                  const void* q_bias, const void* k_bias, const void* v_bias,
                                  void* k_cache, void* v_cache, const void* k_ref,
                                  int rows, int n_q_heads, int n_kv_heads, int head_dim,
                                  int position_offset, int cache_offset, const int* d_position,
                                  float theta, int kv_format, int keep_k, void* stream) {
    const vvb_kv_append_t a = {q, k, v, q_bias, k_bias, v_bias, k_cache, v_cache, k_ref, NULL, d_position,
                               rows, n_q_heads, n_kv_heads, head_dim, position_offset, cache_offset,
                               theta, kv_format, keep_k, NULL, NULL};
    return vvb_kv_append_dev(&a, stream);
}

vv_status_t vvb_rope_qk_append_dev(void* q, void* k, const void* v,
                                   const void* q_bias, const void* k_bias, const void* v_bias,
                                   void* k_cache, void* v_cache,
                                   int rows, int n_q_heads, int n_kv_heads, int head_dim,
                                   int position_offset, int cache_offset, const int* d_position,
                                   float theta, int keep_k, void* stream) {
    return rope_qk_append(q, k, v, q_bias, k_bias, v_bias, k_cache, v_cache, NULL, rows, n_q_heads,
                          n_kv_heads, head_dim, position_offset, cache_offset, d_position, theta,
                          0, keep_k, stream);
}

vv_status_t vvb_rope_qk_append_fp8_dev(void* q, void* k, const void* v,
                                       const void* q_bias, const void* k_bias, const void* v_bias,
                                       void* k_store, void* v_store, const void* k_ref,
                                       int rows, int n_q_heads, int n_kv_heads, int head_dim,
                                       int position_offset, int cache_offset, const int* d_position,
                                       float theta, int kv_format, int keep_k, void* stream) {
    /* the reference's vv_kv_format_t: 1 = FP8 E4M3, 2 = FP8 E5M2 (its own FP8
     * store takes head_dim 128 only, src/cuda/kv_quant.cu:527; the byte layout
     * is defined for any head_dim and this kernel takes multiples of 16) */
    if (kv_format != VVB_KV_FP8_E4M3 && kv_format != VVB_KV_FP8_E5M2) return VV_ERR_UNSUPPORTED;
    return rope_qk_append(q, k, v, q_bias, k_bias, v_bias, k_store, v_store, k_ref, rows, n_q_heads,
                          n_kv_heads, head_dim, position_offset, cache_offset, d_position, theta,
                          kv_format, keep_k, stream);
}

vv_status_t vv_rope_dev(void* x, int seq_len, int n_heads, int head_dim,
                        int position_offset, const int* d_position, float theta,
                        void* stream) {
    if (!x) return VV_ERR_NULL_PTR;
    return vvb_rope_qk_dev(x, NULL, seq_len, n_heads, 0, head_dim, position_offset,
                           d_position, theta, stream);
}

vv_status_t vvb_swiglu_dev(const void* gate, const void* up, void* output,
                           size_t n_elements, void* stream) {
    if (!gate || !up || !output) return VV_ERR_NULL_PTR;
    if (n_elements == 0) return VV_OK;
    return from_cuda(vvbk_swiglu(gate, up, output, n_elements, stream));
}

vv_status_t vv_swiglu_dev(const void* gate, const void* up, void* output,
                          int n_elements, void* stream) {
    if (!gate || !up || !output) return VV_ERR_NULL_PTR;
    if (n_elements < 0) return VV_ERR_INVALID_ARG;
    return vvb_swiglu_dev(gate, up, output, (size_t)n_elements, stream);
}

vv_status_t vv_swiglu_fused_dev(const void* gate_up, void* output, int rows,
                                int inter, void* stream) {
    if (!gate_up || !output) return VV_ERR_NULL_PTR;
    if (rows < 0 || inter < 0) return VV_ERR_INVALID_ARG;
    if (rows == 0 || inter == 0) return VV_OK;
    return from_cuda(vvbk_swiglu_fused(gate_up, output, rows, inter, stream));
}

vv_status_t vvb_residual_add_dev(void* x, const void* y, size_t total, void* stream) {
    if (!x || !y) return VV_ERR_NULL_PTR;
    if (total == 0) return VV_OK;
    return from_cuda(vvbk_residual_add(x, y, total, stream));
}

vv_status_t vv_residual_add_dev(void* x, const void* y, int total, void* stream) {
    if (!x || !y) return VV_ERR_NULL_PTR;
    if (total < 0) return VV_ERR_INVALID_ARG;
    return vvb_residual_add_dev(x, y, (size_t)total, stream);
}

vv_status_t vv_bias_add_dev(void* output, const void* bias, int M, int N, void* stream) {
    if (!output || !bias) return VV_ERR_NULL_PTR;
    if (M < 0 || N < 0) return VV_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return VV_OK;
    return from_cuda(vvbk_bias_add(output, bias, M, N, stream));
}

vv_status_t vv_fp32_to_fp16_dev(const void* in_fp32, void* out_fp16, int n, void* stream) {
    if (!in_fp32 || !out_fp16) return VV_ERR_NULL_PTR;
    if (n < 0) return VV_ERR_INVALID_ARG;
    if (n == 0) return VV_OK;
    return from_cuda(vvbk_f32_to_f16(in_fp32, out_fp16, (size_t)n, stream));
}

vv_status_t vv_fp16_to_fp32_dev(const void* in_fp16, void* out_fp32, int n, void* stream) {
    if (!in_fp16 || !out_fp32) return VV_ERR_NULL_PTR;
    if (n < 0) return VV_ERR_INVALID_ARG;
    if (n == 0) return VV_OK;
    return from_cuda(vvbk_f16_to_f32(in_fp16, out_fp32, (size_t)n, stream));
}

/* ------------------------------------------------------------------ group 2 */

vv_status_t vvb_add_rmsnorm_dev(void* hidden_inout, const void* delta,
                                const void* weight, void* normed_out,
                                int rows, int hidden_size, float eps, void* stream) {
    if (!hidden_inout || !weight || !normed_out) return VV_ERR_NULL_PTR;
    if (rows < 0 || hidden_size < 0) return VV_ERR_INVALID_ARG;
    if (rows == 0 || hidden_size == 0) return VV_OK;
    /* With a delta the updated row is written back over hidden; without one
     * hidden is only read. */
    return from_cuda(vvbk_row_norm(hidden_inout, delta, NULL, 0,
                                   delta ? hidden_inout : NULL, weight, normed_out,
                                   rows, hidden_size, eps, stream));
}

vv_status_t vvb_embedding_rmsnorm_dev(const void* table, const int32_t* ids,
                                      void* hidden_out, const void* weight,
                                      void* normed_out, int rows, int hidden_size,
                                      int vocab, float eps, void* stream) {
    if (!table || !ids || !hidden_out) return VV_ERR_NULL_PTR;
    if (normed_out && !weight) return VV_ERR_NULL_PTR;
    if (rows < 0 || hidden_size < 0) return VV_ERR_INVALID_ARG;
    if (rows == 0 || hidden_size == 0) return VV_OK;
    return from_cuda(vvbk_row_norm(table, NULL, ids, vocab, hidden_out, weight, normed_out,
                                   rows, hidden_size, eps, stream));
}

vv_status_t vvb_layer_chain_dev(const vvb_layer_chain_t* c, void* stream) {
    if (!c) return VV_ERR_NULL_PTR;
    if (c->rows < 0 || c->hidden_size < 0 || c->inter < 0 || c->n_q_heads < 0 ||
        c->n_kv_heads < 0 || c->head_dim < 0)
        return VV_ERR_INVALID_ARG;
    if (c->rows == 0) return VV_OK;      /* nothing to do, whatever the pointers are */
    /* The three operations touch disjoint tensors: when the shapes allow it
     * they go out as one grid (csrc/chain.cu), else as three launches. */
    if (c->rows > 0 && c->hidden && c->delta && c->norm_w && c->normed && c->q && c->k &&
        c->gate && c->up && c->head_dim >= 2 && c->head_dim / 2 <= VVB_ROPE_MAX_HALF) {
        float inv_freq[VVB_ROPE_MAX_HALF];
        fill_inv_freq(inv_freq, c->head_dim, c->theta);
        const int err = vvbk_layer_chain(c->hidden, c->delta, c->norm_w, c->normed, c->q, c->k,
                                         c->gate, c->up, c->rows, c->hidden_size, c->n_q_heads,
                                         c->n_kv_heads, c->head_dim, c->inter, c->position_offset,
                                         inv_freq, c->eps, stream);
        if (err != 801 /* cudaErrorNotSupported: shapes do not fit the single launch */)
            return from_cuda(err);
    }
    vv_status_t st = vvb_add_rmsnorm_dev(c->hidden, c->delta, c->norm_w, c->normed,
                                         c->rows, c->hidden_size, c->eps, stream);
    if (st != VV_OK) return st;
    st = vvb_rope_qk_dev(c->q, c->k, c->rows, c->n_q_heads, c->n_kv_heads, c->head_dim,
                         c->position_offset, NULL, c->theta, stream);
    if (st != VV_OK) return st;
    return vvb_swiglu_dev(c->gate, c->up, c->gate, (size_t)c->rows * (size_t)c->inter, stream);
}

/* --------------------------------------------------- int8 activation quantizers */

/* The reference's argument checks, in its order (src/cuda/act_quant.cu:222-233):
 * NULL tensors, then M/K <= 0, then K % 32 / K too wide. */
static vv_status_t q8_check(int M, int K, const void* a, const int8_t* xq, const float* sx) {
    if (!a || !xq || !sx) return VV_ERR_NULL_PTR;
    if (M <= 0 || K <= 0) return VV_ERR_INVALID_ARG;
    if ((K & 31) != 0 || K > VV_ACT_QUANT_MAX_K) return VV_ERR_UNSUPPORTED;
    return VV_OK;
}

static int q8_aligned(const void* p) { return ((uintptr_t)p & 15u) == 0; }

vv_status_t vv_act_quant_dev(const void* x, int M, int K, int layout,
                             int8_t* xq, float* sx, int32_t* xsum, void* stream) {
    vv_status_t st = q8_check(M, K, x, xq, sx);
    if (st != VV_OK) return st;
    if (layout < 0 || layout >= VV_Q8_LAYOUT_COUNT) return VV_ERR_INVALID_ARG;
    if (!q8_aligned(x) || !q8_aligned(xq)) return VV_ERR_UNSUPPORTED;
    return from_cuda(vvbk_act_quant(0, x, NULL, NULL, NULL, M, K, 0.0f, layout, xq, sx, xsum, stream));
}

vv_status_t vvb_add_rmsnorm_q8_dev(void* hidden_inout, const void* delta, const void* weight,
                                   int M, int K, float eps, int layout,
                                   int8_t* xq, float* sx, int32_t* xsum, void* stream) {
    vv_status_t st = q8_check(M, K, hidden_inout, xq, sx);
    if (st != VV_OK) return st;
    if (!weight) return VV_ERR_NULL_PTR;
    if (layout < 0 || layout >= VV_Q8_LAYOUT_COUNT) return VV_ERR_INVALID_ARG;
    if (K < VV_ACT_QUANT_MIN_K) return VV_ERR_UNSUPPORTED;
    if (!q8_aligned(hidden_inout) || !q8_aligned(delta) || !q8_aligned(weight) || !q8_aligned(xq))
        return VV_ERR_UNSUPPORTED;
    return from_cuda(vvbk_act_quant(1, hidden_inout, delta, weight, delta ? hidden_inout : NULL,
                                    M, K, eps, layout, xq, sx, xsum, stream));
}

vv_status_t vv_rmsnorm_q8_dev(const void* x, const void* weight, int M, int K, float eps,
                              int layout, int8_t* xq, float* sx, int32_t* xsum, void* stream) {
    /* no addend: the row is only read */
    return vvb_add_rmsnorm_q8_dev((void*)(uintptr_t)x, NULL, weight, M, K, eps, layout, xq, sx, xsum, stream);
}

vv_status_t vv_swiglu_q8_dev(const void* gate, const void* up, int M, int K, int layout,
                             int8_t* xq, float* sx, int32_t* xsum, void* stream) {
    vv_status_t st = q8_check(M, K, gate, xq, sx);
    if (st != VV_OK) return st;
    if (!up) return VV_ERR_NULL_PTR;
    if (layout < 0 || layout >= VV_Q8_LAYOUT_COUNT) return VV_ERR_INVALID_ARG;
    if (!q8_aligned(gate) || !q8_aligned(up) || !q8_aligned(xq)) return VV_ERR_UNSUPPORTED;
    return from_cuda(vvbk_act_quant(2, gate, up, NULL, NULL, M, K, 0.0f, layout, xq, sx, xsum, stream));
}

vv_status_t vv_col_absmax_dev(const void* x, int M, int K, float* acc, void* stream) {
    if (!x || !acc) return VV_ERR_NULL_PTR;
    if (M <= 0 || K <= 0) return VV_ERR_INVALID_ARG;
    return from_cuda(vvbk_col_absmax(x, M, K, acc, stream));
}

/* -------------------------------------------------------------------- LM head */

#define VVB_ARGMAX_PARTIALS 256   /* the reference's scratch size: src/cuda/lm_head.cu:171 */

vv_status_t vv_lm_head_gemv_dev(const void* x, const void* W, void* logits, int V, int K, void* stream) {
    if (!x || !W || !logits) return VV_ERR_NULL_PTR;
    if (V < 0 || K < 0) return VV_ERR_INVALID_ARG;
    if (V == 0) return VV_OK;
    return from_cuda(vvbk_lm_head(x, NULL, 0.0f, W, (float*)logits, NULL, NULL, NULL, V, K, stream));
}

vv_status_t vv_argmax_dev(const void* logits, int V, void* scratch_v, void* scratch_i,
                          void* out_token, void* out_value, void* stream) {
    if (!logits || !scratch_v || !scratch_i || !out_token) return VV_ERR_NULL_PTR;
    if (V <= 0) return VV_ERR_INVALID_ARG;
    int err = vvbk_argmax_logits((const float*)logits, V, (float*)scratch_v, (int*)scratch_i,
                                 VVB_ARGMAX_PARTIALS, stream);
    if (err == 0)
        err = vvbk_argmax_reduce((const float*)scratch_v, (const int*)scratch_i, VVB_ARGMAX_PARTIALS,
                                 (int*)out_token, (float*)out_value, stream);
    return from_cuda(err);
}

size_t vvb_lm_head_scratch_bytes(int V) {
    return V > 0 ? (size_t)vvbk_lm_head_partials(V) * (sizeof(float) + sizeof(int)) : 0;
}

vv_status_t vvb_lm_head_argmax_dev(const void* x, const void* final_norm_w, float eps, const void* W,
                                   int V, int K, void* logits, void* scratch, size_t scratch_bytes,
                                   int32_t* out_token, float* out_value, void* stream) {
    if (!x || !W || !scratch || !out_token) return VV_ERR_NULL_PTR;
    if (V <= 0 || K <= 0) return VV_ERR_INVALID_ARG;
    if (scratch_bytes < vvb_lm_head_scratch_bytes(V) || ((uintptr_t)scratch & 3u)) return VV_ERR_INVALID_ARG;
    const int cap = vvbk_lm_head_partials(V);
    float* part_v = (float*)scratch;
    int* part_i = (int*)(part_v + cap);
    int n = 0;
    int err = vvbk_lm_head(x, final_norm_w, eps, W, (float*)logits, part_v, part_i, &n, V, K, stream);
    if (err == 801) return VV_ERR_UNSUPPORTED;   /* cudaErrorNotSupported: K % 8, K > 11264 or alignment */
    if (err == 0) err = vvbk_argmax_reduce(part_v, part_i, n, (int*)out_token, out_value, stream);
    return from_cuda(err);
}

/* ------------------------------------------------------------ introspection */

const char* vvb_version(void) { return "vvb200 " VVB_VERSION " sm_100a"; }

const char* vvb_status_string(int status) {
    switch (status) {
        case VV_OK: return "ok";
        case VV_ERR_INVALID_ARG: return "invalid argument";
        case VV_ERR_NULL_PTR: return "null pointer";
        case VV_ERR_OUT_OF_MEMORY: return "out of host memory";
        case VV_ERR_UNSUPPORTED: return "unsupported shape";
        case VV_ERR_OVERFLOW: return "size overflow";
        case VV_ERR_CUDA: return "CUDA runtime error";
        case VV_ERR_CUDA_OOM: return "out of device memory";
        case VV_ERR_CUDA_LAUNCH: return "kernel launch failed";
        default: return "unknown status";
    }
}

uint64_t vvb_launch_count(void) { return vvbk_launch_count(); }
