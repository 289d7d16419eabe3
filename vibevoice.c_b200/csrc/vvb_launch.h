/*
 * vvb_launch.h -- the thin C-ABI between the C11 host layer (the host/ directory) and
 * the CUDA translation units (the csrc/ directory). Each function enqueues exactly the
 * kernels named on `stream` of the current device and returns the
 * cudaError_t of the launch as an int (0 = cudaSuccess). Arguments were
 * validated by the caller; these do no checking beyond choosing a kernel
 * variant from sizes and alignment.
 */
#ifndef VVB_LAUNCH_H
#define VVB_LAUNCH_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VVB_ROPE_MAX_HALF 256 /* head_dim/2 entries carried in kernel parameters */

/* Row kernels (csrc/row_norm.cu).
 *   src_rows : [rows, hidden] FP16 (or the table when ids != NULL)
 *   delta    : NULL or [rows, hidden]
 *   ids      : NULL or int32[rows] (gather source rows from src_rows)
 *   row_out  : NULL or [rows, hidden]: receives the gathered / summed row
 *   weight   : [hidden] (ignored when normed == NULL)
 *   normed   : NULL or [rows, hidden] */
int vvbk_row_norm(const void* src_rows, const void* delta, const int32_t* ids, int vocab,
                  void* row_out, const void* weight, void* normed,
                  int rows, int hidden, float eps, void* stream);

/* RoPE (csrc/rope.cu). inv_freq holds head_dim/2 host-computed floats. */
int vvbk_rope(void* q, void* k, int rows, int n_q_heads, int n_kv_heads, int head_dim,
              int position_offset, const int* d_position, const float* inv_freq, void* stream);

/* Bias add + RoPE + KV-cache append in one launch (csrc/rope_append.cu).
 * Returns cudaErrorNotSupported (801) without launching when head_dim % 16 != 0
 * or a pointer is not 16-byte aligned. kv_format: 0 raw FP16 cache, 1 / 2 the
 * reference's software FP8 E4M3 / E5M2 bytes (one per element); k_ref (FP8
 * only, may be null): FP16 [n_kv_heads * head_dim] subtracted from K first.
 * page_table (may be null): device ints, one per 64-position page of the
 * logical sequence, giving the page's index in the cache arrays. kv_format
 * 3..6: the TurboQuant formats (head_dim 128 only); k_meta / v_meta then receive
 * one FP16 RMS per stored vector, [max_len, n_kv_heads]. */
int vvbk_rope_append(void* q, void* k, const void* v,
                     const void* q_bias, const void* k_bias, const void* v_bias,
                     void* k_cache, void* v_cache,
                     int rows, int n_q_heads, int n_kv_heads, int head_dim,
                     int position_offset, int cache_offset, const int* d_position,
                     const float* inv_freq, int keep_k, int kv_format, const void* k_ref,
                     const int* page_table, void* k_meta, void* v_meta, void* stream);

/* The TurboQuant caches' rotation of Q / un-rotation of the attention output
 * (csrc/kv_rotate.cu): nvec head vectors of 128 halves, in place. */
int vvbk_kv_rotate(void* x, size_t nvec, int inverse, void* stream);

/* SwiGLU (csrc/swiglu.cu). Flat: gate/up/out of n elements. Fused: rows of
 * [gate | up] with 2*inter halves per row. */
int vvbk_swiglu(const void* gate, const void* up, void* out, size_t n, void* stream);
int vvbk_swiglu_fused(const void* gate_up, void* out, int rows, int inter, void* stream);

/* The whole layer chain in one launch (csrc/chain.cu). Returns
 * cudaErrorNotSupported (801) without launching when the shapes or alignments
 * do not fit that form. */
int vvbk_layer_chain(void* hidden, const void* delta, const void* weight, void* normed,
                     void* q, void* k, void* gate, const void* up,
                     int rows, int hidden_size, int n_q_heads, int n_kv_heads, int head_dim,
                     int inter, int position_offset, const float* inv_freq, float eps, void* stream);

/* Per-token int8 activation quantizers (csrc/act_quant.cu).
 *   mode 0: a = x                         -> xq, sx, xsum
 *   mode 1: RMSNorm of a (+ delta b, the updated row written to row_out) -> ...
 *   mode 2: SwiGLU of a = gate, b = up    -> ...
 * K a multiple of 32, pointers 16-byte aligned, layout 0..3. */
int vvbk_act_quant(int mode, const void* a, const void* b, const void* weight, void* row_out,
                   int M, int K, float eps, int layout,
                   int8_t* xq, float* sx, int32_t* xsum, void* stream);

/* acc[k] = max(acc[k], max_m |x[m,k]|), x FP16 [M,K], acc FP32 [K] (csrc/act_quant.cu). */
int vvbk_col_absmax(const void* x, int M, int K, float* acc, void* stream);

/* LM head (csrc/lm_head.cu). vvbk_lm_head: logits (may be NULL) and/or per-CTA
 * argmax partials (may be NULL; at most vvbk_lm_head_partials(V) entries each,
 * the number written is returned in *n_partials);
 * norm_w != NULL applies the final RMSNorm to x first. Returns
 * cudaErrorNotSupported (801) when K / alignment do not fit the fast form and
 * anything but plain logits was asked for. */
int vvbk_lm_head_partials(int V);
int vvbk_lm_head(const void* x, const void* norm_w, float eps, const void* W, float* logits,
                 float* part_v, int* part_i, int* n_partials, int V, int K, void* stream);
int vvbk_argmax_logits(const float* logits, int V, float* part_v, int* part_i, int nparts, void* stream);
int vvbk_argmax_reduce(const float* part_v, const int* part_i, int n, int* out_token, float* out_value,
                       void* stream);

/* Flat elementwise ops (csrc/elementwise.cu). */
int vvbk_residual_add(void* x, const void* y, size_t n, void* stream);
int vvbk_bias_add(void* out, const void* bias, int M, int N, void* stream);
int vvbk_f32_to_f16(const void* in, void* out, size_t n, void* stream);
int vvbk_f16_to_f32(const void* in, void* out, size_t n, void* stream);

/* Launches enqueued so far in this process. */
uint64_t vvbk_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif
