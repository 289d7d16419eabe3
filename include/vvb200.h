/**
 * @file vvb200.h
 * @brief C-ABI of libvvb200: the Qwen2-7B decoder's per-token layer kernels
 *        (residual add + RMSNorm, RoPE on Q/K, SwiGLU, embedding gather),
 *        hand-written CUDA for sm_100a behind vibevoice.c's device op names.
 *
 * The first group of functions has exactly the names, argument lists and
 * argument meaning of the reference's accelerator op set for this path, so a
 * build of the reference that leaves out its own rmsnorm.cu / rope.cu /
 * swiglu.cu / embedding.cu / conv_vae.cu / act_quant.cu / lm_head.cu and
 * links this library resolves the same symbols (the reference picks its
 * backend at link time:
 * include/vibevoice/device.h:11-14). The second group (vvb_*) is additive:
 * fused forms that save HBM passes, a host-buffer pipeline, and the row
 * partition used to shard tokens over the GPUs of one box (the host-buffer
 * pipeline and its multi-GPU form own streams, staging buffers and threads:
 * they block and are not capturable, as their declarations say).
 *
 * Conventions (those of include/vibevoice/device.h:16-21):
 *   - every tensor pointer is caller-owned DEVICE memory of the current
 *     device, FP16 (IEEE binary16) unless the name says otherwise, row-major,
 *     contiguous; ids are int32 in device memory;
 *   - `void* stream` is a cudaStream_t; NULL is the legacy default stream;
 *   - work is enqueued and the call returns; nothing synchronises, allocates,
 *     frees or keeps a pointer, so every *_dev call may be stream-captured;
 *   - kernels are launched with the programmatic stream serialization
 *     attribute and wait for the preceding grid at their first instruction:
 *     ordering on the stream is that of an ordinary launch (also against
 *     kernels that are not this library's), only launch latency overlaps;
 *     captured, a kernel-to-kernel dependency becomes a programmatic graph
 *     edge (CUDA 12.3 or later);
 *   - calls are re-entrant: no file-scope mutable state. The one exception to
 *     this and to the stream-capture rule above is vvb_lm_head_argmax_static_dev:
 *     its calls share one array in the library image (calls that overlap on a
 *     GPU race on it) and its first call per device looks that array's address
 *     up, which belongs before any capture -- see its declaration;
 *   - the return value is a vv_status_t code; nothing throws, aborts or logs;
 *   - rows == 0 / n == 0 is VV_OK and launches nothing;
 *   - there is no CPU fallback anywhere: without a usable CUDA device the
 *     calls return VV_ERR_CUDA / VV_ERR_CUDA_LAUNCH.
 *
 * Pointers that are 16-byte aligned with row widths that are multiples of 8
 * halves take the 128-bit paths; anything else takes slower scalar kernels
 * with the same results.
 */
#ifndef VVB200_H
#define VVB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes: numerically those of include/vibevoice/types.h:18-58. When
 * the reference's own types.h is in scope its enum is used instead. */
#ifndef VV_TYPES_H
typedef enum vv_status {
    VV_OK = 0,
    VV_ERR_INVALID_ARG = -1,
    VV_ERR_NULL_PTR = -2,
    VV_ERR_OUT_OF_MEMORY = -3,
    VV_ERR_UNSUPPORTED = -7,
    VV_ERR_OVERFLOW = -8,
    VV_ERR_CUDA = -100,
    VV_ERR_CUDA_OOM = -101,
    VV_ERR_CUDA_LAUNCH = -102
} vv_status_t;
#endif

/* ====================================================================== *
 *  Group 1 -- the reference's op names (drop-in)                          *
 * ====================================================================== */

/** out[p, :] = table[ids[p], :], a bit copy. Replaces
 *  include/vibevoice/device.h:486-488 (src/cuda/embedding.cu:59). Like the
 *  reference it cannot range-check ids (the table height is not an argument);
 *  vvb_embedding_rmsnorm_dev takes the height and clamps. */
vv_status_t vv_embedding_dev(const void* table, const int32_t* ids, void* output,
                             int seq_len, int hidden_size, void* stream);

/** Per row: y = f16((x * inv) * w), inv = 1/sqrt(mean(x^2) + eps); the sum of
 *  squares is accumulated in double, as the reference's CPU kernel does.
 *  input == output is allowed. Correct for any hidden_size >= 1. Replaces
 *  include/vibevoice/device.h:490-492 (src/cuda/rmsnorm.cu:82). */
vv_status_t vv_rmsnorm_dev(const void* input, const void* weight, void* output,
                           int seq_len, int hidden_size, float eps, void* stream);

/** RoPE in place over x[seq_len, n_heads, head_dim], pairs (i, i + head_dim/2),
 *  freq_i = powf(theta, -2i/head_dim) taken from the HOST libm, angle =
 *  (float)pos * freq_i, pos = row + (d_position ? *d_position : position_offset).
 *  head_dim must be even and <= 512 (VV_ERR_UNSUPPORTED beyond). Replaces
 *  include/vibevoice/device.h:494-502 (src/cuda/rope.cu:89). */
vv_status_t vv_rope_dev(void* x, int seq_len, int n_heads, int head_dim,
                        int position_offset, const int* d_position, float theta,
                        void* stream);

/** out[i] = f16( (g / (1 + exp(-g))) * up[i] ), g = gate[i]; output == gate
 *  (the engine's call, src/inference/decoder.c:977) and output == up are
 *  allowed. Replaces include/vibevoice/device.h:504-506 (src/cuda/swiglu.cu:79). */
vv_status_t vv_swiglu_dev(const void* gate, const void* up, void* output,
                          int n_elements, void* stream);

/** SwiGLU where row r of gate_up[rows, 2*inter] holds gate then up; output is
 *  [rows, inter]. Replaces include/vibevoice/device.h:508-510, which the
 *  reference declares and implements only for Metal
 *  (src/metal/kernels/transformer.metal:94-106). */
vv_status_t vv_swiglu_fused_dev(const void* gate_up, void* output, int rows,
                                int inter, void* stream);

/** x[i] = f16(float(x[i]) + float(y[i])). Replaces
 *  include/vibevoice/device.h:512 (src/cuda/conv_vae.cu:37). */
vv_status_t vv_residual_add_dev(void* x, const void* y, int total, void* stream);

/** output[m, j] = f16(float(output[m, j]) + float(bias[j])). Replaces
 *  include/vibevoice/device.h:513-514 (src/cuda/conv_vae.cu:72). */
vv_status_t vv_bias_add_dev(void* output, const void* bias, int M, int N, void* stream);

/** FP32 <-> FP16 (round to nearest even). Replace
 *  include/vibevoice/device.h:717-720 (src/cuda/conv_vae.cu:100-116), which
 *  live in the same translation unit as the residual add. */
vv_status_t vv_fp32_to_fp16_dev(const void* in_fp32, void* out_fp16, int n, void* stream);
vv_status_t vv_fp16_to_fp32_dev(const void* in_fp16, void* out_fp32, int n, void* stream);

/* ---- per-token int8 activations (the W8A8 / W4A8 layers' inputs) -------- *
 * sx[m] = max|v[m,:]| / 127, xq = clamp(round-half-even(v * 127 / max|v|),
 * -127, 127), where v is the FP16 value the unfused op would have written;
 * xsum (optional, may be NULL) = sum of xq over each run of 32 columns,
 * [M][K/32]. `layout` orders the bytes inside each run of 32 columns
 * (include/vibevoice/q8.h:19-60). K must be a multiple of 32 and at most
 * VV_ACT_QUANT_MAX_K, M > 0 (the reference's checks and codes:
 * src/cuda/act_quant.cu:222-233). A row is bit-identical to "op, then
 * vv_act_quant_dev" and to the reference's CPU quantizer on the same values. */
#ifndef VV_Q8_H
typedef enum vv_q8_layout {
    VV_Q8_NATURAL = 0,   /* column order */
    VV_Q8_NIBBLE = 1,    /* the 16 even columns, then the 16 odd ones */
    VV_Q8_W4_GEMV = 2,   /* byte order of the W4A16 GPU layout, for the W4A8 GEMV */
    VV_Q8_W4_MMA = 3,    /* the same, arranged for mma.m16n8k32 */
    VV_Q8_LAYOUT_COUNT
} vv_q8_layout_t;
#endif
#ifndef VV_ACT_QUANT_MAX_K
#define VV_ACT_QUANT_MAX_K 22528   /* include/vibevoice/device.h:313 */
#define VV_ACT_QUANT_MIN_K 256     /* include/vibevoice/device.h:315: narrowest row of vv_rmsnorm_q8_dev */
#endif

/** FP16 [M,K] -> int8 [M,K] + FP32 scale [M] (+ xsum). Replaces
 *  include/vibevoice/device.h:317-320 (src/cuda/act_quant.cu:235). */
vv_status_t vv_act_quant_dev(const void* x, int M, int K, int layout,
                             int8_t* xq, float* sx, int32_t* xsum, void* stream);

/** RMSNorm fused with the quantizer. Replaces include/vibevoice/device.h:322-326
 *  (src/cuda/act_quant.cu:247). The FP16 value quantized is vv_rmsnorm_dev's. */
vv_status_t vv_rmsnorm_q8_dev(const void* x, const void* weight, int M, int K, float eps,
                              int layout, int8_t* xq, float* sx, int32_t* xsum, void* stream);

/** SwiGLU fused with the quantizer. Replaces include/vibevoice/device.h:328-331
 *  (src/cuda/act_quant.cu:264). The FP16 value quantized is vv_swiglu_dev's. */
vv_status_t vv_swiglu_q8_dev(const void* gate, const void* up, int M, int K, int layout,
                             int8_t* xq, float* sx, int32_t* xsum, void* stream);

/** Calibration statistics: acc[k] = max(acc[k], max over rows of |x[m,k]|),
 *  x FP16 [M,K], acc FP32 [K] in device memory holding non-negative values,
 *  updated in place (exact in any order). Replaces
 *  include/vibevoice/device.h:333-342 (src/cuda/act_quant.cu:303): with it this
 *  library defines every symbol of the reference's act_quant.cu. */
vv_status_t vv_col_absmax_dev(const void* x, int M, int K, float* acc, void* stream);

/* ---- LM head (the decode step's tail) ---------------------------------- */

/** logits[V] = W[V,K] @ x[K]: FP16 inputs, FP32 accumulation, FP32 output.
 *  Replaces include/vibevoice/device.h:706-708 (src/cuda/lm_head.cu:127). */
vv_status_t vv_lm_head_gemv_dev(const void* x, const void* W, void* logits, int V, int K, void* stream);

/** Two-stage argmax over FP32 logits; scratch_v (256 floats) and scratch_i
 *  (256 ints) are caller-owned device memory, as in the reference. out_value
 *  may be NULL. Ties go to the smaller index. Replaces
 *  include/vibevoice/device.h:710-713 (src/cuda/lm_head.cu:161). */
vv_status_t vv_argmax_dev(const void* logits, int V, void* scratch_v, void* scratch_i,
                          void* out_token, void* out_value, void* stream);

/* ====================================================================== *
 *  Group 2 -- additive entry points (no counterpart symbol in the          *
 *  reference; each states the reference call sequence it equals)           *
 * ====================================================================== */

/** hidden = f16(hidden + delta); normed = rmsnorm(hidden) -- one kernel, four
 *  HBM passes instead of the five of vv_residual_add_dev followed by
 *  vv_rmsnorm_dev (src/inference/decoder.c:950-958 and :988 with the next
 *  layer's :810). delta == normed_out is allowed (the engine reuses that
 *  buffer); delta == NULL skips the add and leaves hidden untouched. */
vv_status_t vvb_add_rmsnorm_dev(void* hidden_inout, const void* delta,
                                const void* weight, void* normed_out,
                                int rows, int hidden_size, float eps, void* stream);

/** hidden = f16(hidden + delta), then RMSNorm + int8 quantization of the
 *  updated row in one kernel: vv_residual_add_dev + vv_rmsnorm_q8_dev
 *  (src/inference/decoder.c:950 then :920). delta == NULL skips the add. */
vv_status_t vvb_add_rmsnorm_q8_dev(void* hidden_inout, const void* delta, const void* weight,
                                   int M, int K, float eps, int layout,
                                   int8_t* xq, float* sx, int32_t* xsum, void* stream);

/** vv_rope_dev on Q[rows, n_q_heads, head_dim] and K[rows, n_kv_heads,
 *  head_dim] in one launch, cos/sin computed once per row for both
 *  (src/inference/decoder.c:850-855 issues two launches). Either of q, k may
 *  be NULL with a head count of 0. */
vv_status_t vvb_rope_qk_dev(void* q, void* k, int rows, int n_q_heads, int n_kv_heads,
                            int head_dim, int position_offset, const int* d_position,
                            float theta, void* stream);

/** The projections' bias adds, RoPE on Q and K, and the KV-cache append of one
 *  layer in ONE launch: q = rope(f16(q + q_bias)) in place; the cache row
 *  (cache_offset + r) of k_cache receives rope(f16(k[r] + k_bias)) and that of
 *  v_cache receives f16(v[r] + v_bias). Replaces up to six passes of the
 *  reference: vv_bias_add_dev x3 (src/inference/decoder.c:463-464), vv_rope_dev
 *  x2 (:850-855) and the two device copies of vv_kv_cache_append for the raw
 *  FP16 cache (src/inference/kv_cache.c:229-246). k_cache and v_cache are one
 *  layer's [max_len, n_kv_heads * head_dim] FP16 arrays; the caller guarantees
 *  cache_offset + rows <= max_len. Each bias may be NULL. When d_position is
 *  non-NULL the device int gives BOTH the RoPE position and the cache row of
 *  row 0 (the decode step's kv length, src/inference/decoder.c:735-737).
 *  keep_k != 0 also writes the rotated K back over k. head_dim must be a
 *  multiple of 16 and every pointer 16-byte aligned (VV_ERR_UNSUPPORTED
 *  otherwise: use the separate ops). */
vv_status_t vvb_rope_qk_append_dev(void* q, void* k, const void* v,
                                   const void* q_bias, const void* k_bias, const void* v_bias,
                                   void* k_cache, void* v_cache,
                                   int rows, int n_q_heads, int n_kv_heads, int head_dim,
                                   int position_offset, int cache_offset, const int* d_position,
                                   float theta, int keep_k, void* stream);

/** kv_format values of vvb_rope_qk_append_fp8_dev: numerically the reference's
 *  vv_kv_format_t (include/vibevoice/kv_quant.h:34-36). */
#define VVB_KV_FP16     0
#define VVB_KV_FP8_E4M3 1
#define VVB_KV_FP8_E5M2 2
#define VVB_KV_TQ4      3   /* TurboQuant 4 / 3 / 2 / 1.5 bits per value: include/vibevoice/kv_quant.h:37-40 */
#define VVB_KV_TQ3      4
#define VVB_KV_TQ2      5
#define VVB_KV_TQ1_5    6

/** vvb_rope_qk_append_dev for the FP8 KV cache: the same single launch, but the
 *  cache rows receive the reference's software FP8 byte of every value (one
 *  byte per element, [max_len, n_kv_heads * head_dim] uint8 per layer -- the
 *  layout vv_kv_quant_store_dev writes with no page table,
 *  src/cuda/kv_quant.cu:60-83; encodings src/cuda/kv_codec.cuh:68-120: mantissa
 *  rounded to nearest even, saturating at +-448 / +-57344, subnormals rounded
 *  half up, NaN stored as zero). Equivalent, byte for byte, to vv_bias_add_dev
 *  x3, vv_rope_dev x2 and vv_kv_quant_store_dev on the FP16 results: K is
 *  rounded to FP16 after the rotation, then k_ref (FP16 [n_kv_heads *
 *  head_dim], the layer's reference key, NULL when the cache keeps none) is
 *  subtracted in float and the difference encoded; V is encoded as it is.
 *  Building the reference key (the mean over the first chunk) stays a call of
 *  its own. kv_format is VVB_KV_FP8_E4M3 or VVB_KV_FP8_E5M2 (anything else:
 *  VV_ERR_UNSUPPORTED). Other arguments as vvb_rope_qk_append_dev. */
vv_status_t vvb_rope_qk_append_fp8_dev(void* q, void* k, const void* v,
                                       const void* q_bias, const void* k_bias, const void* v_bias,
                                       void* k_store, void* v_store, const void* k_ref,
                                       int rows, int n_q_heads, int n_kv_heads, int head_dim,
                                       int position_offset, int cache_offset, const int* d_position,
                                       float theta, int kv_format, int keep_k, void* stream);

/** The general form of the two calls above, which also covers the PAGED cache
 *  of the reference's server (contexts share one pool of 64-position pages,
 *  include/vibevoice/kv_quant.h:47-53): logical position t = cache_offset + r
 *  (or *d_position + r) is written to row page_table[t / 64] * 64 + t % 64 of
 *  k_store / v_store, the mapping of src/cuda/kv_codec.cuh:29-36 that
 *  vv_kv_store_dev applies (src/cuda/kv_quant.cu:508-551). page_table is a
 *  device array with an entry for every page the call touches; NULL means a
 *  contiguous cache (row t). kv_format: VVB_KV_FP16 (k_ref ignored),
 *  VVB_KV_FP8_E4M3 or VVB_KV_FP8_E5M2, or one of the four TurboQuant formats
 *  VVB_KV_TQ4 / TQ3 / TQ2 / TQ1_5 (head_dim 128 only, as in the reference). For
 *  those, each 128-wide head vector -- K after bias, rotation, rounding to FP16
 *  and minus k_ref; V after its bias -- is stored as the reference's
 *  vv_kv_quant_store_dev stores it (src/cuda/kv_quant.cu:85-120): randomized
 *  Hadamard transform, quantization against the vector's RMS with the format's
 *  Lloyd-Max code book, head_dim * bits / 8 bytes of codes in k_store / v_store
 *  ([max_len, n_kv_heads * bytes_per_vec]) and the RMS as FP16 in k_meta /
 *  v_meta ([max_len, n_kv_heads], required). The bytes are those of the
 *  reference's kernel (same operations in the same order, its fast-math square
 *  root and reciprocal included). Everything else as documented for
 *  vvb_rope_qk_append_dev and vvb_rope_qk_append_fp8_dev, which are this call
 *  with page_table == NULL. */
typedef struct vvb_kv_append {
    void* q;                   /* [rows, n_q_heads, head_dim], rotated in place            */
    void* k;                   /* [rows, n_kv_heads, head_dim], read (written if keep_k)   */
    const void* v;             /* [rows, n_kv_heads, head_dim], read                       */
    const void* q_bias;        /* [n_q_heads * head_dim] or NULL                           */
    const void* k_bias;        /* [n_kv_heads * head_dim] or NULL                          */
    const void* v_bias;        /* [n_kv_heads * head_dim] or NULL                          */
    void* k_store;             /* one layer's K cache rows: FP16, bytes, or packed codes   */
    void* v_store;             /* one layer's V cache rows                                 */
    const void* k_ref;         /* FP8 / TurboQuant: FP16 [n_kv_heads * head_dim] or NULL   */
    const int* page_table;     /* device ints or NULL                                      */
    const int* d_position;     /* device int or NULL                                       */
    int rows, n_q_heads, n_kv_heads, head_dim;
    int position_offset;       /* RoPE position of row 0 when d_position is NULL           */
    int cache_offset;          /* logical cache position of row 0 when d_position is NULL  */
    float theta;
    int kv_format;
    int keep_k;
    void* k_meta;              /* TurboQuant only: FP16 [max_len, n_kv_heads], else NULL   */
    void* v_meta;
} vvb_kv_append_t;

vv_status_t vvb_kv_append_dev(const vvb_kv_append_t* args, void* stream);

/** The other half of a TurboQuant cache: its stored vectors are rotated, so the
 *  reference rotates Q once before attention and un-rotates the attention
 *  output after it (src/inference/decoder.c:878-901;
 *  include/vibevoice/kv_quant.h:89-101 vv_kv_rotate_dev / vv_kv_unrotate_dev,
 *  kernel src/cuda/kv_quant.cu:173-200). These are those two operations, in
 *  place on FP16 x [rows, n_heads, head_dim], bit-identical to the reference's
 *  kernel: per 128-wide head vector a fixed +-1 sign pattern, a 128-point
 *  Walsh-Hadamard transform and the factor 1 / sqrt(128) (un-rotate: transform
 *  first, then sign and factor). head_dim must be 128 (VV_ERR_UNSUPPORTED
 *  otherwise, as the reference); rows == 0 or n_heads == 0 is VV_OK. The names
 *  carry this library's prefix because the reference defines its own in a file
 *  this library does not replace (src/cuda/kv_quant.cu holds its attention
 *  kernels too). */
vv_status_t vvb_kv_rotate_dev(void* x_fp16, int n_heads, int head_dim, int rows, void* stream);
vv_status_t vvb_kv_unrotate_dev(void* x_fp16, int n_heads, int head_dim, int rows, void* stream);

/** Final RMSNorm + LM head + greedy argmax in two launches (the reference
 *  issues four: vv_rmsnorm_dev, vv_lm_head_gemv_dev and vv_argmax_dev's two,
 *  src/inference/pipeline.c:1962-1978). x[K] is the last hidden row when
 *  final_norm_w is non-NULL (the norm is applied inside the GEMV's CTAs), else
 *  the already normalised row. logits (FP32 [V]) may be NULL: the argmax comes
 *  from per-CTA partials, not from a pass over the logits. scratch is
 *  caller-owned device memory of at least vvb_lm_head_scratch_bytes(V) bytes,
 *  4-byte aligned; its contents need no initialisation and are overwritten.
 *  K must be a multiple of 8 and at most 11264 with 16-byte aligned x, W and
 *  final_norm_w (VV_ERR_UNSUPPORTED otherwise). out_value may be NULL. */
size_t vvb_lm_head_scratch_bytes(int V);
vv_status_t vvb_lm_head_argmax_dev(const void* x, const void* final_norm_w, float eps, const void* W,
                                   int V, int K, void* logits, void* scratch, size_t scratch_bytes,
                                   int32_t* out_token, float* out_value, void* stream);

/** vvb_lm_head_argmax_dev without the scratch argument, for callers that
 *  cannot allocate device memory. (No counterpart in the reference, whose
 *  argmax takes caller scratch: include/vibevoice/device.h:710-713.)
 *
 *  Meant for a decode loop whose engine spent its device budget on one
 *  workspace at load time and passes ops only their inputs and outputs, or for
 *  a host application that calls this library from a callback without exposing
 *  its allocator: such code cannot call cudaMalloc (the memory may be gone, and
 *  the call stalls every stream of the device mid-token). The argmax partials
 *  therefore live in a 64 KB array inside the library image, held by every GPU
 *  that loads the library until the process exits.
 *
 *  Limit: V <= VVB_LM_HEAD_STATIC_MAX_V (VV_ERR_OVERFLOW beyond; use
 *  vvb_lm_head_argmax_dev for taller heads). K, alignment and the meaning of
 *  every other argument are those of vvb_lm_head_argmax_dev. The call makes no
 *  cudaMalloc / cudaFree and no allocating library call.
 *
 *  The first call made while a given device is current looks up the array's
 *  device address (cudaGetSymbolAddress) and caches it; make that first call
 *  during start-up, before any stream capture. All calls on a device share the
 *  array: it needs no clearing between calls (each launch overwrites what its
 *  reduce step reads), but calls that overlap on the same GPU -- two streams or
 *  two threads -- race on it; serialise them on one stream or give the others
 *  their own scratch through vvb_lm_head_argmax_dev. */
#define VVB_LM_HEAD_STATIC_MAX_V 262144
vv_status_t vvb_lm_head_argmax_static_dev(const void* x, const void* final_norm_w, float eps,
                                          const void* W, int V, int K, void* logits,
                                          int32_t* out_token, float* out_value, void* stream);

/** hidden_out[p] = table[clamp(ids[p], 0, vocab-1)] (bit copy) and
 *  normed_out[p] = rmsnorm(hidden_out[p]) in one kernel: the gather of
 *  src/inference/pipeline.c:2309 fused with layer 0's first norm
 *  (decoder.c:810). vocab <= 0 disables the clamp. normed_out may be NULL
 *  (gather only, weight ignored). */
vv_status_t vvb_embedding_rmsnorm_dev(const void* table, const int32_t* ids,
                                      void* hidden_out, const void* weight,
                                      void* normed_out, int rows, int hidden_size,
                                      int vocab, float eps, void* stream);

/** Sizes above INT_MAX elements for the flat ops (the reference's `int`
 *  counts stop at 2^31-1, about 113k rows of 18944). */
vv_status_t vvb_swiglu_dev(const void* gate, const void* up, void* output,
                           size_t n_elements, void* stream);
vv_status_t vvb_residual_add_dev(void* x, const void* y, size_t total, void* stream);

/** One decoder layer's elementwise chain on one stream, in the engine's
 *  order: add + RMSNorm, RoPE on Q and K, SwiGLU in place on gate
 *  (src/inference/decoder.c:950-977). The three operations touch disjoint
 *  tensors, so when shapes and alignment allow (hidden_size <= 4096 and a
 *  multiple of 8, head_dim a multiple of 16, 16-byte aligned pointers) they go
 *  out as ONE grid whose CTAs are split between them; otherwise as three
 *  launches. Results are byte-identical either way. */
typedef struct vvb_layer_chain {
    void* hidden;          /* [rows, hidden_size] in/out */
    const void* delta;     /* [rows, hidden_size] */
    const void* norm_w;    /* [hidden_size] */
    void* normed;          /* [rows, hidden_size] out */
    void* q;               /* [rows, n_q_heads, head_dim] in place */
    void* k;               /* [rows, n_kv_heads, head_dim] in place */
    void* gate;            /* [rows, inter] in/out (receives silu(gate)*up) */
    const void* up;        /* [rows, inter] */
    int rows, hidden_size, n_q_heads, n_kv_heads, head_dim, inter;
    int position_offset;   /* position of row 0 (a shard passes its first row) */
    float eps, theta;
} vvb_layer_chain_t;
vv_status_t vvb_layer_chain_dev(const vvb_layer_chain_t* c, void* stream);

/* ---- token-row sharding over the GPUs of one box (no collective) -------- */

/** Rows [*first, *first + *count) of `total_rows` that part `part` of `parts`
 *  owns: contiguous blocks of ceil(total/parts), the last ones shorter or
 *  empty. RoPE on a shard passes *first as position_offset. */
vv_status_t vvb_shard_rows(int64_t total_rows, int parts, int part,
                           int64_t* first, int64_t* count);

/* ---- host-buffer pipeline ------------------------------------------------ */

/** A per-device context that owns staging buffers, streams and events, for
 *  callers whose tensors live in HOST memory. Not a CPU fallback: the math
 *  runs on the GPU; this only moves rows host -> device -> host in slices so
 *  that copies in both directions overlap the kernels. */
typedef struct vvb_host_ctx vvb_host_ctx_t;

/** Creates a context on `device` able to process slices of up to
 *  `max_slice_rows` rows of the given layer shape. */
vv_status_t vvb_host_ctx_create(vvb_host_ctx_t** out, int device, int max_slice_rows,
                                int hidden_size, int n_q_heads, int n_kv_heads,
                                int head_dim, int inter);
void vvb_host_ctx_destroy(vvb_host_ctx_t* ctx);

/** vvb_layer_chain_dev with every tensor pointer in HOST memory (pinned for
 *  full speed; pageable works but serialises). Blocks until the results are
 *  back in host memory. */
vv_status_t vvb_layer_chain_host(vvb_host_ctx_t* ctx, const vvb_layer_chain_t* host_tensors);

/** Bytes moved host->device and device->host by the last
 *  vvb_layer_chain_host call on this context. */
void vvb_host_ctx_last_traffic(const vvb_host_ctx_t* ctx, uint64_t* h2d_bytes, uint64_t* d2h_bytes);

/** Device-side duration of the last vvb_layer_chain_host call on this context
 *  in milliseconds, from CUDA events recorded before its first upload and
 *  after its last download. */
float vvb_host_ctx_last_ms(const vvb_host_ctx_t* ctx);

/* ---- the same pipeline on several GPUs of one box ------------------------ */

/** One vvb_host_ctx_t per device and a host thread to drive each. The
 *  reference walks its devices from the host in the same way
 *  (src/inference/pipeline.c:389-513, vv_dev_set_device at
 *  src/cuda/cuda_utils.cu:301-325); rows are independent, so nothing is
 *  exchanged between devices and no device reads another's memory.
 *  `devices` lists the CUDA ordinals to use (NULL: 0 .. n_devices-1). */
typedef struct vvb_host_multi vvb_host_multi_t;
vv_status_t vvb_host_multi_create(vvb_host_multi_t** out, const int* devices, int n_devices,
                                  int max_slice_rows, int hidden_size, int n_q_heads,
                                  int n_kv_heads, int head_dim, int inter);
void vvb_host_multi_destroy(vvb_host_multi_t* m);
int vvb_host_multi_devices(const vvb_host_multi_t* m);

/** vvb_layer_chain_host over all the context's devices: device g of n takes
 *  the rows vvb_shard_rows(rows, n, g) gives it, with its first row added to
 *  position_offset. Blocks until every shard is back in host memory; the
 *  first failing shard's status is returned. Results are byte-identical to
 *  the one-device call. */
vv_status_t vvb_layer_chain_host_multi(vvb_host_multi_t* m, const vvb_layer_chain_t* host_tensors);

/** Slowest device's device-side duration (ms) and the summed bytes moved by
 *  the last vvb_layer_chain_host_multi call. */
float vvb_host_multi_last_ms(const vvb_host_multi_t* m);
void vvb_host_multi_last_traffic(const vvb_host_multi_t* m, uint64_t* h2d_bytes, uint64_t* d2h_bytes);

/* ---- introspection ------------------------------------------------------ */

/** "vvb200 <version> sm_100a". */
const char* vvb_version(void);
/** Short text for a status code. */
const char* vvb_status_string(int status);
/** Number of kernel launches this library has enqueued in this process
 *  (a relaxed atomic counter; for benchmarks that must state launch counts). */
uint64_t vvb_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* VVB200_H */
