/*
 * vvb_oracle.c -- CPU restatement of the reference's per-token layer kernels.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the shipped library links, loads or
 * calls this file; it exists so the CUDA kernels can be checked against the
 * arithmetic the reference's CPU path performs. Parity is pinned: this file is
 * checked bit-for-bit against the reference's own compiled CPU kernels
 * (oracle/_ref/libvvref_cpu.so, built by oracle/Makefile from the reference's
 * src/cpu/cpu_kernels.c) and against fixtures that build produced
 * (tests/golden/, written by tests/golden/make_golden.py).
 *
 * Activations are FP32 and weights FP16, as on the reference's CPU path
 * (include/vibevoice/cpu_kernels.h:5-7). Each function names the reference
 * lines whose arithmetic it follows. The loops are arranged differently from
 * the reference (trigonometry hoisted out of the head loop, explicit row
 * blocking) but every floating-point operation that reaches a result is the
 * same operation on the same operands in the same order, so results are
 * bit-identical.
 *
 * Build: gcc -O2 -std=c11 -fopenmp -fPIC -shared (no -ffast-math, no -mfma:
 * a fused multiply-add would change the RoPE and SwiGLU roundings).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_OK 0
#define ORC_ERR_INVALID_ARG (-1) /* include/vibevoice/types.h:22 */
#define ORC_ERR_NULL_PTR (-2)    /* include/vibevoice/types.h:23 */

/* IEEE binary16 -> binary32, exact (include/vibevoice/types.h:107-129). */
float orc_half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1Fu;
    uint32_t m = h & 0x3FFu;
    uint32_t bits;
    if (e == 31u) {
        bits = sign | 0x7F800000u | (m << 13);
    } else if (e != 0u) {
        bits = sign | ((e + 112u) << 23) | (m << 13);
    } else if (m == 0u) {
        bits = sign;
    } else {
        /* subnormal: value = m * 2^-24; normalise the mantissa */
        uint32_t ex = 113u;
        do { m <<= 1; ex--; } while (!(m & 0x400u));
        bits = sign | (ex << 23) | ((m & 0x3FFu) << 13);
    }
    float f;
    memcpy(&f, &bits, sizeof f);
    return f;
}

/* binary32 -> binary16, round to nearest even: the rounding CUDA's
 * __float2half and torch's .half() perform (include/vibevoice/types.h:171-196). */
uint16_t orc_float_to_half_rne(float f) {
    uint32_t u;
    memcpy(&u, &f, sizeof u);
    const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    const uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);       /* NaN */
    if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);      /* inf / overflow */
    if (a >= 0x38800000u) {                                       /* normal */
        uint32_t h = (a >> 13) - (112u << 10);
        const uint32_t rest = a & 0x1FFFu;
        h += (rest > 0x1000u) || (rest == 0x1000u && (h & 1u));
        return (uint16_t)(sign | h);
    }
    if (a <= 0x33000000u) return sign;                            /* <= 2^-25 */
    const uint32_t shift = 126u - (a >> 23);                      /* 14..24 */
    const uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
    uint32_t h = m >> shift;
    const uint32_t rest = m & ((1u << shift) - 1u);
    const uint32_t halfway = 1u << (shift - 1u);
    h += (rest > halfway) || (rest == halfway && (h & 1u));
    return (uint16_t)(sign | h);
}

void orc_widen_f16(const uint16_t* src, float* dst, size_t n) {
    ptrdiff_t i;
#pragma omp parallel for schedule(static)
    for (i = 0; i < (ptrdiff_t)n; i++) dst[i] = orc_half_to_float(src[i]);
}

void orc_round_f16(const float* src, uint16_t* dst, size_t n) {
    ptrdiff_t i;
#pragma omp parallel for schedule(static)
    for (i = 0; i < (ptrdiff_t)n; i++) dst[i] = orc_float_to_half_rne(src[i]);
}

/* RMSNorm, src/cpu/cpu_kernels.c:1432-1451: sum of squares in double,
 * inv = 1/sqrtf((float)(ss/n) + eps) in float, y = (x*inv)*w. */
int orc_rmsnorm(const float* in, const uint16_t* w_f16, float* out,
                int rows, int n, float eps) {
    if (!in || !w_f16 || !out) return ORC_ERR_NULL_PTR;
    if (rows < 0 || n <= 0) return ORC_ERR_INVALID_ARG;
    float* w = (float*)malloc(sizeof(float) * (size_t)n);
    if (!w) return ORC_ERR_INVALID_ARG;
    for (int i = 0; i < n; i++) w[i] = orc_half_to_float(w_f16[i]);
    int r;
#pragma omp parallel for schedule(static)
    for (r = 0; r < rows; r++) {
        const float* x = in + (size_t)r * (size_t)n;
        float* y = out + (size_t)r * (size_t)n;
        double acc = 0.0;
        for (int i = 0; i < n; i++) acc += (double)x[i] * x[i];
        const float mean = (float)(acc / n);
        const float inv = 1.0f / sqrtf(mean + eps);
        for (int i = 0; i < n; i++) {
            const float scaled = x[i] * inv;
            y[i] = scaled * w[i];
        }
    }
    free(w);
    return ORC_OK;
}

/* RoPE, src/cpu/cpu_kernels.c:1453-1478: freq_i = powf(theta, -2i/hd),
 * ang = (float)pos * freq_i, pairs (i, i + hd/2):
 *   v[i] = a*c - b*s ; v[i+hd/2] = a*s + b*c   (four products, each rounded).
 * cos/sin depend only on (pos, i), so they are computed once per row. */
int orc_rope(float* x, int rows, int n_heads, int head_dim,
             int position_offset, float theta) {
    if (!x) return ORC_ERR_NULL_PTR;
    if (rows < 0 || n_heads < 0 || head_dim < 0) return ORC_ERR_INVALID_ARG;
    const int half = head_dim / 2;
    if (half == 0) return ORC_OK;
    float* freq = (float*)malloc(sizeof(float) * (size_t)half);
    if (!freq) return ORC_ERR_INVALID_ARG;
    for (int i = 0; i < half; i++)
        freq[i] = powf(theta, -2.0f * (float)i / (float)head_dim);
    int r;
#pragma omp parallel
    {
        float* cs = (float*)malloc(sizeof(float) * 2u * (size_t)half);
#pragma omp for schedule(static)
        for (r = 0; r < rows; r++) {
            const float pos = (float)(position_offset + r);
            for (int i = 0; i < half; i++) {
                const float ang = pos * freq[i];
                cs[i] = cosf(ang);
                cs[half + i] = sinf(ang);
            }
            for (int h = 0; h < n_heads; h++) {
                float* v = x + ((size_t)r * (size_t)n_heads + (size_t)h) * (size_t)head_dim;
                for (int i = 0; i < half; i++) {
                    const float c = cs[i], s = cs[half + i];
                    const float a = v[i], b = v[i + half];
                    const float ac = a * c, bs = b * s;
                    const float as = a * s, bc = b * c;
                    v[i] = ac - bs;
                    v[i + half] = as + bc;
                }
            }
        }
        free(cs);
    }
    free(freq);
    return ORC_OK;
}

/* The 64 (head_dim/2) inverse frequencies exactly as the reference's CPU
 * kernel forms them (cpu_kernels.c:1468), for tests that need the table. */
int orc_rope_inv_freq(float* out, int head_dim, float theta) {
    if (!out) return ORC_ERR_NULL_PTR;
    for (int i = 0; i < head_dim / 2; i++)
        out[i] = powf(theta, -2.0f * (float)i / (float)head_dim);
    return ORC_OK;
}

/* SwiGLU, src/cpu/cpu_kernels.c:1536-1548: (g / (1 + expf(-g))) * up. */
int orc_swiglu(const float* gate, const float* up, float* out, size_t n) {
    if (!gate || !up || !out) return ORC_ERR_NULL_PTR;
    ptrdiff_t i;
#pragma omp parallel for schedule(static)
    for (i = 0; i < (ptrdiff_t)n; i++) {
        const float g = gate[i];
        const float den = 1.0f + expf(-g);
        const float act = g / den;
        out[i] = act * up[i];
    }
    return ORC_OK;
}

/* Residual add, src/cpu/cpu_kernels.c:1550-1558: x += y in float. */
int orc_residual_add(float* x, const float* y, size_t n) {
    if (!x || !y) return ORC_ERR_NULL_PTR;
    ptrdiff_t i;
#pragma omp parallel for schedule(static)
    for (i = 0; i < (ptrdiff_t)n; i++) x[i] = x[i] + y[i];
    return ORC_OK;
}

/* Embedding gather, src/cpu/cpu_kernels.c:1560-1568: row ids[r] of the FP16
 * table, widened exactly to float. */
int orc_embedding(const uint16_t* table, const int32_t* ids, float* out,
                  int rows, int hidden) {
    if (!table || !ids || !out) return ORC_ERR_NULL_PTR;
    int r;
#pragma omp parallel for schedule(static)
    for (r = 0; r < rows; r++) {
        const uint16_t* src = table + (size_t)ids[r] * (size_t)hidden;
        float* dst = out + (size_t)r * (size_t)hidden;
        for (int i = 0; i < hidden; i++) dst[i] = orc_half_to_float(src[i]);
    }
    return ORC_OK;
}

/* ---- FP16-boundary composites: what the engine's FP16 buffers would hold
 * if each reference CPU op ran on the widened values and its result were
 * rounded back to FP16 (the device stores FP16: src/cuda/conv_vae.cu:29-31,
 * src/cuda/rmsnorm.cu:61). ---- */

/* hidden' = f16(hidden + delta); normed = f16(rmsnorm(widen(hidden'))).
 * Mirrors vv_residual_add_dev followed by vv_rmsnorm_dev
 * (src/inference/decoder.c:950-958). delta may be NULL (plain norm). */
int orc_add_rmsnorm_f16(uint16_t* hidden, const uint16_t* delta,
                        const uint16_t* w_f16, uint16_t* normed,
                        int rows, int n, float eps) {
    if (!hidden || !w_f16 || !normed) return ORC_ERR_NULL_PTR;
    const size_t total = (size_t)rows * (size_t)n;
    float* h = (float*)malloc(sizeof(float) * (total ? total : 1));
    float* y = (float*)malloc(sizeof(float) * (total ? total : 1));
    if (!h || !y) { free(h); free(y); return ORC_ERR_INVALID_ARG; }
    orc_widen_f16(hidden, h, total);
    if (delta) {
        float* d = (float*)malloc(sizeof(float) * (total ? total : 1));
        if (!d) { free(h); free(y); return ORC_ERR_INVALID_ARG; }
        orc_widen_f16(delta, d, total);
        orc_residual_add(h, d, total);
        free(d);
        orc_round_f16(h, hidden, total);
        orc_widen_f16(hidden, h, total);
    }
    int st = orc_rmsnorm(h, w_f16, y, rows, n, eps);
    if (st == ORC_OK) orc_round_f16(y, normed, total);
    free(h); free(y);
    return st;
}

int orc_rope_f16(uint16_t* x, int rows, int n_heads, int head_dim,
                 int position_offset, float theta) {
    if (!x) return ORC_ERR_NULL_PTR;
    const size_t total = (size_t)rows * (size_t)n_heads * (size_t)head_dim;
    float* f = (float*)malloc(sizeof(float) * (total ? total : 1));
    if (!f) return ORC_ERR_INVALID_ARG;
    orc_widen_f16(x, f, total);
    int st = orc_rope(f, rows, n_heads, head_dim, position_offset, theta);
    if (st == ORC_OK) orc_round_f16(f, x, total);
    free(f);
    return st;
}

int orc_swiglu_f16(const uint16_t* gate, const uint16_t* up, uint16_t* out, size_t n) {
    if (!gate || !up || !out) return ORC_ERR_NULL_PTR;
    ptrdiff_t i;
#pragma omp parallel for schedule(static)
    for (i = 0; i < (ptrdiff_t)n; i++) {
        const float g = orc_half_to_float(gate[i]);
        const float u = orc_half_to_float(up[i]);
        const float den = 1.0f + expf(-g);
        const float act = g / den;
        out[i] = orc_float_to_half_rne(act * u);
    }
    return ORC_OK;
}

/* LM head, src/cpu/cpu_kernels.c:1570-1606: logit_t = dot(x, widen(W[t,:])),
 * token = argmax. The reference sums each dot in FP32 in an order fixed by its
 * SIMD width (dot_f32, cpu_kernels.c:598-614) and breaks ties by the OpenMP
 * schedule; this restatement accumulates in DOUBLE (so it is closer to the
 * exact value than either FP32 order) and takes the first maximum. Tests
 * compare FP32 implementations with it under a tolerance and demand the same
 * token whenever the winner's margin exceeds that tolerance. */
int orc_lm_head(const float* x, const uint16_t* w_f16, int V, int K,
                double* logits, int32_t* token, double* value) {
    if (!x || !w_f16 || !logits || !token) return ORC_ERR_NULL_PTR;
    if (V <= 0 || K <= 0) return ORC_ERR_INVALID_ARG;
    int t;
#pragma omp parallel for schedule(static)
    for (t = 0; t < V; t++) {
        const uint16_t* row = w_f16 + (size_t)t * (size_t)K;
        double acc = 0.0;
        for (int k = 0; k < K; k++) acc += (double)x[k] * (double)orc_half_to_float(row[k]);
        logits[t] = acc;
    }
    int best = 0;
    for (t = 1; t < V; t++)
        if (logits[t] > logits[best]) best = t;
    *token = best;
    if (value) *value = logits[best];
    return ORC_OK;
}

int orc_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---- per-token int8 activation quantizer (src/cpu/cpu_int8.c:158-190) ----
 * amax = max|x| over the row; inv = 127/amax (0 for an all-zero row);
 * sx = amax/127; q = clamp(rintf(x*inv), -127, 127) stored at
 * orc_q8_pos(layout, j) inside each run of 32 columns; xsum = sum of q per run. */

/* Where column j (0..31) of a run is stored (include/vibevoice/q8.h:64-73). */
int orc_q8_pos(int layout, int j) {
    const int odd = j & 1, word = (j >> 1) & 3, slot = (j >> 3) + 4 * odd;
    if (layout == 1) return odd ? 16 + (j >> 1) : (j >> 1);               /* NIBBLE  */
    if (layout == 2) return 8 * word + 4 * (slot & 1) + (slot >> 1);      /* W4_GEMV */
    if (layout == 3) return 16 * odd + 4 * word + (slot & 3);             /* W4_MMA  */
    return j;                                                             /* NATURAL */
}

int orc_quant_act_q8(const float* x, int M, int K, int layout,
                     int8_t* xq, float* sx, int32_t* xsum) {
    if (!x || !xq || !sx) return ORC_ERR_NULL_PTR;
    if (M <= 0 || K <= 0 || (K % 32) != 0 || layout < 0 || layout > 3) return ORC_ERR_INVALID_ARG;
    int pos[32];
    for (int j = 0; j < 32; j++) pos[j] = orc_q8_pos(layout, j);
    int m;
#pragma omp parallel for schedule(static)
    for (m = 0; m < M; m++) {
        const float* row = x + (size_t)m * (size_t)K;
        int8_t* q = xq + (size_t)m * (size_t)K;
        float amax = 0.0f;
        for (int k = 0; k < K; k++) {
            const float a = fabsf(row[k]);
            if (a > amax) amax = a;
        }
        const float inv = (amax > 0.0f) ? 127.0f / amax : 0.0f;
        sx[m] = amax / 127.0f;
        for (int run = 0; run < K / 32; run++) {
            int s = 0;
            for (int j = 0; j < 32; j++) {
                float v = rintf(row[run * 32 + j] * inv);
                if (v > 127.0f) v = 127.0f;
                if (v < -127.0f) v = -127.0f;
                const int qi = (int)v;
                s += qi;
                q[run * 32 + pos[j]] = (int8_t)qi;
            }
            if (xsum) xsum[(size_t)m * (size_t)(K / 32) + run] = s;
        }
    }
    return ORC_OK;
}

/* ---- software FP8 of the KV cache (src/cuda/kv_codec.cuh:68-120) ----------
 * The reference stores a float as one byte: sign, E exponent bits (bias B),
 * M mantissa bits; E4M3 has B = 7 and tops out at 448 (0x7E), E5M2 has B = 15
 * and tops out at 57344 (0x7B). Step by step, as kv_codec.cuh does it:
 *   zero or NaN -> the sign bit alone;
 *   a >= 464 (E4M3) / 61440 (E5M2) -> the largest finite code;
 *   exponent below the normal range -> q = (int)(a * 2^(M+B-1) + 0.5f) in float
 *     arithmetic, capped at 2^M (which is the smallest normal's code);
 *   else take the top M mantissa bits, round on the remainder to nearest, ties
 *     to even, carry into the exponent, and saturate if the exponent left the
 *     range.
 * fmt: 1 = E4M3, 2 = E5M2 (include/vibevoice/kv_quant.h:34-36). */
uint8_t orc_fp8_encode(float f, int fmt) {
    const int M = (fmt == 1) ? 3 : 2;
    const int bias = (fmt == 1) ? 7 : 15;
    const int emax = (fmt == 1) ? 8 : 15;
    const uint8_t top = (fmt == 1) ? 0x7E : 0x7B;
    const float sat = (fmt == 1) ? 464.0f : 61440.0f;
    uint32_t b;
    memcpy(&b, &f, 4);
    const uint8_t s = (uint8_t)((b >> 24) & 0x80u);
    const float a = fabsf(f);
    if (!(a > 0.0f)) return s;
    if (a >= sat) return (uint8_t)(s | top);
    int e = (int)((b >> 23) & 0xFFu) - 127;
    if (e < 1 - bias) {
        const float scaled = a * ldexpf(1.0f, M + bias - 1);   /* exact: a power of two */
        int q = (int)(scaled + 0.5f);
        if (q > (1 << M)) q = 1 << M;
        return (uint8_t)(s | q);
    }
    const uint32_t frac = b & 0x7FFFFFu;
    const int drop = 23 - M;
    uint32_t keep = frac >> drop;
    const uint32_t rem = frac & ((1u << drop) - 1u);
    const uint32_t half = 1u << (drop - 1);
    if (rem > half || (rem == half && (keep & 1u))) {
        keep++;
        if (keep == (1u << M)) { keep = 0; e++; }
    }
    if (e > emax) return (uint8_t)(s | top);
    return (uint8_t)(s | ((uint32_t)(e + bias) << M) | keep);
}

/* The store of src/cuda/kv_quant.cu:60-83 with no page table: x is FP16
 * [n_pos, n_kv_heads * head_dim]; ref (may be null) FP16 [n_kv_heads * head_dim]
 * is subtracted in float before encoding; out[(first_row + p) * width + j]. */
int orc_kv_store_fp8(const uint16_t* x_f16, const uint16_t* ref_f16, int n_pos, int width,
                     int first_row, int fmt, uint8_t* out) {
    if (!x_f16 || !out) return ORC_ERR_NULL_PTR;
    if (n_pos < 0 || width <= 0 || first_row < 0 || (fmt != 1 && fmt != 2)) return ORC_ERR_INVALID_ARG;
    for (int p = 0; p < n_pos; p++) {
        for (int j = 0; j < width; j++) {
            float v = orc_half_to_float(x_f16[(size_t)p * width + j]);
            if (ref_f16) v -= orc_half_to_float(ref_f16[j]);
            /* On the device every NaN that reaches the encoder is the canonical
             * one, whose sign bit is clear (the FP16 -> float conversion and the
             * float subtraction both produce it), so a NaN of either sign is
             * stored as 0x00: the golden bytes of the reference kernel show it. */
            out[(size_t)(first_row + p) * width + j] = (v != v) ? (uint8_t)0 : orc_fp8_encode(v, fmt);
        }
    }
    return ORC_OK;
}

/* Decoding (src/cuda/kv_codec.cuh:91-97,122-128), for round-trip checks. */
float orc_fp8_decode(uint8_t v, int fmt) {
    const int M = (fmt == 1) ? 3 : 2;
    const int bias = (fmt == 1) ? 7 : 15;
    const int e = (v >> M) & ((fmt == 1) ? 0xF : 0x1F);
    const int m = v & ((1 << M) - 1);
    const float r = (e == 0) ? ldexpf((float)m, 1 - bias - M) : ldexpf(1.0f + (float)m / (float)(1 << M), e - bias);
    return (v & 0x80) ? -r : r;
}

/* ---- TurboQuant KV-cache formats (include/vibevoice/kv_quant.h:37-40) ---------
 * The store of src/cuda/kv_quant.cu:40-121 for formats 3..6 (4, 3, 2 and 1.5
 * bits per value), one 128-wide head vector at a time:
 *   v = half -> float, minus the layer's reference key in float (:60-73);
 *   v[d] *= sign(d), a fixed +-1 pattern hashed from the index
 *     (src/cuda/kv_codec.cuh:133-137);
 *   a 128-point Walsh-Hadamard transform, seven butterfly stages of stride
 *     1, 2, 4 .. 64 (kv_codec.cuh:145-163: two stages inside a lane's four
 *     values, five across lanes; each stage is lower + upper / lower - upper
 *     on the previous stage's values), then v *= 1/sqrt(128) as a float
 *     constant (kv_codec.cuh:64);
 *   sigma = sqrtf(max(sum(v*v) / 128, 1e-12)), the sum taken as the device takes
 *     it: a fused multiply-add chain over each lane's four values, then a
 *     butterfly of pairwise float additions across the 32 lanes (:92-95);
 *   each value is coded by the number of decision thresholds 0.5 * (level[j] +
 *     level[j + 1]) that v / sigma exceeds (kv_codec.cuh:232-266); the 1.5-bit
 *     format codes PAIRS of values by the nearest of eight 2-D code words
 *     (:267-288);
 *   lane L's codes occupy bits [nb * L, nb * (L + 1)) of the vector's bytes,
 *     little endian (:99-117), and sigma is kept as FP16 beside them (:118-119).
 * The device kernel is compiled with fast-math: its square root and reciprocal
 * are the hardware approximations and it flushes subnormals, where this file
 * uses sqrtf and a division. The two agree except when v / sigma lands within
 * a few float ulps of a threshold, or sigma within as much of a FP16 rounding
 * boundary; tests compare with that allowance. The code books are the
 * format's definition (Lloyd-Max levels of a unit Gaussian, kv_codec.cuh:42-62)
 * and are restated here digit for digit: a reader needs the same numbers. */
static const float orc_lev4[16] = {-2.725112f, -2.065280f, -1.613787f, -1.251845f, -0.938657f, -0.654379f,
                                   -0.386970f, -0.127960f, +0.127960f, +0.386970f, +0.654379f, +0.938657f,
                                   +1.251845f, +1.613787f, +2.065280f, +2.725112f};
static const float orc_lev3[8] = {-2.150300f, -1.343258f, -0.755588f, -0.244756f,
                                  +0.244756f, +0.755588f, +1.343258f, +2.150300f};
static const float orc_lev2[4] = {-1.511418f, -0.452456f, +0.452456f, +1.511418f};
static const float orc_vq15[16] = {-1.500251f, +0.674678f, -1.127883f, -0.787015f, -0.283251f, +0.390133f,
                                   -0.103102f, +1.624620f, +0.100120f, -1.618563f, +0.286482f, -0.379555f,
                                   +1.134227f, +0.790368f, +1.496572f, -0.666578f};
#define ORC_WHT_NORM 0.0883883476f

float orc_kv_sign(int d) {
    uint32_t h = (uint32_t)d * 2654435761u + 0x9E3779B9u;
    h ^= h >> 15;
    h *= 0x85EBCA6Bu;
    h ^= h >> 13;
    return (h & 1u) ? -1.0f : 1.0f;
}

/* fmt 3..6 -> bits per lane of four values (kv_codec.cuh:181-185). */
static int orc_tq_lane_bits(int fmt) { return fmt == 3 ? 16 : fmt == 4 ? 12 : fmt == 5 ? 8 : fmt == 6 ? 6 : 0; }
int orc_tq_bytes_per_vec(int fmt) { return orc_tq_lane_bits(fmt) * 4; }     /* 32 lanes * bits / 8 */

/* The rotation alone (sign flips, transform, scale): what vv_kv_rotate_dev
 * applies to Q (src/cuda/kv_quant.cu:175-205, forward direction). In place. */
void orc_tq_rotate128(float v[128]) {
    for (int d = 0; d < 128; d++) v[d] *= orc_kv_sign(d);
    for (int s = 1; s < 128; s <<= 1)
        for (int d = 0; d < 128; d++)
            if (!(d & s)) {
                const float lo = v[d], hi = v[d + s];
                v[d] = lo + hi;
                v[d + s] = lo - hi;
            }
    for (int d = 0; d < 128; d++) v[d] *= ORC_WHT_NORM;
}

/* vv_kv_rotate_dev / vv_kv_unrotate_dev on FP16 head vectors, in place
 * (src/cuda/kv_quant.cu:173-200): forward = widen, sign flips, transform,
 * scale, round to FP16; inverse = widen, transform, one multiplication by
 * (scale * sign), round to FP16. */
int orc_kv_rotate_f16(uint16_t* x_f16, size_t nvec, int inverse) {
    if (!x_f16) return ORC_ERR_NULL_PTR;
    for (size_t n = 0; n < nvec; n++) {
        uint16_t* p = x_f16 + n * 128;
        float v[128];
        for (int d = 0; d < 128; d++) v[d] = orc_half_to_float(p[d]);
        if (!inverse) {
            orc_tq_rotate128(v);
        } else {
            for (int s = 1; s < 128; s <<= 1)
                for (int d = 0; d < 128; d++)
                    if (!(d & s)) {
                        const float lo = v[d], hi = v[d + s];
                        v[d] = lo + hi;
                        v[d + s] = lo - hi;
                    }
            for (int d = 0; d < 128; d++) v[d] *= ORC_WHT_NORM * orc_kv_sign(d);
        }
        for (int d = 0; d < 128; d++) p[d] = orc_float_to_half_rne(v[d]);
    }
    return ORC_OK;
}

static uint32_t orc_tq_pack4(const float y[4], float inv_sigma, int fmt) {
    uint32_t bits = 0;
    if (fmt == 6) {
        for (int p = 0; p < 2; p++) {
            const float a = y[2 * p] * inv_sigma, b = y[2 * p + 1] * inv_sigma;
            uint32_t best = 0;
            float bd = 3.402823466e+38f;
            for (uint32_t c = 0; c < 8; c++) {
                const float da = a - orc_vq15[2 * c], db = b - orc_vq15[2 * c + 1];
                const float d = fmaf(da, da, db * db);      /* the device contracts da*da + db*db */
                if (d < bd) { bd = d; best = c; }
            }
            bits |= best << (3 * p);
        }
        return bits;
    }
    const float* lev = fmt == 3 ? orc_lev4 : fmt == 4 ? orc_lev3 : orc_lev2;
    const int nlev = fmt == 3 ? 16 : fmt == 4 ? 8 : 4;
    const int w = fmt == 3 ? 4 : fmt == 4 ? 3 : 2;
    for (int i = 0; i < 4; i++) {
        const float t = y[i] * inv_sigma;
        uint32_t c = 0;
        for (int j = 0; j + 1 < nlev; j++) c += (t > 0.5f * (lev[j] + lev[j + 1])) ? 1u : 0u;
        bits |= c << (w * i);
    }
    return bits;
}

/* x: FP16 [n_pos, n_heads, 128]; ref (may be null): FP16 [n_heads, 128];
 * store: bytes [first_row + n_pos, n_heads, bytes_per_vec]; meta: FP16
 * [first_row + n_pos, n_heads]; rows first_row.. are written. */
int orc_kv_store_tq(const uint16_t* x_f16, const uint16_t* ref_f16, int n_pos, int n_heads, int first_row, int fmt,
                    uint8_t* store, uint16_t* meta) {
    if (!x_f16 || !store || !meta) return ORC_ERR_NULL_PTR;
    const int nb = orc_tq_lane_bits(fmt);
    if (n_pos < 0 || n_heads <= 0 || first_row < 0 || nb == 0) return ORC_ERR_INVALID_ARG;
    const int bpv = nb * 4;
    for (int p = 0; p < n_pos; p++) {
        for (int h = 0; h < n_heads; h++) {
            float v[128];
            const uint16_t* src = x_f16 + ((size_t)p * n_heads + h) * 128;
            for (int d = 0; d < 128; d++) {
                v[d] = orc_half_to_float(src[d]);
                if (ref_f16) v[d] -= orc_half_to_float(ref_f16[(size_t)h * 128 + d]);
            }
            orc_tq_rotate128(v);
            float part[32];
            for (int l = 0; l < 32; l++) {
                float ss = 0.0f;
                for (int i = 0; i < 4; i++) ss = fmaf(v[4 * l + i], v[4 * l + i], ss);
                part[l] = ss;
            }
            for (int o = 16; o > 0; o >>= 1) {
                float next[32];
                for (int l = 0; l < 32; l++) next[l] = part[l] + part[l ^ o];
                memcpy(part, next, sizeof part);
            }
            const float sigma = sqrtf(fmaxf(part[0] / 128.0f, 1e-12f));
            const float inv_sigma = 1.0f / sigma;
            uint32_t words[16] = {0};
            for (int l = 0; l < 32; l++) {
                const uint32_t bits = orc_tq_pack4(v + 4 * l, inv_sigma, fmt);
                const int bit = nb * l;
                words[bit >> 5] |= bits << (bit & 31);
                if ((bit & 31) + nb > 32) words[(bit >> 5) + 1] |= bits >> (32 - (bit & 31));
            }
            const size_t row = (size_t)(first_row + p) * n_heads + h;
            memcpy(store + row * (size_t)bpv, words, (size_t)bpv);      /* little-endian host, as the device */
            meta[row] = orc_float_to_half_rne(sigma);
        }
    }
    return ORC_OK;
}

/* Decoding one stored vector back to the ROTATED domain (kv_codec.cuh:207-229):
 * value = sigma * level[code]. For round-trip checks. */
int orc_kv_load_tq(const uint8_t* vec, uint16_t sigma_f16, int fmt, float out[128]) {
    const int nb = orc_tq_lane_bits(fmt);
    if (!vec || !out) return ORC_ERR_NULL_PTR;
    if (nb == 0) return ORC_ERR_INVALID_ARG;
    const float sigma = orc_half_to_float(sigma_f16);
    uint32_t words[17] = {0};
    memcpy(words, vec, (size_t)nb * 4);
    for (int l = 0; l < 32; l++) {
        const int bit = nb * l, wi = bit >> 5, sh = bit & 31;
        uint32_t b = sh ? ((words[wi] >> sh) | (words[wi + 1] << (32 - sh))) : words[wi];
        b &= (1u << nb) - 1u;
        for (int i = 0; i < 4; i++) {
            if (fmt == 3) out[4 * l + i] = sigma * orc_lev4[(b >> (4 * i)) & 15u];
            else if (fmt == 4) out[4 * l + i] = sigma * orc_lev3[(b >> (3 * i)) & 7u];
            else if (fmt == 5) out[4 * l + i] = sigma * orc_lev2[(b >> (2 * i)) & 3u];
            else out[4 * l + i] = sigma * orc_vq15[2 * ((b >> (3 * (i >> 1))) & 7u) + (i & 1)];
        }
    }
    return ORC_OK;
}
