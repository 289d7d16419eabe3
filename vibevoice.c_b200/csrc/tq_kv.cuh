/*
 * tq_kv.cuh -- the reference's TurboQuant encodings of the KV cache
 * (include/vibevoice/kv_quant.h:37-40: VV_KV_TQ4 = 3, TQ3 = 4, TQ2 = 5,
 * TQ1_5 = 6; the stored bits are defined by src/cuda/kv_quant.cu:40-121 and
 * src/cuda/kv_codec.cuh:42-62,133-163,232-291), one 128-wide head vector per
 * warp.
 *
 * A stored vector is its randomized Hadamard transform, quantized against its
 * own RMS:
 *   v[d]  = value - reference key (float), times a fixed +-1 hashed from d;
 *   v     = WHT128(v) / sqrt(128): lane L of the warp holds v[4L .. 4L+3], two
 *           butterfly stages run inside the lane and five across lanes;
 *   sigma = sqrt(max(sum(v^2) / 128, 1e-12)), kept as FP16 beside the codes;
 *   code  = per value, how many of the format's decision thresholds
 *           v / sigma exceeds (4 / 3 / 2 bits); the 1.5-bit format codes pairs
 *           by the nearest of eight 2-D code words (3 bits a pair);
 *   lane L's codes are bits [nb*L, nb*(L+1)) of the vector, little endian.
 *
 * The reference builds with fast-math, so its square root, its 1 / sigma (which
 * the compiler turns into a reciprocal square root of the mean square) and its
 * division by head_dim are the hardware approximations; this file names the
 * same PTX instructions (sqrt.approx.ftz, rsqrt.approx.ftz, div.approx.ftz)
 * and performs every other operation in the reference's order, so the bytes
 * are those of the reference's kernel on the same GPU (tests/test_tq_kv.py
 * compares them with the live kernel). The code books are the format's
 * definition -- Lloyd-Max levels of a unit Gaussian -- and have to be these
 * numbers for a stored cache to be readable by the reference's attention
 * kernels.
 */
#pragma once
#include "vvb_device.cuh"

namespace vvb {

enum { KV_TQ4 = 3, KV_TQ3 = 4, KV_TQ2 = 5, KV_TQ1_5 = 6 };

template <int FMT> struct TqBits { static constexpr int N = 0; };
template <> struct TqBits<KV_TQ4> { static constexpr int N = 16; };      /* bits per lane: 4 values x 4 */
template <> struct TqBits<KV_TQ3> { static constexpr int N = 12; };
template <> struct TqBits<KV_TQ2> { static constexpr int N = 8; };
template <> struct TqBits<KV_TQ1_5> { static constexpr int N = 6; };
__host__ __device__ constexpr bool kv_is_tq(int fmt) { return fmt >= KV_TQ4 && fmt <= KV_TQ1_5; }
__host__ __device__ constexpr int tq_bytes_per_vec(int fmt) {
    return fmt == KV_TQ4 ? 64 : fmt == KV_TQ3 ? 48 : fmt == KV_TQ2 ? 32 : fmt == KV_TQ1_5 ? 24 : 0;
}

constexpr float kTqWhtNorm = 0.0883883476f;      /* 1 / sqrt(128) as the reference's float constant */

__device__ __forceinline__ float tq_sign(int d) {
    uint32_t h = (uint32_t)d * 2654435761u + 0x9E3779B9u;
    h ^= h >> 15;
    h *= 0x85EBCA6Bu;
    h ^= h >> 13;
    return (h & 1u) ? -1.0f : 1.0f;
}

/* The same pattern as bits, worked out by the compiler: bit (d & 31) of word d >> 5 is set
 * where the sign is negative. */
__host__ __device__ constexpr uint32_t tq_sign_word(int w) {
    uint32_t bits = 0;
    for (int b = 0; b < 32; b++) {
        uint32_t h = (uint32_t)(32 * w + b) * 2654435761u + 0x9E3779B9u;
        h ^= h >> 15;
        h *= 0x85EBCA6Bu;
        h ^= h >> 13;
        bits |= (h & 1u) << b;
    }
    return bits;
}

/* The levels (src/cuda/kv_codec.cuh:46-62). Scalar formats compare against the
 * decision thresholds 0.5f * (level[j] + level[j + 1]), which the reference forms
 * in float at run time; as compile-time constants they are the same floats (one
 * rounded addition, one exact halving) and become immediates of the compares. */
__host__ __device__ constexpr float tq_lev4(int j) {
    constexpr float v[16] = {-2.725112f, -2.065280f, -1.613787f, -1.251845f, -0.938657f, -0.654379f,
                             -0.386970f, -0.127960f, +0.127960f, +0.386970f, +0.654379f, +0.938657f,
                             +1.251845f, +1.613787f, +2.065280f, +2.725112f};
    return v[j];
}
__host__ __device__ constexpr float tq_lev3(int j) {
    constexpr float v[8] = {-2.150300f, -1.343258f, -0.755588f, -0.244756f,
                            +0.244756f, +0.755588f, +1.343258f, +2.150300f};
    return v[j];
}
__host__ __device__ constexpr float tq_lev2(int j) {
    constexpr float v[4] = {-1.511418f, -0.452456f, +0.452456f, +1.511418f};
    return v[j];
}
/* the 1.5-bit format's eight 2-D code words, (first, second) coordinate interleaved */
__host__ __device__ constexpr float tq_vq15(int j) {
    constexpr float v[16] = {-1.500251f, +0.674678f, -1.127883f, -0.787015f, -0.283251f, +0.390133f,
                             -0.103102f, +1.624620f, +0.100120f, -1.618563f, +0.286482f, -0.379555f,
                             +1.134227f, +0.790368f, +1.496572f, -0.666578f};
    return v[j];
}
template <int FMT>
__host__ __device__ constexpr float tq_threshold(int j) {
    return FMT == KV_TQ4 ? 0.5f * (tq_lev4(j) + tq_lev4(j + 1))
         : FMT == KV_TQ3 ? 0.5f * (tq_lev3(j) + tq_lev3(j + 1))
                         : 0.5f * (tq_lev2(j) + tq_lev2(j + 1));
}

/* 128-point Walsh-Hadamard transform over a warp, four values per lane: strides
 * 1 and 2 inside the lane, strides 4 .. 64 against lane ^ 1 .. lane ^ 16; the
 * lane with the stride's bit set keeps (other - own), the other (own + other).
 * Both are one fused multiply-add of the own value by -1 or +1 onto the other:
 * the product is exact, so the single rounding is that of the addition. */
template <int NV>
__device__ __forceinline__ void tq_wht128(float (&v)[NV][4], int lane) {
#pragma unroll
    for (int n = 0; n < NV; n++) {
        float a;
        a = __fadd_rn(v[n][0], v[n][1]); v[n][1] = __fsub_rn(v[n][0], v[n][1]); v[n][0] = a;
        a = __fadd_rn(v[n][2], v[n][3]); v[n][3] = __fsub_rn(v[n][2], v[n][3]); v[n][2] = a;
        a = __fadd_rn(v[n][0], v[n][2]); v[n][2] = __fsub_rn(v[n][0], v[n][2]); v[n][0] = a;
        a = __fadd_rn(v[n][1], v[n][3]); v[n][3] = __fsub_rn(v[n][1], v[n][3]); v[n][1] = a;
    }
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        const float own = (lane & m) ? -1.0f : 1.0f;
        float o[NV][4];
#pragma unroll
        for (int n = 0; n < NV; n++)
#pragma unroll
            for (int i = 0; i < 4; i++) o[n][i] = __shfl_xor_sync(0xffffffffu, v[n][i], m);
#pragma unroll
        for (int n = 0; n < NV; n++)
#pragma unroll
            for (int i = 0; i < 4; i++) v[n][i] = __fmaf_rn(v[n][i], own, o[n][i]);
    }
}

__device__ __forceinline__ float tq_sqrt_approx(float x) {
    float r;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float tq_rsqrt_approx(float x) {
    float r;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float tq_div_approx(float x, float y) {
    float r;
    asm("div.approx.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(x), "f"(y));
    return r;
}

/* The threshold to test at bit STEP of a code whose higher bits are known:
 * threshold number BASE + 2^STEP - 1, BASE the value of the higher bits; a tree
 * of selects on those bits (LEVEL walks from the top bit down to STEP + 1). */
template <int FMT, int LEVEL, int STEP, int BASE>
struct TqPivot {
    static __device__ __forceinline__ float get(const bool (&hit)[4]) {
        if constexpr (LEVEL <= STEP) {
            return tq_threshold<FMT>(BASE + (1 << STEP) - 1);
        } else {
            return hit[LEVEL] ? TqPivot<FMT, LEVEL - 1, STEP, BASE + (1 << LEVEL)>::get(hit)
                              : TqPivot<FMT, LEVEL - 1, STEP, BASE>::get(hit);
        }
    }
};

/* A second way to the same count, used by the 4-bit format: the real line is cut
 * into 32 cells of width 1/4 ((-inf, -3.75), [-3.75, -3.5), ... [3.75, inf)); the
 * thresholds of a format lie more than 1/4 apart and inside (-3.75, 3.75), so a cell
 * holds at most one. A value's code is the number of thresholds below its cell plus one
 * compare against the threshold inside it (+inf when there is none). The cell index is
 * floor(4 t), exact in float; a NaN is clamped into cell 0, whose count is 0 and whose
 * threshold is +inf: code 0, as by counting. Two conflict-free shared-memory loads (32
 * entries, 32 banks) replace the select tree: 10 instructions a value instead of ~24 for
 * 15 thresholds. */
struct TqCells {
    float inside[32];
    int below[32];
};
template <int FMT>
__host__ __device__ constexpr bool tq_cells_fit() {
    constexpr int n = (FMT == KV_TQ4) ? 15 : (FMT == KV_TQ3) ? 7 : 3;
    for (int j = 0; j < n; j++) {
        if (!(tq_threshold<FMT>(j) > -3.75f && tq_threshold<FMT>(j) < 3.75f)) return false;
        if (j + 1 < n && !(tq_threshold<FMT>(j + 1) - tq_threshold<FMT>(j) > 0.25f)) return false;
    }
    return true;
}
/* measured at 14449 rows: 4-bit 71.6 -> 63.2 us with the table; 3-bit 64.1 -> 64.5, so it keeps the tree */
template <int FMT> struct TqUsesCells { static constexpr bool value = (FMT == KV_TQ4); };

/* Threads 0..31 of a CTA fill the table; the caller puts a barrier before its first use. */
template <int FMT>
__device__ __forceinline__ void tq_cells_fill(TqCells& cells, int t) {
    static_assert(tq_cells_fit<FMT>(), "thresholds must lie more than a cell apart");
    if (t >= 32) return;
    constexpr int n = (FMT == KV_TQ4) ? 15 : (FMT == KV_TQ3) ? 7 : 3;
    const float inf = __int_as_float(0x7f800000);
    const float lower = (t == 0) ? -inf : (float)(t - 16) * 0.25f;
    const float upper = (t == 31) ? inf : (float)(t - 15) * 0.25f;
    int below = 0;
    float inside = inf;
#pragma unroll
    for (int j = 0; j < n; j++) {
        const float thr = tq_threshold<FMT>(j);
        if (thr < lower) below++;
        else if (thr < upper) inside = thr;
    }
    cells.inside[t] = inside;
    cells.below[t] = below;
}

/* Codes of a lane's four values. `cells` is read by the 4-bit format only. */
template <int FMT>
__device__ __forceinline__ uint32_t tq_pack4(const float (&y)[4], float inv_sigma, const TqCells* cells) {
    uint32_t bits = 0;
    if (FMT == KV_TQ1_5) {
#pragma unroll
        for (int p = 0; p < 2; p++) {
            const float a = __fmul_rn(y[2 * p], inv_sigma), b = __fmul_rn(y[2 * p + 1], inv_sigma);
            uint32_t best = 0;
            float bd = 3.402823466e+38f;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const float da = __fsub_rn(a, tq_vq15(2 * c)), db = __fsub_rn(b, tq_vq15(2 * c + 1));
                const float d = __fmaf_rn(da, da, __fmul_rn(db, db));
                if (d < bd) { bd = d; best = (uint32_t)c; }
            }
            bits |= best << (3 * p);
        }
        return bits;
    }
    constexpr int W = (FMT == KV_TQ4) ? 4 : (FMT == KV_TQ3) ? 3 : 2;
    if constexpr (TqUsesCells<FMT>::value) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float t = __fmul_rn(y[i], inv_sigma);
            const int cell = __float2int_rd(fminf(fmaxf(__fmul_rn(t, 4.0f), -16.0f), 15.0f)) + 16;
            const uint32_t c = (uint32_t)cells->below[cell] + ((t > cells->inside[cell]) ? 1u : 0u);
            bits |= c << (W * i);
        }
    } else {
        /* The code of a value is how many of the ascending thresholds it exceeds: a
         * binary search over them, every pivot picked among immediates by the
         * outcomes so far (the 2- and 3-bit formats; the 4-bit one takes the cell table).
         * A NaN exceeds nothing: code 0, as by counting. */
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float t = __fmul_rn(y[i], inv_sigma);
            bool hit[4] = {false, false, false, false};      /* hit[s]: bit s of the code */
            uint32_t c = 0;
#pragma unroll
            for (int step = W - 1; step >= 0; step--) {
                const float pivot = step == 3 ? TqPivot<FMT, 3, 3, 0>::get(hit)
                                  : step == 2 ? TqPivot<FMT, W - 1, 2, 0>::get(hit)
                                  : step == 1 ? TqPivot<FMT, W - 1, 1, 0>::get(hit)
                                              : TqPivot<FMT, W - 1, 0, 0>::get(hit);
                hit[step] = t > pivot;
                c |= hit[step] ? (1u << step) : 0u;
            }
            bits |= c << (W * i);
        }
    }
    return bits;
}

/* NV head vectors, a warp, worked on side by side (the stages of one vector are a chain of
 * shuffles; two or four chains in flight hide each other's latency): lane holds the four
 * values x[4*lane ..] of each (already minus the reference key). Writes bytes_per_vec bytes
 * at dst[n] (2-byte aligned) and the FP16 sigma at meta[n] for every n with live[n]
 * (warp-uniform). `cells`: the CTA's filled cell table (4-bit format). Every lane
 * of the warp must call. */
template <int FMT, int NV>
__device__ __forceinline__ void tq_store_vecs(float (&v)[NV][4], int lane, uint8_t* const (&dst)[NV],
                                              __half* const (&meta)[NV], const bool (&live)[NV],
                                              const TqCells* cells) {
    constexpr int NB = TqBits<FMT>::N;
    /* the signs of values 4 lane .. 4 lane + 3 out of the compile-time bit pattern */
    constexpr uint32_t s0 = tq_sign_word(0), s1 = tq_sign_word(1), s2 = tq_sign_word(2), s3 = tq_sign_word(3);
    const uint32_t word = (lane & 16) ? ((lane & 8) ? s3 : s2) : ((lane & 8) ? s1 : s0);
    const uint32_t mine = word >> (4 * (lane & 7));
    float sgn[4];
#pragma unroll
    for (int i = 0; i < 4; i++) sgn[i] = ((mine >> i) & 1u) ? -1.0f : 1.0f;
#pragma unroll
    for (int n = 0; n < NV; n++)
#pragma unroll
        for (int i = 0; i < 4; i++) v[n][i] = __fmul_rn(v[n][i], sgn[i]);
    tq_wht128<NV>(v, lane);
    float ss[NV];
#pragma unroll
    for (int n = 0; n < NV; n++) {
        ss[n] = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            v[n][i] = __fmul_rn(v[n][i], kTqWhtNorm);
            ss[n] = __fmaf_rn(v[n][i], v[n][i], ss[n]);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int n = 0; n < NV; n++) ss[n] = __fadd_rn(ss[n], __shfl_xor_sync(0xffffffffu, ss[n], o));
#pragma unroll
    for (int n = 0; n < NV; n++) {
        /* sigma (stored) is the approximate square root of the mean square; the scale the codes
         * are taken against is the approximate RECIPROCAL square root of that same mean -- what the
         * reference's fast-math build makes of 1.0f / sigma -- not a reciprocal of sigma: the two
         * differ in the last bit often enough to move a code once in some 10^4 vectors. */
        const float mean_sq = fmaxf(tq_div_approx(ss[n], 128.0f), 1e-12f);
        const float sigma = tq_sqrt_approx(mean_sq);
        const uint32_t bits = tq_pack4<FMT>(v[n], tq_rsqrt_approx(mean_sq), cells);

        /* Lane L's NB bits are bits [NB * L, NB * (L + 1)) of the vector. 16 and 8 bits are a
         * lane's own aligned store; 12 and 6 bits are put together over lane pairs / quads into
         * three whole bytes, which the first lanes of the group store one byte each. The warp's
         * stores cover one contiguous run of bytes_per_vec bytes. */
        if constexpr (NB == 16) {
            if (live[n]) reinterpret_cast<uint16_t*>(dst[n])[lane] = (uint16_t)bits;
        } else if constexpr (NB == 8) {
            if (live[n]) dst[n][lane] = (uint8_t)bits;
        } else if constexpr (NB == 12) {
            const uint32_t other = __shfl_xor_sync(0xffffffffu, bits, 1);
            const uint32_t three = (lane & 1) ? (other | (bits << 12)) : (bits | (other << 12));
            if (live[n]) {
                uint8_t* at = dst[n] + 3 * (lane >> 1);
                if (lane & 1) at[2] = (uint8_t)(three >> 16);
                else { at[0] = (uint8_t)three; at[1] = (uint8_t)(three >> 8); }
            }
        } else {
            uint32_t three = bits << (6 * (lane & 3));
            three |= __shfl_xor_sync(0xffffffffu, three, 1);
            three |= __shfl_xor_sync(0xffffffffu, three, 2);
            if (live[n] && (lane & 3) != 3) dst[n][3 * (lane >> 2) + (lane & 3)] = (uint8_t)(three >> (8 * (lane & 3)));
        }
        if (live[n] && lane == 0) *meta[n] = __float2half_rn(sigma);
    }
}

}  // namespace vvb
