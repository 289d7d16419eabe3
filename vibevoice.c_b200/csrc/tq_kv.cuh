/*
 * tq_kv.cuh -- the reference's TurboQuant encodings of the KV cache
 * (include/vibevoice/kv_quant.h:37-40: VV_KV_TQ4 = 3, TQ3 = 4, TQ2 = 5,
 * TQ1_5 = 6; the stored bits are defined by src/cuda/kv_quant.cu:40-121 and
 * src/cuda/kv_codec.cuh:42-62,133-163,232-291).
 *
 * A stored vector is its randomized Hadamard transform, quantized against its
 * own RMS:
 *   v[d]  = value - reference key (float), times a fixed +-1 hashed from d;
 *   v     = WHT128(v) / sqrt(128): in the reference a warp holds a vector, lane L
 *           the values v[4L .. 4L+3], two butterfly stages in the lane and five across
 *           lanes; the store below gives a vector to eight lanes instead (the stages
 *           pair the same values whoever holds them, so the bits are the same);
 *   sigma = sqrt(max(sum(v^2) / 128, 1e-12)), kept as FP16 beside the codes;
 *   code  = per value, how many of the format's decision thresholds
 *           v / sigma exceeds (4 / 3 / 2 bits); the 1.5-bit format codes pairs
 *           by the nearest of eight 2-D code words (3 bits a pair);
 *   the codes of values 4L .. 4L+3 are bits [nb*L, nb*(L+1)) of the vector, little endian.
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

/* ---- the store: EIGHT lanes to a vector, 16 consecutive values each ---------------------
 * (The 32-lane form above, four values a lane, is the reference kernel's own distribution and
 * is what the one-vector-per-warp rotation kernel for small inputs uses.) A butterfly stage computes (lo + hi, lo - hi) for the pairs (d, d + stride) whoever holds
 * them, so any distribution of a vector over lanes gives the same bits; with 16 values in a
 * lane four stages run there and only three cross lanes, and everything that is per vector
 * (addresses, the RMS, its square roots) is paid by 8 lanes instead of 32. A warp works on
 * four vectors at once (lane >> 3 says which); `sub` = lane & 7 is the place in the vector. */

/* FP16 sign masks for values 16 sub .. 16 sub + 15, two values per word: flipping the sign
 * bit of the half commutes with every rounding that follows, so it stands for the
 * multiplication by +-1. */
__device__ __forceinline__ void tq_flips16(int sub, uint32_t (&flip)[8]) {
    constexpr uint32_t s0 = tq_sign_word(0), s1 = tq_sign_word(1), s2 = tq_sign_word(2), s3 = tq_sign_word(3);
    const uint32_t word = (sub & 4) ? ((sub & 2) ? s3 : s2) : ((sub & 2) ? s1 : s0);
    const uint32_t mine = (sub & 1) ? (word >> 16) : word;      /* low 16 bits: this lane's values */
#pragma unroll
    for (int w = 0; w < 8; w++)
        flip[w] = ((mine << (15 - 2 * w)) & 0x8000u) | ((mine << (30 - 2 * w)) & 0x80000000u);
}

/* stages of stride 1..8 in the lane, 16..64 against lanes ^1, ^2, ^4 */
__device__ __forceinline__ void tq_wht128_16(float (&v)[16], int lane) {
#pragma unroll
    for (int s = 1; s < 16; s <<= 1)
#pragma unroll
        for (int d = 0; d < 16; d++)
            if (!(d & s)) {
                const float lo = v[d], hi = v[d + s];
                v[d] = __fadd_rn(lo, hi);
                v[d + s] = __fsub_rn(lo, hi);
            }
#pragma unroll
    for (int m = 1; m < 8; m <<= 1) {
        const float own = (lane & m) ? -1.0f : 1.0f;
        float o[16];
#pragma unroll
        for (int d = 0; d < 16; d++) o[d] = __shfl_xor_sync(0xffffffffu, v[d], m);
#pragma unroll
        for (int d = 0; d < 16; d++) v[d] = __fmaf_rn(v[d], own, o[d]);     /* other -+ own, one rounding */
    }
}

/* v: this lane's 16 values of its group's vector, sign flips already applied (and the
 * reference key subtracted). Writes the lane's share of the codes at dst (the vector's first
 * byte; 2-byte aligned) and, from the group's first lane, the FP16 RMS at meta, when `live`
 * (uniform over the group of eight). Every lane of the warp must call. */
template <int FMT>
__device__ __forceinline__ void tq_store16(float (&v)[16], int lane, uint8_t* dst, __half* meta, bool live,
                                           const TqCells* cells) {
    constexpr int NB = TqBits<FMT>::N;                  /* bits of four values */
    const int sub = lane & 7;
    tq_wht128_16(v, lane);
    /* sum of squares in the association of the 32-lane form: partial sums over runs of four
     * values (what a lane holds there), then the halving tree over the run index 4 sub + j from
     * its top bit down: bits 4, 3, 2 cross lanes (sub ^ 4, 2, 1), bits 1, 0 stay in the lane */
    float part[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        part[j] = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            v[4 * j + i] = __fmul_rn(v[4 * j + i], kTqWhtNorm);
            part[j] = __fmaf_rn(v[4 * j + i], v[4 * j + i], part[j]);
        }
    }
#pragma unroll
    for (int m = 4; m > 0; m >>= 1)
#pragma unroll
        for (int j = 0; j < 4; j++) part[j] = __fadd_rn(part[j], __shfl_xor_sync(0xffffffffu, part[j], m));
    const float ss = __fadd_rn(__fadd_rn(part[0], part[2]), __fadd_rn(part[1], part[3]));
    const float mean_sq = fmaxf(tq_div_approx(ss, 128.0f), 1e-12f);
    const float sigma = tq_sqrt_approx(mean_sq);
    /* sigma (stored) is the approximate square root of the mean square; the scale the codes are
     * taken against is the approximate RECIPROCAL square root of that same mean -- what the
     * reference's fast-math build makes of 1.0f / sigma -- not a reciprocal of sigma: the two
     * differ in the last bit often enough to move a code once in some 10^4 vectors. */
    const float inv = tq_rsqrt_approx(mean_sq);
    uint32_t bits[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float y[4] = {v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]};
        bits[j] = tq_pack4<FMT>(y, inv, cells);         /* NB bits: those of lane 4 sub + j of the 32-lane form */
    }
    if (!live) return;
    if constexpr (NB == 16) {
        *reinterpret_cast<uint2*>(dst + 8 * sub) = make_uint2(bits[0] | (bits[1] << 16), bits[2] | (bits[3] << 16));
    } else if constexpr (NB == 8) {
        *reinterpret_cast<uint32_t*>(dst + 4 * sub) = bits[0] | (bits[1] << 8) | (bits[2] << 16) | (bits[3] << 24);
    } else if constexpr (NB == 12) {
        uint16_t* d16 = reinterpret_cast<uint16_t*>(dst + 6 * sub);
        const uint32_t lo = bits[0] | (bits[1] << 12) | (bits[2] << 24);        /* bits 0..31 of the lane's 48 */
        d16[0] = (uint16_t)lo;
        d16[1] = (uint16_t)(lo >> 16);
        d16[2] = (uint16_t)((bits[2] >> 8) | (bits[3] << 4));
    } else {
        const uint32_t all = bits[0] | (bits[1] << 6) | (bits[2] << 12) | (bits[3] << 18);
        uint8_t* d8 = dst + 3 * sub;
        d8[0] = (uint8_t)all;
        d8[1] = (uint8_t)(all >> 8);
        d8[2] = (uint8_t)(all >> 16);
    }
    if (sub == 0) *meta = __float2half_rn(sigma);
}

}  // namespace vvb
