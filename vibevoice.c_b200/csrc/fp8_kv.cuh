/*
 * fp8_kv.cuh -- the reference's software FP8 encodings of the KV cache
 * (include/vibevoice/kv_quant.h:34-36: VV_KV_FP8_E4M3 = 1, VV_KV_FP8_E5M2 = 2;
 * the byte each float maps to is defined by src/cuda/kv_codec.cuh:68-120).
 *
 * The mapping, for sign s, magnitude a = |f| (M mantissa bits, exponent bias
 * B, smallest normal 2^(1-B)):
 *   a == 0 or NaN          -> s                      (NaN is stored as zero)
 *   a <  2^(1-B)           -> s | min(int(a * 2^(M+B-1) + 0.5), 2^M)
 *                             fixed point, round half UP, in float arithmetic
 *   otherwise              -> mantissa rounded to M bits, nearest even, carry
 *                             into the exponent, then clamped to the largest
 *                             finite code (E4M3: 0x7E = 448, E5M2: 0x7B = 57344)
 * The clamp also covers the reference's early saturation tests (a >= 464,
 * a >= 61440): those are exactly the magnitudes whose rounded code would
 * exceed the largest finite one.
 *
 * Two implementations of that mapping live here, byte for byte equal on all
 * 65 536 FP16 inputs and on the reference-key cases (tests/test_fp8_kv.py):
 *   fp8_encode<FMT>(float)  integer arithmetic on the bit pattern: the normal
 *     range is one add (the rounding increment 2^(22-M) - 1 + the kept LSB, so
 *     the carry runs into the exponent field by itself), a shift, a re-bias and
 *     a min; the subnormal range is fma(a, 2^k, 0.5) truncated by adding 2^23
 *     toward zero; both evaluated, one selected. About 26 instructions per
 *     element with the packing. Kept as the plain statement of the mapping and
 *     for builds with -DVVB_FP8_SOFT.
 *   fp8_encode8 (default)   the hardware conversion cvt.rn.satfinite to
 *     e4m3x2 / e5m2x2, two elements per instruction, with its two differences
 *     from the reference repaired (see there). It took the fused append from
 *     53.8 to 48.0 us at 14449 rows.
 */
#pragma once
#include "vvb_device.cuh"

#include <cuda_fp8.h>

namespace vvb {

enum { KV_RAW = 0, KV_E4M3 = 1, KV_E5M2 = 2 };

template <int FMT>
__device__ __forceinline__ uint32_t fp8_encode(float f) {
    constexpr int M = (FMT == KV_E4M3) ? 3 : 2;
    constexpr int BIAS = (FMT == KV_E4M3) ? 7 : 15;
    constexpr uint32_t MAX_CODE = (FMT == KV_E4M3) ? 0x7Eu : 0x7Bu;
    constexpr uint32_t MIN_NORMAL = (uint32_t)(127 + 1 - BIAS) << 23;      /* bits of 2^(1-BIAS) */
    const float sub_scale = (FMT == KV_E4M3) ? 512.0f : 65536.0f;          /* 2^(M+BIAS-1) */

    /* Branch-free: both ranges are evaluated and one is selected (lanes of a
     * warp hold values of both ranges nearly always, so a branch would run
     * both sides anyway, plus the divergence). */
    const uint32_t b = __float_as_uint(f);
    const uint32_t ab = b & 0x7fffffffu;
    const float a = __uint_as_float(ab);
    /* below the smallest normal (zero included): int(a * scale + 0.5), truncated.
     * Adding 2^23 toward zero leaves that integer in the low mantissa bits. */
    const float t = __fmaf_rn(a, sub_scale, 0.5f);
    uint32_t sub = __float_as_uint(__fadd_rz(t, 8388608.0f)) & 0xFu;
    sub = min(sub, 1u << M);
    /* normal range */
    const uint32_t r = ab + ((1u << (22 - M)) - 1u) + ((ab >> (23 - M)) & 1u);
    uint32_t nor = (r >> (23 - M)) - ((uint32_t)(127 - BIAS) << M);
    nor = min(nor, MAX_CODE);
    uint32_t code = (ab < MIN_NORMAL) ? sub : nor;
    code = (ab > 0x7f800000u) ? 0u : code;                       /* NaN */
    return ((b >> 24) & 0x80u) | code;
}

/* Eight FP16 values (optionally minus eight FP16 reference values, the
 * subtraction in float as src/cuda/kv_quant.cu:66-73 does it) -> eight bytes,
 * element e in byte e. */
template <int FMT>
__device__ __forceinline__ uint2 fp8_encode8(const vec16& x, const vec16* ref) {
    float f[8];
    unpack8(x, f);
    if (ref != nullptr) {
        float r[8];
        unpack8(*ref, r);
#pragma unroll
        for (int e = 0; e < 8; e++) f[e] = __fsub_rn(f[e], r[e]);
    }
#ifndef VVB_FP8_SOFT
    /* The hardware conversion (cvt.rn.satfinite to e4m3x2 / e5m2x2) agrees
     * with the mapping above except in two places, both repaired here:
     *  - below the smallest normal it rounds ties to even where the reference
     *    rounds them up. Scaling such a value by 1 + 2^-19 first moves every
     *    exact tie above its half-way point and nothing else across one: ties
     *    are odd multiples of 2^-10 (2^-17 for E5M2), the inputs lie on the
     *    FP16 grid or are differences of two FP16 values, so the nearest input
     *    below a tie is at least 2^-24 away, and the scaling moves a value
     *    below 2^-6 by less than 2^-25;
     *  - it stores NaN as NaN; the reference stores zero. */
    constexpr uint32_t MIN_NORMAL = (uint32_t)(127 + 1 - ((FMT == KV_E4M3) ? 7 : 15)) << 23;
    constexpr uint32_t NAN_ADD = (FMT == KV_E4M3) ? 0x01010101u : 0x04040404u;   /* 0x80 - (largest finite code + 1) */
    const float nudge = 1.0f + 1.9073486328125e-06f;                             /* 1 + 2^-19 */
    uint32_t w[4];
#pragma unroll
    for (int p = 0; p < 4; p++) {
        float a0 = f[2 * p], a1 = f[2 * p + 1];
        if ((__float_as_uint(a0) & 0x7fffffffu) < MIN_NORMAL) a0 = __fmul_rn(a0, nudge);
        if ((__float_as_uint(a1) & 0x7fffffffu) < MIN_NORMAL) a1 = __fmul_rn(a1, nudge);
        w[p] = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a0, a1), __NV_SATFINITE,
                                                  (FMT == KV_E4M3) ? __NV_E4M3 : __NV_E5M2);
    }
    uint32_t lo = w[0] | (w[1] << 16), hi = w[2] | (w[3] << 16);
    /* a byte whose low seven bits exceed the largest finite code is a NaN: clear it */
    const uint32_t nlo = (((lo & 0x7f7f7f7fu) + NAN_ADD) & 0x80808080u) >> 7;
    const uint32_t nhi = (((hi & 0x7f7f7f7fu) + NAN_ADD) & 0x80808080u) >> 7;
    lo &= ~(nlo * 0xFFu);
    hi &= ~(nhi * 0xFFu);
    return make_uint2(lo, hi);
#else
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int e = 0; e < 4; e++) {
        lo |= fp8_encode<FMT>(f[e]) << (8 * e);
        hi |= fp8_encode<FMT>(f[e + 4]) << (8 * e);
    }
    return make_uint2(lo, hi);
#endif
}

}  // namespace vvb
