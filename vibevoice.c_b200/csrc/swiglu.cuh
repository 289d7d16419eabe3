/*
 * swiglu.cuh -- the SwiGLU element function and a CTA's streaming body,
 * shared by swiglu.cu and the single-launch layer chain (chain.cu). The
 * arithmetic is documented at the top of swiglu.cu.
 */
#pragma once
#include "vvb_device.cuh"

namespace vvb {

__device__ __forceinline__ float silu_mul(float g, float u) {
    float e, r;
    const float p = __fmul_rn(g, -1.4426950408889634f);               /* -g * log2(e) */
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(p));            /* exp(-g) */
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(__fadd_rn(1.0f, e)));
    return __fmul_rn(__fmul_rn(g, r), u);
}

__device__ __forceinline__ vec16 silu_mul_vec(const vec16& g, const vec16& u) {
    float a[8], b[8];
    unpack8(g, a);
    unpack8(u, b);
#pragma unroll
    for (int e = 0; e < 8; e++) a[e] = silu_mul(a[e], b[e]);
    return pack8(a);
}

/* CTA `bx` of a flat stream over nvec vectors: kUnroll vectors per thread,
 * kThreads threads. out may alias gate or up. */
template <int kUnroll, int kThreads>
__device__ __forceinline__ void swiglu_stream_body(const vec16* g, const vec16* u, vec16* o,
                                                   size_t nvec, size_t bx, int t) {
    const size_t base = bx * (size_t)(kThreads * kUnroll) + t;
    vec16 gv[kUnroll], uv[kUnroll];
#pragma unroll
    for (int j = 0; j < kUnroll; j++) {
        const size_t v = base + (size_t)j * kThreads;
        if (v < nvec) {
            gv[j] = ld_stream(g + v);
            uv[j] = ld_stream(u + v);
        }
    }
#pragma unroll
    for (int j = 0; j < kUnroll; j++) {
        const size_t v = base + (size_t)j * kThreads;
        if (v < nvec) st_stream(o + v, silu_mul_vec(gv[j], uv[j]));
    }
}

}  // namespace vvb
