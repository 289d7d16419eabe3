/*
 * vvb_device.cuh -- device-side helpers shared by the sm_100a kernels:
 * 128-bit streaming loads/stores, FP16 pack/unpack, warp reductions.
 *
 * Everything on this path is read once and written once, so loads and stores
 * carry the streaming (evict-first) cache operator; the only reused data are
 * gamma (read through the read-only path, it stays in L1/L2) and the cos/sin
 * values, which each RoPE CTA computes once into shared memory.
 */
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vvb {

/* One 16-byte vector = 8 halves. */
typedef uint4 vec16;

__device__ __forceinline__ vec16 ld_stream(const vec16* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(vec16* p, const vec16& v) { __stcs(p, v); }

__device__ __forceinline__ float2 unpack2(uint32_t u) {
    __half2 h = *reinterpret_cast<const __half2*>(&u);
    return __half22float2(h);
}
/* Two floats -> two halves, each rounded to nearest even (what __float2half
 * does); low half = a. */
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ uint32_t pack2(float2 a) { return pack2(a.x, a.y); }

/* Sum of two half pairs, each lane rounded once to nearest even. This equals
 * what the CPU kernels compute (widen to float, add, round to half): the sum
 * of two halves is exact in float unless their exponents differ by more than
 * 13, and then the float rounding cannot land on a half-way point of the half
 * grid, so the second rounding decides alone. Checked on the host over
 * 2.7e8 pairs (every half against every sign and exponent): no difference.
 * One instruction for two elements instead of two widenings, an add and a
 * narrowing. (__hadd2_rn: never contracted into a fused multiply-add.) */
__device__ __forceinline__ uint32_t hadd2_bits(uint32_t a, uint32_t b) {
    const __half2 r = __hadd2_rn(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ vec16 hadd8(const vec16& a, const vec16& b) {
    return make_uint4(hadd2_bits(a.x, b.x), hadd2_bits(a.y, b.y), hadd2_bits(a.z, b.z), hadd2_bits(a.w, b.w));
}

/* Packed FP32 pairs: sm_100 issues one instruction for two lanes, each
 * rounded to nearest even exactly as the scalar operation is, so results do
 * not change; the kernels that are bound by instruction issue use these.
 * HAZARD: never feed a mul2 result into an add2. The toolchain (CUDA 12.9)
 * merges a packed product and a packed sum into one fused multiply-add,
 * with the __fmul2_rn / __fadd2_rn intrinsics and with PTX that names .rn
 * alike, which skips the rounding of the product (observed: ties of the int8
 * quantizer rounded the wrong way). Products of products and lone sums are
 * safe; a product that is summed keeps its add scalar. */
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 r;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "mul.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return r;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 r;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(r.x), "=f"(r.y) : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return r;
}
__device__ __forceinline__ float2 splat2(float a) { return make_float2(a, a); }

__device__ __forceinline__ void unpack8(const vec16& v, float (&f)[8]) {
    float2 t;
    t = unpack2(v.x); f[0] = t.x; f[1] = t.y;
    t = unpack2(v.y); f[2] = t.x; f[3] = t.y;
    t = unpack2(v.z); f[4] = t.x; f[5] = t.y;
    t = unpack2(v.w); f[6] = t.x; f[7] = t.y;
}
__device__ __forceinline__ vec16 pack8(const float (&f)[8]) {
    vec16 v;
    v.x = pack2(f[0], f[1]);
    v.y = pack2(f[2], f[3]);
    v.z = pack2(f[4], f[5]);
    v.w = pack2(f[6], f[7]);
    return v;
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

/* Programmatic dependent launch (sm_90+). A kernel launched through
 * launch_pdl() may be scheduled while the kernel before it on the stream is
 * still draining; it must call pdl_wait() before its first global-memory
 * access -- the wait returns when the preceding grid has completed and its
 * writes are visible, so results are those of an ordinary launch -- and calls
 * pdl_trigger() to let the kernel after it be scheduled in turn. Both are
 * no-ops in a kernel launched the ordinary way. What overlaps is the launch
 * latency and the prologue: for the one-row decode shapes, where a kernel is
 * a handful of CTAs, that is most of the kernel's cost. */
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#ifdef __CUDACC__
template <typename... P, typename... A>
static inline cudaError_t launch_pdl(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                     A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}
#endif

}  // namespace vvb
