/*
 * swiglu.cu -- out = silu(gate) * up, flat over n FP16 elements. sm_100a.
 *
 * Two reads and one write per element and nothing reused: the kernel is a
 * pure HBM stream (113 664 bytes per token of the 7B model, 72 % of the whole
 * layer chain's traffic). Each thread issues one 16-byte load from gate and
 * one from up, with the streaming cache operator on loads and stores; eight
 * 256-thread CTAs per SM keep 64 KB in flight per SM, and small CTAs (4 KB per
 * tensor) keep the ramp and the tail short -- measured on B200 this beats 2, 4
 * and 8 vectors per thread at every size from 1 to 14449 rows. The
 * reference launches one half2 per thread with no instruction-level
 * parallelism (src/cuda/swiglu.cu:45-63).
 *
 * Arithmetic: silu(g)*u = (g / (1 + exp(-g))) * u in float, as
 * src/cpu/cpu_kernels.c:1544-1545. At 8 elements per 16-byte vector the
 * instruction stream matters (a fully IEEE expf + divide is ~30 instructions
 * per element, which would make the kernel issue-bound at B200's HBM rate), so
 * exp is one multiply + ex2.approx and the divide is rcp.approx + multiply.
 * Their combined relative error (< 2e-6 for |g| <= 20) is under 1/100 of an
 * FP16 ulp: after rounding to FP16 the result equals the CPU kernel's rounded
 * value except when the exact value sits within that distance of a rounding
 * boundary, where it is one FP16 ulp away -- never two.
 *
 * out == gate (the engine's call, src/inference/decoder.c:977) and out == up
 * are safe: a thread writes only indices it has already read.
 */
#include "swiglu.cuh"
#include "vvb_launch.h"

#include <atomic>

namespace vvb {

extern std::atomic<uint64_t> g_launches;

constexpr int kSwigluThreads = 256;
constexpr int kSwigluUnroll = 1;

/* gate/up/out rows of `row_vecs` vectors; row r of gate starts at
 * gate + r*gate_stride (vectors), likewise up and out. The flat op is the
 * single-row case. grid.y indexes rows. */
template <int kUnroll>
__global__ void __launch_bounds__(kSwigluThreads)
swiglu_vec_kernel(const vec16* gate, const vec16* up, vec16* out,
                  size_t row_vecs, size_t gate_stride, size_t up_stride, size_t out_stride,
                  const __half* tail_gate, const __half* tail_up, __half* tail_out, int tail) {
    pdl_wait();
    pdl_trigger();
    const size_t r = blockIdx.y;
    const vec16* g = gate + r * gate_stride;
    const vec16* u = up + r * up_stride;
    vec16* o = out + r * out_stride;
    swiglu_stream_body<kUnroll, kSwigluThreads>(g, u, o, row_vecs, blockIdx.x, threadIdx.x);
    /* up to 7 trailing elements of a flat call whose n is not a multiple of 8 */
    if (tail > 0 && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x < tail) {
        const int i = threadIdx.x;
        const float gf = __half2float(tail_gate[i]);
        const float uf = __half2float(tail_up[i]);
        tail_out[i] = __float2half_rn(silu_mul(gf, uf));
    }
}

/* Any alignment: scalar halves. */
__global__ void __launch_bounds__(256)
swiglu_scalar_kernel(const __half* gate, const __half* up, __half* out,
                     size_t row_elems, size_t gate_stride, size_t up_stride, size_t out_stride) {
    pdl_wait();
    pdl_trigger();
    const size_t r = blockIdx.y;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < row_elems; i += (size_t)gridDim.x * 256) {
        const float gf = __half2float(gate[r * gate_stride + i]);
        const float uf = __half2float(up[r * up_stride + i]);
        out[r * out_stride + i] = __float2half_rn(silu_mul(gf, uf));
    }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace vvb

using namespace vvb;

extern "C" int vvbk_swiglu(const void* gate, const void* up, void* out, size_t n, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (n == 0) return (int)cudaSuccess;
    if (aligned16(gate) && aligned16(up) && aligned16(out)) {
        const size_t nvec = n / 8;
        const int tail = (int)(n - nvec * 8);
        const size_t per_cta = (size_t)kSwigluThreads * kSwigluUnroll;
        size_t blocks = (nvec + per_cta - 1) / per_cta;
        if (blocks == 0) blocks = 1;
        if (blocks > 0x7fffffffu) return (int)cudaErrorInvalidValue;
        const __half* tg = (const __half*)gate + nvec * 8;
        const __half* tu = (const __half*)up + nvec * 8;
        __half* to = (__half*)out + nvec * 8;
        const dim3 grid((unsigned)blocks, 1);
        launch_pdl(swiglu_vec_kernel<kSwigluUnroll>, grid, dim3(kSwigluThreads), 0, s,
                   (const vec16*)gate, (const vec16*)up, (vec16*)out, nvec, 0, 0, 0, tg, tu, to, tail);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return (int)cudaGetLastError();
    }
    size_t blocks = (n + 255) / 256;
    if (blocks > 148u * 64u) blocks = 148u * 64u;
    launch_pdl(swiglu_scalar_kernel, dim3((unsigned)blocks, 1), dim3(256), 0, s, 
        (const __half*)gate, (const __half*)up, (__half*)out, n, 0, 0, 0);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

extern "C" int vvbk_swiglu_fused(const void* gate_up, void* out, int rows, int inter, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (rows <= 0 || inter <= 0) return (int)cudaSuccess;
    /* grid.y is limited to 65535 rows per launch: slice taller inputs. */
    const int kMaxRows = 65535;
    for (int r0 = 0; r0 < rows; r0 += kMaxRows) {
        const int nr = rows - r0 < kMaxRows ? rows - r0 : kMaxRows;
        const __half* gu = (const __half*)gate_up + (size_t)r0 * 2u * (size_t)inter;
        __half* o = (__half*)out + (size_t)r0 * (size_t)inter;
        if (inter % 8 == 0 && aligned16(gate_up) && aligned16(out)) {
            const size_t row_vecs = (size_t)inter / 8;
            const size_t per_cta = (size_t)kSwigluThreads * kSwigluUnroll;
            const unsigned bx = (unsigned)((row_vecs + per_cta - 1) / per_cta);
            launch_pdl(swiglu_vec_kernel<kSwigluUnroll>, dim3(bx, (unsigned)nr), dim3(kSwigluThreads), 0, s, 
                (const vec16*)gu, (const vec16*)(gu + inter), (vec16*)o,
                row_vecs, 2 * row_vecs, 2 * row_vecs, row_vecs, nullptr, nullptr, nullptr, 0);
        } else {
            unsigned bx = (unsigned)(((size_t)inter + 255) / 256);
            if (bx > 64) bx = 64;
            launch_pdl(swiglu_scalar_kernel, dim3(bx, (unsigned)nr), dim3(256), 0, s, 
                gu, gu + inter, o, (size_t)inter, 2 * (size_t)inter, 2 * (size_t)inter, (size_t)inter);
        }
        g_launches.fetch_add(1, std::memory_order_relaxed);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return (int)cudaSuccess;
}
