/*
 * elementwise.cu -- residual add, bias add and FP32<->FP16 conversion: the
 * flat ops that share a translation unit with the residual add in the
 * reference (src/cuda/conv_vae.cu:21-116). sm_100a; 16-byte vectors with
 * several loads in flight per thread, scalar kernels for odd sizes and
 * unaligned pointers. All sums are formed in float and rounded once to FP16
 * (round to nearest even), as the reference's kernels do.
 */
#include "vvb_device.cuh"
#include "vvb_launch.h"

#include <atomic>

namespace vvb {

std::atomic<uint64_t> g_launches{0};

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

__device__ __forceinline__ vec16 add_vec(const vec16& a, const vec16& b) {
    return hadd8(a, b);      /* == widen, add, round to FP16 (vvb_device.cuh) */
}

/* x[i] += y[i] over nvec vectors, then `tail` (< 8) scalar elements. */
__global__ void __launch_bounds__(kThreads)
residual_add_vec_kernel(vec16* x, const vec16* y, size_t nvec, __half* tx, const __half* ty, int tail) {
    pdl_wait();
    pdl_trigger();
    const size_t base = (size_t)blockIdx.x * (kThreads * kUnroll) + threadIdx.x;
    vec16 xv[kUnroll], yv[kUnroll];
#pragma unroll
    for (int j = 0; j < kUnroll; j++) {
        const size_t v = base + (size_t)j * kThreads;
        if (v < nvec) { xv[j] = ld_stream(x + v); yv[j] = ld_stream(y + v); }
    }
#pragma unroll
    for (int j = 0; j < kUnroll; j++) {
        const size_t v = base + (size_t)j * kThreads;
        if (v < nvec) st_stream(x + v, add_vec(xv[j], yv[j]));
    }
    if (tail > 0 && blockIdx.x == 0 && threadIdx.x < tail) {
        const int i = threadIdx.x;
        tx[i] = __float2half_rn(__fadd_rn(__half2float(tx[i]), __half2float(ty[i])));
    }
}

__global__ void __launch_bounds__(kThreads)
residual_add_scalar_kernel(__half* x, const __half* y, size_t n) {
    pdl_wait();
    pdl_trigger();
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (size_t)gridDim.x * kThreads)
        x[i] = __float2half_rn(__fadd_rn(__half2float(x[i]), __half2float(y[i])));
}

/* out[m, :] += bias over row vectors; grid.y = row blocks, each CTA keeps its
 * bias vectors in registers across the rows it walks. */
__global__ void __launch_bounds__(kThreads)
bias_add_vec_kernel(vec16* out, const vec16* bias, int M, int nvec) {
    pdl_wait();
    pdl_trigger();
    const int v = blockIdx.x * kThreads + threadIdx.x;
    if (v >= nvec) return;
    const vec16 b = __ldg(bias + v);
    for (int m = blockIdx.y; m < M; m += gridDim.y) {
        vec16* p = out + (size_t)m * (size_t)nvec + v;
        st_stream(p, add_vec(ld_stream(p), b));
    }
}

__global__ void __launch_bounds__(kThreads)
bias_add_scalar_kernel(__half* out, const __half* bias, size_t total, int N) {
    pdl_wait();
    pdl_trigger();
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += (size_t)gridDim.x * kThreads) {
        const int j = (int)(i % (size_t)N);
        out[i] = __float2half_rn(__fadd_rn(__half2float(out[i]), __half2float(bias[j])));
    }
}

/* 8 floats (two 16-byte loads) -> one 16-byte store, and back. */
__global__ void __launch_bounds__(kThreads)
f32_to_f16_kernel(const float* in, __half* out, size_t n, int vec_ok) {
    pdl_wait();
    pdl_trigger();
    const size_t n8 = vec_ok ? n / 8 : 0;
    for (size_t v = (size_t)blockIdx.x * kThreads + threadIdx.x; v < n8; v += (size_t)gridDim.x * kThreads) {
        const float4 a = __ldcs(reinterpret_cast<const float4*>(in) + 2 * v);
        const float4 b = __ldcs(reinterpret_cast<const float4*>(in) + 2 * v + 1);
        const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        st_stream(reinterpret_cast<vec16*>(out) + v, pack8(f));
    }
    for (size_t i = n8 * 8 + (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (size_t)gridDim.x * kThreads)
        out[i] = __float2half_rn(in[i]);
}

__global__ void __launch_bounds__(kThreads)
f16_to_f32_kernel(const __half* in, float* out, size_t n, int vec_ok) {
    pdl_wait();
    pdl_trigger();
    const size_t n8 = vec_ok ? n / 8 : 0;
    for (size_t v = (size_t)blockIdx.x * kThreads + threadIdx.x; v < n8; v += (size_t)gridDim.x * kThreads) {
        float f[8];
        unpack8(ld_stream(reinterpret_cast<const vec16*>(in) + v), f);
        __stcs(reinterpret_cast<float4*>(out) + 2 * v, make_float4(f[0], f[1], f[2], f[3]));
        __stcs(reinterpret_cast<float4*>(out) + 2 * v + 1, make_float4(f[4], f[5], f[6], f[7]));
    }
    for (size_t i = n8 * 8 + (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (size_t)gridDim.x * kThreads)
        out[i] = __half2float(in[i]);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static unsigned capped_blocks(size_t work_items, size_t per_block, size_t cap) {
    size_t b = (work_items + per_block - 1) / per_block;
    if (b < 1) b = 1;
    if (b > cap) b = cap;
    return (unsigned)b;
}

}  // namespace vvb

using namespace vvb;

extern "C" uint64_t vvbk_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int vvbk_residual_add(void* x, const void* y, size_t n, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (n == 0) return (int)cudaSuccess;
    if (aligned16(x) && aligned16(y)) {
        const size_t nvec = n / 8;
        const int tail = (int)(n - nvec * 8);
        const size_t per_cta = (size_t)kThreads * kUnroll;
        size_t blocks = (nvec + per_cta - 1) / per_cta;
        if (blocks == 0) blocks = 1;
        if (blocks > 0x7fffffffu) return (int)cudaErrorInvalidValue;
        launch_pdl(residual_add_vec_kernel, dim3((unsigned)blocks), dim3(kThreads), 0, s, (vec16*)x, (const vec16*)y, nvec, (__half*)x + nvec * 8, (const __half*)y + nvec * 8, tail);
    } else {
        launch_pdl(residual_add_scalar_kernel, dim3(capped_blocks(n, kThreads, 148u * 64u)), dim3(kThreads), 0, s, (__half*)x, (const __half*)y, n);
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

extern "C" int vvbk_bias_add(void* out, const void* bias, int M, int N, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (M <= 0 || N <= 0) return (int)cudaSuccess;
    if (N % 8 == 0 && aligned16(out) && aligned16(bias)) {
        const int nvec = N / 8;
        const unsigned bx = (unsigned)((nvec + kThreads - 1) / kThreads);
        unsigned by = (unsigned)M;
        const unsigned want = (148u * 16u + bx - 1) / bx;   /* enough CTAs to fill the machine */
        if (by > want) by = want;
        if (by > 65535u) by = 65535u;
        launch_pdl(bias_add_vec_kernel, dim3(bx, by), dim3(kThreads), 0, s, (vec16*)out, (const vec16*)bias, M, nvec);
    } else {
        const size_t total = (size_t)M * (size_t)N;
        launch_pdl(bias_add_scalar_kernel, dim3(capped_blocks(total, kThreads, 148u * 64u)), dim3(kThreads), 0, s, (__half*)out, (const __half*)bias, total, N);
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

extern "C" int vvbk_f32_to_f16(const void* in, void* out, size_t n, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (n == 0) return (int)cudaSuccess;
    const int vec_ok = aligned16(in) && aligned16(out);
    launch_pdl(f32_to_f16_kernel, dim3(capped_blocks(n / 8 + 1, kThreads, 148u * 32u)), dim3(kThreads), 0, s, (const float*)in, (__half*)out, n, vec_ok);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

extern "C" int vvbk_f16_to_f32(const void* in, void* out, size_t n, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (n == 0) return (int)cudaSuccess;
    const int vec_ok = aligned16(in) && aligned16(out);
    launch_pdl(f16_to_f32_kernel, dim3(capped_blocks(n / 8 + 1, kThreads, 148u * 32u)), dim3(kThreads), 0, s, (const __half*)in, (float*)out, n, vec_ok);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}
