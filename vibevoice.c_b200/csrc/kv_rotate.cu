/*
 * kv_rotate.cu -- the randomized Hadamard rotation the TurboQuant KV caches
 * put around attention: the stored K and V vectors are rotated
 * (tq_kv.cuh), so the reference rotates Q once before the attention call and
 * un-rotates the attention output after it instead of inverting the transform
 * per key (src/inference/decoder.c:878-901, include/vibevoice/kv_quant.h:89-101;
 * kernel src/cuda/kv_quant.cu:173-200, entry points :473-494).
 *
 * One 128-wide head vector per warp, lane L holding values 4L .. 4L+3 (one
 * 8-byte load), in place:
 *   forward   v = half -> float; v *= sign(d); WHT128; v *= 1/sqrt(128); -> half
 *   inverse   WHT128; v *= (1/sqrt(128)) * sign(d); -> half
 * in the reference kernel's order of operations, so the bytes are its bytes
 * (the sign factor is +-1: both multiplications round once, whichever way the
 * compiler associates them). HBM-bound: 512 bytes per head vector; a warp keeps
 * kVecs vectors' loads in flight.
 */
#include "tq_kv.cuh"
#include "vvb_launch.h"

#include <atomic>

namespace vvb {

constexpr int kRotThreads = 256;
constexpr int kRotWarps = kRotThreads / 32;
constexpr int kRotVecs = 4;            /* head vectors a warp has in flight */

template <bool INVERSE, bool ALIGNED>
__global__ void __launch_bounds__(kRotThreads)
kv_rotate_kernel(__half* x, size_t nvec) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const size_t first = ((size_t)blockIdx.x * kRotWarps + (threadIdx.x >> 5)) * kRotVecs;
    float sgn[4];
#pragma unroll
    for (int i = 0; i < 4; i++) sgn[i] = tq_sign(4 * lane + i);

    float v[kRotVecs][4];
    bool live[kRotVecs];
#pragma unroll
    for (int n = 0; n < kRotVecs; n++) {
        live[n] = first + n < nvec;                       /* warp-uniform */
        __half* p = x + (first + n) * 128 + 4 * lane;
        if (live[n]) {
            if (ALIGNED) {
                const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(p));
                const float2 a = unpack2(raw.x), b = unpack2(raw.y);
                v[n][0] = a.x; v[n][1] = a.y; v[n][2] = b.x; v[n][3] = b.y;
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) v[n][i] = __half2float(p[i]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) v[n][i] = 0.0f;
        }
    }
    if (!INVERSE) {
#pragma unroll
        for (int n = 0; n < kRotVecs; n++)
#pragma unroll
            for (int i = 0; i < 4; i++) v[n][i] = __fmul_rn(v[n][i], sgn[i]);
    }
    tq_wht128<kRotVecs>(v, lane);                          /* every lane of the warp takes part */
#pragma unroll
    for (int n = 0; n < kRotVecs; n++) {
#pragma unroll
        for (int i = 0; i < 4; i++)
            v[n][i] = __fmul_rn(v[n][i], INVERSE ? __fmul_rn(kTqWhtNorm, sgn[i]) : kTqWhtNorm);
        if (!live[n]) continue;
        __half* p = x + (first + n) * 128 + 4 * lane;
        if (ALIGNED) {
            __stcs(reinterpret_cast<uint2*>(p), make_uint2(pack2(v[n][0], v[n][1]), pack2(v[n][2], v[n][3])));
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) p[i] = __float2half_rn(v[n][i]);
        }
    }
}

extern std::atomic<uint64_t> g_launches;

}  // namespace vvb

using namespace vvb;

extern "C" int vvbk_kv_rotate(void* x, size_t nvec, int inverse, void* stream) {
    if (nvec == 0) return (int)cudaSuccess;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t per_cta = (size_t)kRotWarps * kRotVecs;
    const size_t ctas = (nvec + per_cta - 1) / per_cta;
    if (ctas > 0x7fffffffull) return (int)cudaErrorInvalidValue;
    const bool aligned = (reinterpret_cast<uintptr_t>(x) & 7u) == 0;
    const dim3 grid((unsigned)ctas), block(kRotThreads);
    if (inverse) {
        if (aligned) launch_pdl(kv_rotate_kernel<true, true>, grid, block, 0, s, (__half*)x, nvec);
        else launch_pdl(kv_rotate_kernel<true, false>, grid, block, 0, s, (__half*)x, nvec);
    } else {
        if (aligned) launch_pdl(kv_rotate_kernel<false, true>, grid, block, 0, s, (__half*)x, nvec);
        else launch_pdl(kv_rotate_kernel<false, false>, grid, block, 0, s, (__half*)x, nvec);
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}
