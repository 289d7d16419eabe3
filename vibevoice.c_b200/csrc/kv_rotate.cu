/*
 * kv_rotate.cu -- the randomized Hadamard rotation the TurboQuant KV caches
 * put around attention: the stored K and V vectors are rotated
 * (tq_kv.cuh), so the reference rotates Q once before the attention call and
 * un-rotates the attention output after it instead of inverting the transform
 * per key (src/inference/decoder.c:878-901, include/vibevoice/kv_quant.h:89-101;
 * kernel src/cuda/kv_quant.cu:173-200, entry points :473-494).
 *
 * Per 128-wide head vector, in place:
 *   forward   v = half -> float; v *= sign(d); WHT128; v *= 1/sqrt(128); -> half
 *   inverse   WHT128; v *= (1/sqrt(128)) * sign(d); -> half
 * A butterfly stage computes (lo + hi, lo - hi) for the pairs (d, d + stride) whatever
 * thread holds them, so the results are the reference kernel's bits for any
 * distribution of the vector over lanes. Here EIGHT lanes share a vector, 16
 * consecutive values each (two 16-byte loads): four stages run inside the lane and
 * three by shuffle, against two and five with four values per lane -- the kernel is
 * bound by instruction issue, and the shuffle stages cost twice the in-lane ones. The
 * sign pattern is applied to the FP16 bits (a sign flip commutes with every rounding):
 * one XOR per pair of values, on the input going forward, on the output coming back.
 * A warp takes four consecutive vectors (1 KB) per step and has two steps' loads in
 * flight. HBM traffic: 512 bytes per head vector.
 */
#include "tq_kv.cuh"
#include "vvb_launch.h"

#include <atomic>

namespace vvb {

constexpr int kRotThreads = 256;
constexpr int kRotWarps = kRotThreads / 32;
constexpr int kRotSteps = 2;           /* groups of four vectors a warp has in flight */

template <bool INVERSE>
__global__ void __launch_bounds__(kRotThreads)
kv_rotate_kernel(vec16* x, size_t nvec) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int sub = lane & 7;                                   /* which 16 values of the vector */
    uint32_t flip[8];                                           /* FP16 sign masks of this lane's 16 values */
    tq_flips16(sub, flip);
    /* vector index of this lane in step n: warps take consecutive groups of 4 vectors */
    const size_t first = ((size_t)blockIdx.x * kRotWarps + (threadIdx.x >> 5)) * (4 * kRotSteps) + (lane >> 3);
    vec16 raw[kRotSteps][2];
    bool live[kRotSteps];
#pragma unroll
    for (int n = 0; n < kRotSteps; n++) {
        const size_t vec = first + 4 * n;
        live[n] = vec < nvec;
        if (live[n]) {
            const vec16* p = x + vec * 16 + 2 * sub;            /* a vector is 16 x 16 bytes */
            raw[n][0] = ld_stream(p);
            raw[n][1] = ld_stream(p + 1);
        } else {
            raw[n][0] = raw[n][1] = make_uint4(0, 0, 0, 0);
        }
    }
#pragma unroll
    for (int n = 0; n < kRotSteps; n++) {
        /* a whole warp runs the shuffles; lanes whose vector lies beyond the end carry zeros */
        uint32_t* w = reinterpret_cast<uint32_t*>(&raw[n][0]);
        float v[16];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float2 f = unpack2(INVERSE ? w[i] : (w[i] ^ flip[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
        tq_wht128_16(v, lane);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t packed = pack2(__fmul_rn(v[2 * i], kTqWhtNorm), __fmul_rn(v[2 * i + 1], kTqWhtNorm));
            w[i] = INVERSE ? (packed ^ flip[i]) : packed;
        }
        if (live[n]) {
            vec16* p = x + (first + 4 * n) * 16 + 2 * sub;
            st_stream(p, raw[n][0]);
            st_stream(p + 1, raw[n][1]);
        }
    }
}

/* The plain statement, a vector per warp, lane L holding values 4L .. 4L+3: for pointers
 * that are not 16-byte aligned (ALIGNED8 false: half by half) and for a handful of vectors
 * (a decode step's 28 heads), where the sign masks of the form above cost more than they
 * save. */
template <bool INVERSE, bool ALIGNED8>
__global__ void __launch_bounds__(kRotThreads)
kv_rotate_small_kernel(__half* x, size_t nvec) {
    pdl_wait();
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const size_t vec = (size_t)blockIdx.x * kRotWarps + (threadIdx.x >> 5);
    const bool live = vec < nvec;                               /* warp-uniform */
    __half* p = x + (live ? vec : 0) * 128 + 4 * lane;
    float v[1][4] = {{0.0f, 0.0f, 0.0f, 0.0f}};
    if (live) {
        if (ALIGNED8) {
            const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(p));
            const float2 a = unpack2(raw.x), b = unpack2(raw.y);
            v[0][0] = a.x; v[0][1] = a.y; v[0][2] = b.x; v[0][3] = b.y;
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) v[0][i] = __half2float(p[i]);
        }
    }
    if (!INVERSE) {
#pragma unroll
        for (int i = 0; i < 4; i++) v[0][i] = __fmul_rn(v[0][i], tq_sign(4 * lane + i));
    }
    tq_wht128<1>(v, lane);
    if (!live) return;
#pragma unroll
    for (int i = 0; i < 4; i++)
        v[0][i] = __fmul_rn(v[0][i], INVERSE ? __fmul_rn(kTqWhtNorm, tq_sign(4 * lane + i)) : kTqWhtNorm);
    if (ALIGNED8) {
        __stcs(reinterpret_cast<uint2*>(p), make_uint2(pack2(v[0][0], v[0][1]), pack2(v[0][2], v[0][3])));
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) p[i] = __float2half_rn(v[0][i]);
    }
}

extern std::atomic<uint64_t> g_launches;

}  // namespace vvb

using namespace vvb;

extern "C" int vvbk_kv_rotate(void* x, size_t nvec, int inverse, void* stream) {
    if (nvec == 0) return (int)cudaSuccess;
    cudaStream_t s = (cudaStream_t)stream;
    constexpr size_t kSmall = 512;                       /* vectors: below this the plain form is faster */
    const bool aligned16 = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    const bool aligned8 = (reinterpret_cast<uintptr_t>(x) & 7u) == 0;
    const bool fast = aligned16 && nvec >= kSmall;
    const size_t per_cta = fast ? (size_t)kRotWarps * 4 * kRotSteps : (size_t)kRotWarps;
    const size_t ctas = (nvec + per_cta - 1) / per_cta;
    if (ctas > 0x7fffffffull) return (int)cudaErrorInvalidValue;
    const dim3 grid((unsigned)ctas), block(kRotThreads);
    if (fast) {
        if (inverse) launch_pdl(kv_rotate_kernel<true>, grid, block, 0, s, (vec16*)x, nvec);
        else launch_pdl(kv_rotate_kernel<false>, grid, block, 0, s, (vec16*)x, nvec);
    } else if (aligned8) {
        if (inverse) launch_pdl(kv_rotate_small_kernel<true, true>, grid, block, 0, s, (__half*)x, nvec);
        else launch_pdl(kv_rotate_small_kernel<false, true>, grid, block, 0, s, (__half*)x, nvec);
    } else {
        if (inverse) launch_pdl(kv_rotate_small_kernel<true, false>, grid, block, 0, s, (__half*)x, nvec);
        else launch_pdl(kv_rotate_small_kernel<false, false>, grid, block, 0, s, (__half*)x, nvec);
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}
