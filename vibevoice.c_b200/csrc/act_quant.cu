/*
 * act_quant.cu -- per-token int8 activation quantization fused into the op
 * that produces the activation: plain (attention output -> o_proj), RMSNorm
 * (-> q/k/v and gate/up) and SwiGLU (-> down). sm_100a, HBM-bound.
 *
 * Contract (include/vibevoice/device.h:297-333, src/cuda/act_quant.cu:11-22):
 *   amax = max |v| over the row of FP16 values v the unfused op would write
 *   sx   = amax / 127                     inv = 127 / amax (0 for a zero row)
 *   q    = clamp(round-half-even(v * inv), -127, 127)
 * stored inside each run of 32 columns in the order the reading GEMM wants
 * (include/vibevoice/q8.h:19-73), plus the optional sum of q per run. Every
 * step is an explicitly rounded operation, so a row is bit-identical to "op,
 * then vv_act_quant_dev" and to the reference's CPU quantizer
 * (src/cpu/cpu_int8.c:158-190) on the same FP16 values.
 *
 * One CTA per row, the row in REGISTERS (a quarter of its 16-byte vectors per
 * thread, as in the row-norm kernel) instead of the reference's shared-memory
 * copy: the FP16 row is produced, its absolute maximum reduced with warp
 * shuffles and one shared-memory step, and each thread quantizes the vectors
 * it holds. The RMSNorm variant is the same device code as vv_rmsnorm_dev
 * (row_norm.cuh), the SwiGLU variant the same as vv_swiglu_dev (swiglu.cuh),
 * so "fused == unfused then quantized" holds by construction.
 */
#include "row_norm.cuh"
#include "swiglu.cuh"
#include "vvb_launch.h"

#include <atomic>

namespace vvb {

extern std::atomic<uint64_t> g_launches;

enum { Q_PLAIN = 0, Q_RMSNORM = 1, Q_SWIGLU = 2 };

/* Deep grids of rows that split into whole vectors over 64 threads (hidden
 * sizes 1536 .. 4096 in steps of 512: 3 .. 8 vectors per thread) run as TWO
 * WARPS PER ROW. These kernels are bound by instruction issue and by the
 * latency of their per-row reductions, not by HBM; two warps per row keep 12
 * rows resident per SM instead of 8, put no thread on padding (128 threads x 4
 * vectors leave an eighth of a 3584-wide row's slots empty) and halve the
 * cross-warp part of both reductions. Measured at [14449, 3584]: rmsnorm_q8
 * 40.3 us against 49.1 us for 128 x 4 (45.2 against 52.0 in the weight-GEMM
 * layout), act_quant 22.3 against 26.3; 224 threads x 2 vectors, the other
 * padding-free shape, is slower than both (55 us). */
constexpr int kTwoWarpThreads = 64;
/* CTAs per SM of the two-warp shape. Measured on rmsnorm_q8 [14449, 3584]: 12 (80 registers)
 * 35.1 us; 14 (72 registers, three spilled words) 33.9; 16 (64 registers, 22 spilled words) 35.2. */
constexpr int kTwoWarpMinB = 14;
static inline int two_warp_vpt(int rows, int nvec, int mode) {
    if (mode == 2 || rows <= kLatencyRows || nvec % kTwoWarpThreads != 0) return 0;
    const int v = nvec / kTwoWarpThreads;
    return (v >= 3 && v <= 8) ? v : 0;
}

struct ActQuantArgs {
    RowNormArgs norm;        /* Q_RMSNORM: src/delta/row_out/weight/eps; normed unused */
    const vec16* a;          /* Q_PLAIN: x;  Q_SWIGLU: gate */
    const vec16* b;          /* Q_SWIGLU: up */
    int8_t* xq;
    float* sx;
    int32_t* xsum;           /* may be null */
    int rows, nvec, layout;
};

/* Byte position of column j (0..31) of a run in the four layouts
 * (include/vibevoice/q8.h:64-73), with odd = j & 1, word = (j >> 1) & 3,
 * slot = (j >> 3) + 4 * odd:
 *   0 natural:  j
 *   1:          odd ? 16 + (j >> 1) : (j >> 1)
 *   2:          8 * word + 4 * (slot & 1) + (slot >> 1)
 *   3 w4_mma:   16 * odd + 4 * word + (slot & 3)
 * quantize_vectors below builds whole 32-bit words of these orders. */

/* 4 x 4 byte transpose across four consecutive lanes: lane i (0..3) gives the
 * word [v_i.b0 .. v_i.b3] and receives [v_0.b_i, v_1.b_i, v_2.b_i, v_3.b_i].
 * Two butterfly steps (halves with lane ^ 2, bytes with lane ^ 1); every lane
 * of the warp must call it. */
__device__ __forceinline__ uint32_t transpose4(uint32_t v, int i) {
    const uint32_t x = __shfl_xor_sync(0xffffffffu, v, 2);
    v = (i & 2) ? __byte_perm(x, v, 0x7632) : __byte_perm(v, x, 0x5410);
    const uint32_t y = __shfl_xor_sync(0xffffffffu, v, 1);
    return (i & 1) ? __byte_perm(y, v, 0x7351) : __byte_perm(v, y, 0x6240);
}

/* Quantizes and stores the VPT vectors a thread holds (vector v = t + j*G covers
 * columns 8v .. 8v+7: chunk i = v & 3 of run v >> 2; four consecutive threads
 * hold the four chunks of a run -- G is a multiple of 32 -- which is what the
 * per-run sum and the interleaved layouts need). */
template <int VPT, int GUARD, int LAYOUT, bool SUMS>
__device__ __forceinline__ void quantize_vectors(const vec16 (&yv)[VPT], float inv, int t, int G, int nvec,
                                                 int8_t* xq, int32_t* xsum) {
    const float2 inv2 = splat2(inv);
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        const int v = t + j * G;
        const bool ok = vec_inside<VPT, GUARD>(j, v, nvec);
        /* round-half-even without the conversion unit: p = v*inv is rounded
         * to float first (as the CPU does) and adding 1.5*2^23 rounds it to an
         * integer in the float adder's nearest-even mode; the low byte of the
         * sum's bit pattern is then q as a signed byte (the constant's low
         * byte is zero). The reference's clamp to +-127 can never act: amax is
         * the exact maximum of |v|, so |p| <= amax * fl(127/amax) <
         * 127.00002 and rounds to at most 127. (Rows holding an infinity or
         * a NaN have no defined quantization on the CPU path either.) */
        uint32_t rb[8];
        const uint32_t* yw = reinterpret_cast<const uint32_t*>(&yv[j]);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            /* two columns per packed multiply; the adds stay scalar: the
             * assembler merges a packed multiply and a packed add into one
             * fused multiply-add even when both name .rn, which skips the
             * rounding of the product and moves ties */
            const float2 p = mul2(unpack2(yw[e]), inv2);
            rb[2 * e] = __float_as_uint(__fadd_rn(p.x, 12582912.0f));
            rb[2 * e + 1] = __float_as_uint(__fadd_rn(p.y, 12582912.0f));
        }
        const uint32_t lo = __byte_perm(__byte_perm(rb[0], rb[1], 0x0040), __byte_perm(rb[2], rb[3], 0x0040), 0x5410);
        const uint32_t hi = __byte_perm(__byte_perm(rb[4], rb[5], 0x0040), __byte_perm(rb[6], rb[7], 0x0040), 0x5410);
        int8_t* run = xq + ((size_t)(v >> 2) << 5);
        const int i = v & 3;
        /* The two weight-GEMM layouts interleave the bytes of the four threads
         * that share a run: the bytes are exchanged with shuffles so that every
         * thread stores two whole 32-bit words instead of eight single bytes.
         * (All four threads of a run are in range together: nvec % 4 == 0.) */
        if (LAYOUT == 0) {
            if (ok) *reinterpret_cast<uint2*>(run + (i << 3)) = make_uint2(lo, hi);
        } else if (LAYOUT == 1) {
            /* evens of the chunk at 4i.., odds at 16 + 4i.. */
            if (ok) {
                *reinterpret_cast<uint32_t*>(run + (i << 2)) = __byte_perm(lo, hi, 0x6420);
                *reinterpret_cast<uint32_t*>(run + 16 + (i << 2)) = __byte_perm(lo, hi, 0x7531);
            }
        } else if (LAYOUT == 3) {
            /* byte position 16*odd + 4*word + i: word w of the run's first half
             * is column 2w of the four chunks, of its second half column 2w+1 */
            const uint32_t w0 = transpose4(__byte_perm(lo, hi, 0x6420), t & 3);
            const uint32_t w1 = transpose4(__byte_perm(lo, hi, 0x7531), t & 3);
            if (ok) {
                *reinterpret_cast<uint32_t*>(run + (i << 2)) = w0;
                *reinterpret_cast<uint32_t*>(run + 16 + (i << 2)) = w1;
            }
        } else {
            /* word 2w + (i & 1) = [chunk i&1: col 2w, chunk (i&1)+2: col 2w, then both again for
             * col 2w+1]: threads i and i^2 swap halves and each builds two words */
            const bool high = (t & 2) != 0;
            const uint32_t x = __shfl_xor_sync(0xffffffffu, high ? lo : hi, 2);
            const uint32_t first = high ? x : lo, second = high ? hi : x;
            const int o0 = (high ? 16 : 0) + 4 * (t & 1);
            if (ok) {
                *reinterpret_cast<uint32_t*>(run + o0) = __byte_perm(first, second, 0x5140);
                *reinterpret_cast<uint32_t*>(run + o0 + 8) = __byte_perm(first, second, 0x7362);
            }
        }
        if (SUMS) {
            int s = __dp4a((int)lo, 0x01010101, __dp4a((int)hi, 0x01010101, 0));   /* sum of the 8 signed bytes */
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            if (ok && (t & 3) == 0) xsum[v >> 2] = s;
        }
    }
}

/* MAXT: the largest CTA an instance is launched with; MINB: CTAs per SM it is
 * compiled for, i.e. a register budget of 65536 / (MAXT * MINB). These kernels
 * alternate loads, two CTA-wide reductions and a long arithmetic tail, and they
 * live on warps in flight: an instance that takes 38 registers instead of 32
 * loses a resident CTA per SM and with it 10-18 % (measured: swiglu_q8 297 us
 * against 252 us at 14449 rows, the 512-row norm 3.4 us against 2.7 us because
 * its 512 CTAs then need two waves), so the budget is stated, not left to the
 * compiler. GUARD: how much of the inside-the-row test it carries (row_norm.cuh). */
template <int VPT, int MODE, int GUARD, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB)
act_quant_kernel(const ActQuantArgs a) {
    pdl_wait();
    pdl_trigger();
    __shared__ float red_max[32];
    const int t = threadIdx.x, G = blockDim.x;
    const int row = blockIdx.x;
    const size_t roff = (size_t)row * (size_t)a.nvec;
#define VVB_Q_IN(j) vec_inside<VPT, GUARD>(j, t + (j) * G, a.nvec)

    /* 1. the FP16 row the unfused op would write, in registers */
    vec16 yv[VPT];
    if (MODE == Q_RMSNORM) {
        row_norm_produce<VPT, 1, GUARD, (VPT > 4)>(a.norm, row, t, G, 0, yv);
    } else {
        vec16 bv[VPT];
        const vec16* ap = a.a + roff + t;
        const vec16* bp = a.b + roff + t;
#pragma unroll
        for (int j = 0; j < VPT; j++) {
            yv[j] = VVB_Q_IN(j) ? ld_stream(ap + j * G) : make_uint4(0, 0, 0, 0);
            if (MODE == Q_SWIGLU) bv[j] = VVB_Q_IN(j) ? ld_stream(bp + j * G) : make_uint4(0, 0, 0, 0);
        }
        if (MODE == Q_SWIGLU) {
#pragma unroll
            for (int j = 0; j < VPT; j++) yv[j] = silu_mul_vec(yv[j], bv[j]);
        }
    }

    /* 2. absolute maximum of the row */
    /* the maximum of FP16 magnitudes is itself an FP16 value: take it with
     * packed half2 max (two elements per instruction), widen once */
    __half2 m2 = __float2half2_rn(0.0f);
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        const __half2* h2 = reinterpret_cast<const __half2*>(&yv[j]);
#pragma unroll
        for (int e = 0; e < 4; e++) m2 = __hmax2(m2, __habs2(h2[e]));
    }
    float amax = fmaxf(__low2float(m2), __high2float(m2));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((t & 31) == 0) red_max[t >> 5] = amax;
    __syncthreads();
    /* every lane folds the per-warp maxima with one shared-memory read and a
     * shuffle tree (G <= 1024: at most 32 warps) */
    amax = ((t & 31) < (G >> 5)) ? red_max[t & 31] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));

    /* 3. quantize the vectors this thread holds: the layout and the presence of run
     * sums are decided ONCE per thread here, not once per vector inside the loop (the
     * per-vector tests were a tenth of the kernel's instructions). */
    const float inv = (amax > 0.0f) ? __fdiv_rn(127.0f, amax) : 0.0f;
    if (t == 0) a.sx[row] = __fdiv_rn(amax, 127.0f);
    int8_t* xq = a.xq + (size_t)row * (size_t)a.nvec * 8u;
    int32_t* xsum = a.xsum ? a.xsum + (size_t)row * (size_t)(a.nvec >> 2) : nullptr;
    if (xsum != nullptr) {
        switch (a.layout) {
            case 0: quantize_vectors<VPT, GUARD, 0, true>(yv, inv, t, G, a.nvec, xq, xsum); break;
            case 1: quantize_vectors<VPT, GUARD, 1, true>(yv, inv, t, G, a.nvec, xq, xsum); break;
            case 2: quantize_vectors<VPT, GUARD, 2, true>(yv, inv, t, G, a.nvec, xq, xsum); break;
            default: quantize_vectors<VPT, GUARD, 3, true>(yv, inv, t, G, a.nvec, xq, xsum); break;
        }
    } else {
        switch (a.layout) {
            case 0: quantize_vectors<VPT, GUARD, 0, false>(yv, inv, t, G, a.nvec, xq, xsum); break;
            case 1: quantize_vectors<VPT, GUARD, 1, false>(yv, inv, t, G, a.nvec, xq, xsum); break;
            case 2: quantize_vectors<VPT, GUARD, 2, false>(yv, inv, t, G, a.nvec, xq, xsum); break;
            default: quantize_vectors<VPT, GUARD, 3, false>(yv, inv, t, G, a.nvec, xq, xsum); break;
        }
    }
}

/* Calibration statistics: acc[k] = max(acc[k], max over rows of |x[m,k]|)
 * (include/vibevoice/device.h:333-342, src/cuda/act_quant.cu:283-300). A thread
 * owns 8 columns (one vector) over a block of kColRows rows, keeps the running
 * maximum as packed halves, and merges with an integer atomicMax on the float
 * bit pattern: the values are non-negative, so float order is integer order
 * and the result is exact in any order. NaNs never win (hmax2 returns the
 * other operand), as in the reference. */
constexpr int kColThreads = 128;
constexpr int kColRows = 32;

__global__ void __launch_bounds__(kColThreads)
col_absmax_kernel(const vec16* __restrict__ x, int M, int nvec, float* __restrict__ acc) {
    pdl_wait();
    pdl_trigger();
    const int v = blockIdx.x * kColThreads + threadIdx.x;
    if (v >= nvec) return;
    const int m0 = blockIdx.y * kColRows;
    const int m1 = min(M, m0 + kColRows);
    __half2 mx[4];
#pragma unroll
    for (int e = 0; e < 4; e++) mx[e] = __float2half2_rn(0.0f);
    int m = m0;
    for (; m + 4 <= m1; m += 4) {
        vec16 r[4];
#pragma unroll
        for (int u = 0; u < 4; u++) r[u] = ld_stream(x + (size_t)(m + u) * (size_t)nvec + v);
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const __half2* h2 = reinterpret_cast<const __half2*>(&r[u]);
#pragma unroll
            for (int e = 0; e < 4; e++) mx[e] = __hmax2(mx[e], __habs2(h2[e]));
        }
    }
    for (; m < m1; m++) {
        const vec16 r = ld_stream(x + (size_t)m * (size_t)nvec + v);
        const __half2* h2 = reinterpret_cast<const __half2*>(&r);
#pragma unroll
        for (int e = 0; e < 4; e++) mx[e] = __hmax2(mx[e], __habs2(h2[e]));
    }
    int* out = reinterpret_cast<int*>(acc) + (size_t)v * 8u;
#pragma unroll
    for (int e = 0; e < 4; e++) {
        atomicMax(out + 2 * e, __float_as_int(__low2float(mx[e])));
        atomicMax(out + 2 * e + 1, __float_as_int(__high2float(mx[e])));
    }
}

__global__ void __launch_bounds__(256)
col_absmax_scalar_kernel(const __half* __restrict__ x, int M, int K, float* __restrict__ acc) {
    pdl_wait();
    pdl_trigger();
    const int k = blockIdx.x * 256 + threadIdx.x;
    if (k >= K) return;
    const int m0 = blockIdx.y * 64;
    const int m1 = min(M, m0 + 64);
    float v = 0.0f;
    for (int m = m0; m < m1; m++) v = fmaxf(v, fabsf(__half2float(x[(size_t)m * (size_t)K + k])));
    if (v == v) atomicMax(reinterpret_cast<int*>(acc) + k, __float_as_int(v));
}

/* Register budgets (see act_quant_kernel): the instances that must take any CTA
 * size get 32 registers (two 1024-thread CTAs per SM) unless they hold a norm
 * row of two or four vectors per thread; the instances for CTAs of at most 256
 * threads get 32 registers too (eight CTAs per SM) when they are light, and 64
 * (four CTAs) when they carry the norm. */
constexpr int q_minb_any(int vpt, int mode) { return (mode == Q_RMSNORM && vpt > 1) ? 1 : 2; }
constexpr int q_minb_256(int mode) { return mode == Q_RMSNORM ? 4 : 8; }

template <int VPT, int MODE>
static void launch_two_warp(const ActQuantArgs& a, cudaStream_t s) {
    launch_pdl(act_quant_kernel<VPT, MODE, GUARD_NONE, kTwoWarpThreads, kTwoWarpMinB>, dim3(a.rows),
               dim3(kTwoWarpThreads), 0, s, a);
}

template <int VPT, int MODE>
static void launch_q_vpt(const ActQuantArgs& a, int threads, cudaStream_t s) {
    const int guard = threads <= 256 ? row_guard_mode(a.nvec, threads, VPT) : GUARD_ALL;
    const dim3 grid(a.rows), block(threads);
    if (guard == GUARD_NONE)
        launch_pdl(act_quant_kernel<VPT, MODE, GUARD_NONE, 256, q_minb_256(MODE)>, grid, block, 0, s, a);
    else if (guard == GUARD_LAST)
        launch_pdl(act_quant_kernel<VPT, MODE, GUARD_LAST, 256, q_minb_256(MODE)>, grid, block, 0, s, a);
    else
        launch_pdl(act_quant_kernel<VPT, MODE, GUARD_ALL, 1024, q_minb_any(VPT, MODE)>, grid, block, 0, s, a);
}

template <int MODE>
static cudaError_t launch_q(const ActQuantArgs& a, cudaStream_t s) {
    if constexpr (MODE != Q_SWIGLU) {
        bool done = true;
        switch (two_warp_vpt(a.rows, a.nvec, MODE)) {
            case 3: launch_two_warp<3, MODE>(a, s); break;
            case 4: launch_two_warp<4, MODE>(a, s); break;
            case 5: launch_two_warp<5, MODE>(a, s); break;
            case 6: launch_two_warp<6, MODE>(a, s); break;
            case 7: launch_two_warp<7, MODE>(a, s); break;
            case 8: launch_two_warp<8, MODE>(a, s); break;
            default: done = false;
        }
        if (done) {
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return cudaGetLastError();
        }
    }
    int threads, vpt;
    row_launch_shape(a.rows, a.nvec, &threads, &vpt);
    switch (vpt) {
        case 1:
            launch_pdl(act_quant_kernel<1, MODE, GUARD_ALL, 1024, q_minb_any(1, MODE)>, dim3(a.rows), dim3(threads), 0,
                       s, a);
            break;
        case 2: launch_q_vpt<2, MODE>(a, threads, s); break;
        case 4: launch_q_vpt<4, MODE>(a, threads, s); break;
        default: return cudaErrorInvalidValue;
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError();
}

}  // namespace vvb

using namespace vvb;

/* mode 0: x -> q8; mode 1: rmsnorm(a [+ b as delta, updated row to row_out]) -> q8;
 * mode 2: swiglu(a = gate, b = up) -> q8. K is a multiple of 32 and all
 * pointers are 16-byte aligned (checked by the caller). */
extern "C" int vvbk_act_quant(int mode, const void* a, const void* b, const void* weight, void* row_out,
                              int M, int K, float eps, int layout,
                              int8_t* xq, float* sx, int32_t* xsum, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    ActQuantArgs q;
    q.a = (const vec16*)a;
    q.b = (const vec16*)b;
    q.xq = xq;
    q.sx = sx;
    q.xsum = xsum;
    q.rows = M;
    q.nvec = K / 8;
    q.layout = layout;
    q.norm = make_row_norm_args(a, b, nullptr, row_out, weight, nullptr, M, K, 0, eps);
    if (mode == Q_RMSNORM) return (int)launch_q<Q_RMSNORM>(q, s);
    if (mode == Q_SWIGLU) return (int)launch_q<Q_SWIGLU>(q, s);
    return (int)launch_q<Q_PLAIN>(q, s);
}

extern "C" int vvbk_col_absmax(const void* x, int M, int K, float* acc, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (K % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
        const int nvec = K / 8;
        const dim3 grid((unsigned)((nvec + kColThreads - 1) / kColThreads),
                        (unsigned)((M + kColRows - 1) / kColRows));
        if (grid.y > 65535u) return (int)cudaErrorInvalidValue;
        launch_pdl(col_absmax_kernel, grid, dim3(kColThreads), 0, s, (const vec16*)x, M, nvec, acc);
    } else {
        const dim3 grid((unsigned)((K + 255) / 256), (unsigned)((M + 63) / 64));
        if (grid.y > 65535u) return (int)cudaErrorInvalidValue;
        launch_pdl(col_absmax_scalar_kernel, grid, dim3(256), 0, s, (const __half*)x, M, K, acc);
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}
