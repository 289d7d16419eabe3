/*
 * row_norm.cu -- the row kernels: RMSNorm, residual add + RMSNorm, embedding
 * gather (+ RMSNorm). sm_100a, HBM-bound, no tensor cores.
 *
 *   row_norm_cta_kernel<VPT>   one CTA per row, VPT 16-byte vectors per thread
 *       held in registers, gamma straight into registers beside the row loads
 *       (it stays L1/L2-resident), warp-shuffle + one shared-memory step for
 *       the sum of squares. The grid is one CTA per row and nothing loops, so
 *       the hardware's CTA scheduler balances rows over SMs and the tail is one
 *       row long. Measured on B200 for 3584-wide rows: 128 threads x 4 vectors
 *       (9 rows resident per SM) streams at the copy rate; more bytes per
 *       thread (a warp per row, 14 vectors per lane) or fewer (448 threads x 1)
 *       both lose 15-25 % when there are many rows.
 *   row_norm_generic_kernel    any hidden size / alignment, scalar halves.
 *   gather_rows_vec_kernel     the plain embedding gather.
 *
 * Arithmetic (identical in all; mirrors the reference's CPU kernels so results
 * agree bit for bit except on rounding-boundary accidents):
 *   h'  = f16(float(h) + float(delta))          src/cuda/conv_vae.cu:29-31
 *   ss  = sum over the ROUNDED h' of h'*h' in double
 *                                               src/cpu/cpu_kernels.c:1444-1445
 *   inv = 1.0f / sqrtf((float)(ss / n) + eps)   src/cpu/cpu_kernels.c:1446
 *   y   = f16((h' * inv) * w)                   src/cpu/cpu_kernels.c:1448
 * Squares of halves are exact in double, so only the order of the double
 * additions differs from the CPU loop (relative 1e-16, far below one float
 * ulp of the mean).
 *
 * Aliasing: every thread reads all of its vectors of a row before it writes
 * any, and it writes exactly the indices it read, so delta == normed and
 * input == output are safe.
 */
#include "row_norm.cuh"
#include "vvb_launch.h"

#include <atomic>

namespace vvb {

extern std::atomic<uint64_t> g_launches;

/* ----------------------------------------------------------------- CTA/row */
/* MAXT: the largest CTA the instance is launched with; MINB: CTAs per SM it is
 * compiled for (a register budget of 65536 / (MAXT * MINB)). The one-vector
 * instance serves the grids of at most one wave, and "one wave" (kLatencyRows)
 * counts four 448-thread CTAs per SM, which needs 32 registers: at 37 the 512
 * rows of a short prefill take two waves and 3.4 us instead of 2.7 us. */
template <int VPT, int GUARD, int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB)
row_norm_cta_kernel(const RowNormArgs a) {
    pdl_wait();
    pdl_trigger();
    row_norm_body<VPT, 1, GUARD>(a, blockIdx.x, threadIdx.x, blockDim.x, 0);
}

/* The norm WITHOUT an addend moves half the bytes per row, so at the same
 * residency it has half the loads in flight (37.1 us for [14449, 3584] in the
 * general instance; the roofline is 31.7). This instance reserves no registers
 * for an addend, fetches gamma after the reduction and is compiled for five
 * 256-thread CTAs per SM (48 registers: ten 128-thread rows resident instead
 * of eight): 35.6 us. Measured beside it: four CTAs with the late gamma 36.5,
 * five without it 45.1 (spills), six 40.6, eight 63.2. */
template <int VPT, int GUARD>
__global__ void __launch_bounds__(256, 5)
row_norm_plain_kernel(const RowNormArgs a) {
    pdl_wait();
    pdl_trigger();
    row_norm_body<VPT, 1, GUARD, true, 0>(a, blockIdx.x, threadIdx.x, blockDim.x, 0);
}

/* ... and when the row splits into whole vectors over 64 threads (hidden sizes
 * 1536 .. 4096 in steps of 512) it runs as TWO WARPS PER ROW, 3 .. 8 vectors per
 * thread, twelve such rows resident per SM: 32.8 us for [14449, 3584] (0.97 of
 * the measured copy rate) against 35.5 for the instance above; compiled for 16
 * CTAs per SM (64 registers) 35.0. The same shape WITH an addend is slower than
 * 128 threads x 4 (64.6 against 62.7 us), so the add + norm keeps that. */
constexpr int kTwoWarpThreads = 64;
template <int VPT>
__global__ void __launch_bounds__(kTwoWarpThreads, 12)
row_norm_two_warp_kernel(const RowNormArgs a) {
    pdl_wait();
    pdl_trigger();
    row_norm_body<VPT, 1, GUARD_NONE, true, 0>(a, blockIdx.x, threadIdx.x, kTwoWarpThreads, 0);
}

/* ----------------------------------------------------------------- generic */
struct RowNormGenericArgs {
    const __half* src;
    const __half* delta;
    const int32_t* ids;
    __half* row_out;
    const __half* weight;
    __half* normed;
    int rows, hidden, vocab;
    float eps;
};

__global__ void __launch_bounds__(256)
row_norm_generic_kernel(const RowNormGenericArgs a) {
    pdl_wait();
    pdl_trigger();
    __shared__ double red[8];
    __shared__ float inv_s;
    const int t = threadIdx.x;
    for (int row = blockIdx.x; row < a.rows; row += gridDim.x) {
        size_t srow = (size_t)row;
        if (a.ids) {
            int id = a.ids[row];
            if (a.vocab > 0) id = min(max(id, 0), a.vocab - 1);
            srow = (size_t)id;
        }
        const __half* sp = a.src + srow * (size_t)a.hidden;
        const size_t roff = (size_t)row * (size_t)a.hidden;
        double ss = 0.0;
        for (int i = t; i < a.hidden; i += 256) {
            float f = __half2float(sp[i]);
            if (a.delta) {
                const __half r = __float2half_rn(__fadd_rn(f, __half2float(a.delta[roff + i])));
                f = __half2float(r);
                if (a.row_out) a.row_out[roff + i] = r;
            } else if (a.row_out) {
                a.row_out[roff + i] = sp[i];
            }
            ss = fma((double)f, (double)f, ss);
        }
        if (a.normed == nullptr) continue;
        ss = warp_sum(ss);
        if ((t & 31) == 0) red[t >> 5] = ss;
        __syncthreads();
        if (t < 32) {
            double s = (t < 8) ? red[t] : 0.0;
            s = warp_sum(s);
            if (t == 0) inv_s = inv_rms(s, a.hidden, a.eps);
        }
        __syncthreads();
        const float inv = inv_s;
        /* Pass 2 re-reads what this same thread produced in pass 1 (same
         * indices), so its own earlier writes are visible without a fence.
         * With a delta the rounded sum lives in row_out (the caller passes
         * hidden as both src and row_out); without one, in src. */
        const __half* hp = (a.delta != nullptr) ? (a.row_out + roff) : sp;
        for (int i = t; i < a.hidden; i += 256) {
            const float f = __half2float(hp[i]);
            a.normed[roff + i] =
                __float2half_rn(__fmul_rn(__fmul_rn(f, inv), __half2float(a.weight[i])));
        }
        __syncthreads();   /* red/inv_s are reused by the next row */
    }
}

/* ------------------------------------------------------------ plain gather */
__global__ void __launch_bounds__(256)
gather_rows_vec_kernel(const vec16* __restrict__ table, const int32_t* __restrict__ ids,
                       vec16* __restrict__ out, int rows, int nvec, int vocab) {
    pdl_wait();
    pdl_trigger();
    /* One CTA per row; 4 independent 16-byte loads per thread per trip. */
    const int row = blockIdx.x;
    int id = ids[row];
    const int far_id = gather_far_id(ids, row, rows, vocab);
    if (vocab > 0) id = min(max(id, 0), vocab - 1);
    const vec16* sp = table + (size_t)id * (size_t)nvec;
    vec16* dp = out + (size_t)row * (size_t)nvec;
    for (int v0 = threadIdx.x; v0 < nvec; v0 += blockDim.x * 4) {
        vec16 r[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int v = v0 + j * blockDim.x;
            if (v < nvec) r[j] = ld_stream(sp + v);
        }
        if (v0 == (int)threadIdx.x) gather_prefetch(table, far_id, nvec, threadIdx.x, blockDim.x);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int v = v0 + j * blockDim.x;
            if (v < nvec) st_stream(dp + v, r[j]);
        }
    }
}

/* ------------------------------------------------------------------ launch */
static int sm_count() {
    /* Per-thread cache keyed by device: no shared mutable state. */
    static thread_local int cached_dev = -1, cached_sms = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached_dev = dev;
        cached_sms = n;
    }
    return cached_sms;
}

template <int VPT>
static void launch_cta_vpt(const RowNormArgs& a, int threads, cudaStream_t s) {
    const int guard = threads <= 256 ? row_guard_mode(a.nvec, threads, VPT) : GUARD_ALL;
    const dim3 grid(a.rows), block(threads);
    if (a.delta == nullptr && a.ids == nullptr && guard != GUARD_ALL) {
        if (guard == GUARD_NONE) launch_pdl(row_norm_plain_kernel<VPT, GUARD_NONE>, grid, block, 0, s, a);
        else launch_pdl(row_norm_plain_kernel<VPT, GUARD_LAST>, grid, block, 0, s, a);
        return;
    }
    if (guard == GUARD_NONE) launch_pdl(row_norm_cta_kernel<VPT, GUARD_NONE, 256, 4>, grid, block, 0, s, a);
    else if (guard == GUARD_LAST) launch_pdl(row_norm_cta_kernel<VPT, GUARD_LAST, 256, 4>, grid, block, 0, s, a);
    else launch_pdl(row_norm_cta_kernel<VPT, GUARD_ALL, 1024, 1>, grid, block, 0, s, a);
}

static cudaError_t launch_cta(const RowNormArgs& a, int vpt, int threads, cudaStream_t s) {
    if (a.rows > kLatencyRows && a.ids == nullptr && a.delta == nullptr && a.nvec % kTwoWarpThreads == 0) {
        const dim3 grid(a.rows), block(kTwoWarpThreads);
        bool done = true;
        switch (a.nvec / kTwoWarpThreads) {
            case 3: launch_pdl(row_norm_two_warp_kernel<3>, grid, block, 0, s, a); break;
            case 4: launch_pdl(row_norm_two_warp_kernel<4>, grid, block, 0, s, a); break;
            case 5: launch_pdl(row_norm_two_warp_kernel<5>, grid, block, 0, s, a); break;
            case 6: launch_pdl(row_norm_two_warp_kernel<6>, grid, block, 0, s, a); break;
            case 7: launch_pdl(row_norm_two_warp_kernel<7>, grid, block, 0, s, a); break;
            case 8: launch_pdl(row_norm_two_warp_kernel<8>, grid, block, 0, s, a); break;
            default: done = false;
        }
        if (done) {
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return cudaGetLastError();
        }
    }
    switch (vpt) {
        case 1: launch_pdl(row_norm_cta_kernel<1, GUARD_ALL, 1024, 2>, dim3(a.rows), dim3(threads), 0, s, a); break;
        case 2: launch_cta_vpt<2>(a, threads, s); break;
        case 4: launch_cta_vpt<4>(a, threads, s); break;
        default: return cudaErrorInvalidValue;
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError();
}

static int round_up_warp(int n) { return ((n + 31) / 32) * 32; }

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace vvb

using namespace vvb;

extern "C" int vvbk_row_norm(const void* src_rows, const void* delta, const int32_t* ids, int vocab,
                             void* row_out, const void* weight, void* normed,
                             int rows, int hidden, float eps, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (rows <= 0 || hidden <= 0) return (int)cudaSuccess;
    const bool vec_ok = (hidden % 8 == 0) && aligned16(src_rows) && aligned16(delta) &&
                        aligned16(row_out) && aligned16(weight) && aligned16(normed);
    const int nvec = hidden / 8;

    if (normed == nullptr) {
        /* gather (or add) without a norm */
        if (ids != nullptr && delta == nullptr && vec_ok) {
            int threads = round_up_warp((nvec + 3) / 4);
            if (threads > 256) threads = 256;
            launch_pdl(gather_rows_vec_kernel, dim3(rows), dim3(threads), 0, s, (const vec16*)src_rows, ids, (vec16*)row_out,
                                                            rows, nvec, vocab);
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return (int)cudaGetLastError();
        }
        RowNormGenericArgs g{(const __half*)src_rows, (const __half*)delta, ids, (__half*)row_out,
                             (const __half*)weight, nullptr, rows, hidden, vocab, eps};
        const int resident = sm_count() * 8;
        launch_pdl(row_norm_generic_kernel, dim3(rows < resident ? rows : resident), dim3(256), 0, s, g);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return (int)cudaGetLastError();
    }

    if (vec_ok && nvec <= 4096) {
        const RowNormArgs a = make_row_norm_args(src_rows, delta, ids, row_out, weight, normed, rows, hidden, vocab, eps);
        /* A quarter of the row's vectors per thread (128 threads x 4 for a
         * 3584-wide row) is fastest once the grid is several waves deep
         * (62.2 us against 63.4 and 81.7 for 2 and 1 at 14449 rows). Up to a
         * few hundred rows the kernel is one wave of latency, and a thread
         * that owns one vector has a quarter of the serial work: 1.88 against
         * 2.06 us at one row (the decode shape), 4.27 against 4.55 at 512. */
        int threads, vpt;
        row_launch_shape(rows, nvec, &threads, &vpt);
        return (int)launch_cta(a, vpt, threads, s);
    }

    /* Scalar path. With a delta, the rounded sum must be re-readable in the
     * second pass, so it needs a row_out buffer (the entry points always pass
     * hidden as row_out when they pass a delta). */
    RowNormGenericArgs g{(const __half*)src_rows, (const __half*)delta, ids, (__half*)row_out,
                         (const __half*)weight, (__half*)normed, rows, hidden, vocab, eps};
    const int resident = sm_count() * 8;
    launch_pdl(row_norm_generic_kernel, dim3(rows < resident ? rows : resident), dim3(256), 0, s, g);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}
