/*
 * row_norm.cu -- the row kernels: RMSNorm, residual add + RMSNorm, embedding
 * gather (+ RMSNorm). sm_100a, HBM-bound, no tensor cores.
 *
 * One row of 3584 halves is 448 16-byte vectors. Two shapes of kernel:
 *
 *   row_norm_warp_kernel<VPT>   one WARP per row, VPT vectors per lane held in
 *       registers, no block-wide barrier; gamma staged once per CTA into
 *       shared memory with cp.async and reused for every row the CTA handles.
 *       Used when there are enough rows to fill the machine with warps
 *       (prefill). A lane has up to 2*VPT 16-byte loads in flight.
 *   row_norm_cta_kernel<VPT>    one CTA per row, one to four vectors per
 *       thread, gamma straight into registers next to the row loads so a
 *       single row costs one DRAM round trip (decode, short slices).
 *   row_norm_generic_kernel     any hidden size / alignment, scalar halves.
 *
 * Arithmetic (identical in all three; mirrors the reference's CPU kernels so
 * results agree bit for bit except on rounding-boundary accidents):
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
#include "vvb_device.cuh"
#include "vvb_launch.h"

#include <atomic>

namespace vvb {

extern std::atomic<uint64_t> g_launches;

struct RowNormArgs {
    const vec16* src;     /* rows or table */
    const vec16* delta;   /* may be null */
    const int32_t* ids;   /* may be null */
    vec16* row_out;       /* may be null */
    const vec16* weight;
    vec16* normed;        /* never null in the norm kernels */
    int rows;
    int nvec;             /* hidden / 8 */
    int hidden;
    int vocab;
    float eps;
};

__device__ __forceinline__ size_t source_row(const RowNormArgs& a, int row) {
    if (a.ids == nullptr) return (size_t)row;
    int id = a.ids[row];
    if (a.vocab > 0) id = min(max(id, 0), a.vocab - 1);
    return (size_t)id;
}

__device__ __forceinline__ float inv_rms(double ss, int hidden, float eps) {
    const float mean = (float)(ss / (double)hidden);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
}

/* Loads this thread's vectors of one row, applies the residual add, stores
 * the updated row, and returns the thread's partial sum of squares. hv[] is
 * left holding the (rounded) row. t = index within the group of G threads. */
template <int VPT>
__device__ __forceinline__ double load_add_square(const RowNormArgs& a, int row, int t, int G,
                                                   vec16 (&hv)[VPT]) {
    const size_t roff = (size_t)row * (size_t)a.nvec;
    const vec16* sp = a.src + source_row(a, row) * (size_t)a.nvec;
    vec16 dv[VPT];
    const bool has_delta = (a.delta != nullptr);
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        const int v = t + j * G;
        hv[j] = (v < a.nvec) ? ld_stream(sp + v) : make_uint4(0, 0, 0, 0);
    }
    if (has_delta) {
        const vec16* dp = a.delta + roff;
#pragma unroll
        for (int j = 0; j < VPT; j++) {
            const int v = t + j * G;
            dv[j] = (v < a.nvec) ? ld_stream(dp + v) : make_uint4(0, 0, 0, 0);
        }
    }
    double ss = 0.0;
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        float f[8];
        unpack8(hv[j], f);
        if (has_delta) {
            float d[8];
            unpack8(dv[j], d);
#pragma unroll
            for (int e = 0; e < 8; e++) f[e] = __fadd_rn(f[e], d[e]);
            hv[j] = pack8(f);       /* round to FP16: this is the new hidden state */
            unpack8(hv[j], f);      /* and the norm sees the rounded values */
        }
#pragma unroll
        for (int e = 0; e < 8; e++) ss = fma((double)f[e], (double)f[e], ss);
    }
    if (a.row_out != nullptr) {
        vec16* rp = a.row_out + roff;
#pragma unroll
        for (int j = 0; j < VPT; j++) {
            const int v = t + j * G;
            if (v < a.nvec) st_stream(rp + v, hv[j]);
        }
    }
    return ss;
}

__device__ __forceinline__ vec16 scale_row_vec(const vec16& h, const vec16& w, float inv) {
    float f[8], g[8];
    unpack8(h, f);
    unpack8(w, g);
#pragma unroll
    for (int e = 0; e < 8; e++) f[e] = __fmul_rn(__fmul_rn(f[e], inv), g[e]);
    return pack8(f);
}

/* ---------------------------------------------------------------- warp/row */
constexpr int kWarpKernelThreads = 128;

template <int VPT>
__device__ __forceinline__ void store_normed_warp(const RowNormArgs& a, int row, int lane,
                                                  const vec16 (&hv)[VPT], const vec16* gamma, float inv) {
    vec16* np_ = a.normed + (size_t)row * (size_t)a.nvec;
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        const int v = lane + j * 32;
        if (v < a.nvec) st_stream(np_ + v, scale_row_vec(hv[j], gamma[v], inv));
    }
}

template <int VPT>
__global__ void __launch_bounds__(kWarpKernelThreads)
row_norm_warp_kernel(const RowNormArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    vec16* gamma = reinterpret_cast<vec16*>(smem_raw);
    for (int v = threadIdx.x; v < a.nvec; v += kWarpKernelThreads) cp_async16(gamma + v, a.weight + v);
    cp_async_commit();

    const int lane = threadIdx.x & 31;
    const int warps_per_cta = kWarpKernelThreads / 32;
    int row = blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const int warp_stride = gridDim.x * warps_per_cta;

    /* First row: its loads are issued before the CTA waits for gamma, so the
     * staging copy and the row loads share one memory round trip. */
    {
        vec16 hv[VPT];
        float inv = 0.0f;
        const bool have = row < a.rows;
        if (have) {
            double ss = load_add_square<VPT>(a, row, lane, 32, hv);
            inv = inv_rms(warp_sum(ss), a.hidden, a.eps);
        }
        cp_async_wait_all();
        __syncthreads();
        if (have) store_normed_warp<VPT>(a, row, lane, hv, gamma, inv);
    }
    for (row += warp_stride; row < a.rows; row += warp_stride) {
        vec16 hv[VPT];
        double ss = load_add_square<VPT>(a, row, lane, 32, hv);
        const float inv = inv_rms(warp_sum(ss), a.hidden, a.eps);
        store_normed_warp<VPT>(a, row, lane, hv, gamma, inv);
    }
}

/* ----------------------------------------------------------------- CTA/row */
template <int VPT>
__global__ void __launch_bounds__(512)
row_norm_cta_kernel(const RowNormArgs a) {
    __shared__ double red[2][32];
    __shared__ float inv_s[2];
    const int t = threadIdx.x, G = blockDim.x;
    const int lane = t & 31, warp = t >> 5, nwarps = G >> 5;

    vec16 wv[VPT];
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        const int v = t + j * G;
        wv[j] = (v < a.nvec) ? __ldg(a.weight + v) : make_uint4(0, 0, 0, 0);
    }
    int parity = 0;
    for (int row = blockIdx.x; row < a.rows; row += gridDim.x, parity ^= 1) {
        vec16 hv[VPT];
        double ss = load_add_square<VPT>(a, row, t, G, hv);
        ss = warp_sum(ss);
        if (lane == 0) red[parity][warp] = ss;
        __syncthreads();
        if (warp == 0) {
            double s = (lane < nwarps) ? red[parity][lane] : 0.0;
            s = warp_sum(s);
            if (lane == 0) inv_s[parity] = inv_rms(s, a.hidden, a.eps);
        }
        __syncthreads();
        const float inv = inv_s[parity];
        vec16* np_ = a.normed + (size_t)row * (size_t)a.nvec;
#pragma unroll
        for (int j = 0; j < VPT; j++) {
            const int v = t + j * G;
            if (v < a.nvec) st_stream(np_ + v, scale_row_vec(hv[j], wv[j], inv));
        }
    }
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
        /* Where the rounded row can be re-read in pass 2: the updated hidden
         * row if one is written, else the source itself (no add happened). */
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
    /* Each CTA copies whole rows; 4 independent 16-byte loads per thread. */
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        int id = ids[row];
        if (vocab > 0) id = min(max(id, 0), vocab - 1);
        const vec16* sp = table + (size_t)id * (size_t)nvec;
        vec16* dp = out + (size_t)row * (size_t)nvec;
        for (int v0 = threadIdx.x; v0 < nvec; v0 += 256 * 4) {
            vec16 r[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int v = v0 + j * 256;
                if (v < nvec) r[j] = ld_stream(sp + v);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int v = v0 + j * 256;
                if (v < nvec) st_stream(dp + v, r[j]);
            }
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
static cudaError_t launch_warp(const RowNormArgs& a, cudaStream_t s) {
    const int rows_per_cta = kWarpKernelThreads / 32;
    const int ctas_needed = (a.rows + rows_per_cta - 1) / rows_per_cta;
    const int resident = sm_count() * 4;
    const int grid = ctas_needed < resident ? ctas_needed : resident;
    const size_t smem = (size_t)a.nvec * sizeof(vec16);
    row_norm_warp_kernel<VPT><<<grid, kWarpKernelThreads, smem, s>>>(a);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError();
}

template <int VPT>
static cudaError_t launch_cta(const RowNormArgs& a, int threads, cudaStream_t s) {
    const int resident = sm_count() * (2048 / threads);
    const int grid = a.rows < resident ? a.rows : resident;
    row_norm_cta_kernel<VPT><<<grid, threads, 0, s>>>(a);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaGetLastError();
}

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
            const int resident = sm_count() * 8;
            const int grid = rows < resident ? rows : resident;
            gather_rows_vec_kernel<<<grid, 256, 0, s>>>((const vec16*)src_rows, ids, (vec16*)row_out,
                                                        rows, nvec, vocab);
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return (int)cudaGetLastError();
        }
        RowNormGenericArgs g{(const __half*)src_rows, (const __half*)delta, ids, (__half*)row_out,
                             (const __half*)weight, nullptr, rows, hidden, vocab, eps};
        const int resident = sm_count() * 8;
        row_norm_generic_kernel<<<rows < resident ? rows : resident, 256, 0, s>>>(g);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return (int)cudaGetLastError();
    }

    if (vec_ok && nvec <= 2048) {
        RowNormArgs a{(const vec16*)src_rows, (const vec16*)delta, ids, (vec16*)row_out,
                      (const vec16*)weight, (vec16*)normed, rows, nvec, hidden, vocab, eps};
        /* Enough rows to give every SM several warps of its own: warp per row. */
        const bool many_rows = rows >= sm_count() * 8;
        if (many_rows && nvec <= 512) {
            const int vpt = (nvec + 31) / 32;
            if (vpt <= 1) return (int)launch_warp<1>(a, s);
            if (vpt <= 2) return (int)launch_warp<2>(a, s);
            if (vpt <= 4) return (int)launch_warp<4>(a, s);
            if (vpt <= 7) return (int)launch_warp<7>(a, s);
            if (vpt <= 8) return (int)launch_warp<8>(a, s);
            if (vpt <= 14) return (int)launch_warp<14>(a, s);
            return (int)launch_warp<16>(a, s);
        }
        int threads = ((nvec + 31) / 32) * 32;
        if (threads > 512) threads = 512;
        const int vpt = (nvec + threads - 1) / threads;
        if (vpt <= 1) return (int)launch_cta<1>(a, threads, s);
        if (vpt <= 2) return (int)launch_cta<2>(a, threads, s);
        return (int)launch_cta<4>(a, threads, s);
    }

    /* Scalar path. With a delta, the rounded sum must be re-readable in the
     * second pass, so it needs a row_out buffer (the entry points always pass
     * hidden as row_out when they pass a delta). */
    RowNormGenericArgs g{(const __half*)src_rows, (const __half*)delta, ids, (__half*)row_out,
                         (const __half*)weight, (__half*)normed, rows, hidden, vocab, eps};
    const int resident = sm_count() * 8;
    row_norm_generic_kernel<<<rows < resident ? rows : resident, 256, 0, s>>>(g);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}
