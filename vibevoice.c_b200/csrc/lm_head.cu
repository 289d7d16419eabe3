/*
 * lm_head.cu -- the decode step's tail: final RMSNorm of the last hidden row,
 * logits = W[V,K] @ x[K], and the greedy argmax. sm_100a, HBM-bound: the FP16
 * head of the 7B model is 1.09 GB read once per token
 * (src/inference/pipeline.c:1962-1986, src/cuda/lm_head.cu:28-96).
 *
 *   lm_head_kernel<NORM>   a grid of exactly the CTAs that fit on the GPU at
 *       once (2 per SM), each owning an equal contiguous block of W's rows, so
 *       x is staged once per CTA and all CTAs finish together; the 8 warps of
 *       a CTA take row pairs round-robin, a lane keeping 14 x 2 16-byte loads
 *       in flight for K = 3584. x sits in shared memory as floats -- with NORM
 *       the CTA first applies the final RMSNorm to the hidden row (row_norm.cuh's
 *       arithmetic, rounded to FP16 as vv_rmsnorm_dev would store it), a 7 KB
 *       L2 read per CTA instead of a separate launch. FP32
 *       multiply-add per element, warp-shuffle sum, FP32 logit. Each CTA also
 *       leaves its best (value, index) in a partials array, so the argmax needs
 *       no pass over the logits.
 *   argmax_reduce_kernel   one CTA reduces the partials (or 256 of them).
 *   argmax_logits_kernel   stage 1 of the stand-alone vv_argmax_dev.
 *
 * Ties go to the smaller index (the reference's reductions leave ties to the
 * thread layout, src/cuda/lm_head.cu:65-118; its CPU path to the OpenMP
 * schedule, src/cpu/cpu_kernels.c:1570-1606).
 */
#include "row_norm.cuh"
#include "vvb_launch.h"

#include <atomic>
#include <cfloat>

namespace vvb {

extern std::atomic<uint64_t> g_launches;

constexpr int kLmThreads = 256;
constexpr int kLmMinRowsPerCta = 32;   /* bounds the number of partials: ceil(V / 32) */
constexpr int kLmPrefetchBytes = 256 * 1024;   /* per CTA, into L2, during the prologue (296 CTAs: 76 MB) */

struct Best {
    float v;
    int i;
};
__device__ __forceinline__ Best better(Best a, Best b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ Best warp_best(Best b) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        Best other;
        other.v = __shfl_xor_sync(0xffffffffu, b.v, o);
        other.i = __shfl_xor_sync(0xffffffffu, b.i, o);
        b = better(b, other);
    }
    return b;
}

struct LmHeadArgs {
    const vec16* x;        /* [K] FP16: the normed row, or (NORM) the hidden row */
    const vec16* norm_w;   /* NORM only */
    const vec16* W;        /* [V, K] */
    float* logits;         /* may be null */
    float* part_v;         /* [gridDim.x] or null */
    int* part_i;
    int V, K, nvec;
    int rows_per_cta;      /* even; gridDim.x * rows_per_cta >= V */
    float eps;
};

template <bool NORM>
__global__ void __launch_bounds__(kLmThreads, 2)
lm_head_kernel(const LmHeadArgs a) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ __align__(16) float xs[];          /* K floats */
    __shared__ double red[8];
    __shared__ float inv_s;
    __shared__ Best cta_best[8];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    /* this CTA's contiguous block of rows */
    const int cta_lo = blockIdx.x * a.rows_per_cta;
    const int cta_hi = min(a.V, cta_lo + a.rows_per_cta);

    /* While x is staged (and normalised: two barriers and a double-precision
     * reduction, a few microseconds in which the CTA would load nothing), pull
     * the head of this CTA's block of W into L2. */
    if (cta_lo < cta_hi) {
        const char* wbase = reinterpret_cast<const char*>(a.W + (size_t)cta_lo * (size_t)a.nvec);
        size_t bytes = (size_t)(cta_hi - cta_lo) * (size_t)a.nvec * sizeof(vec16);
        if (bytes > (size_t)kLmPrefetchBytes) bytes = (size_t)kLmPrefetchBytes;
        for (size_t off = (size_t)t * 128u; off < bytes; off += (size_t)kLmThreads * 128u)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(wbase + off));
    }

    /* stage x (normalised if asked) as floats */
    if (NORM) {
        double ss = 0.0;
        for (int v = t; v < a.nvec; v += kLmThreads) {
            float f[8];
            unpack8(__ldg(a.x + v), f);
#pragma unroll
            for (int e = 0; e < 8; e++) ss = fma((double)f[e], (double)f[e], ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (t < 32) {
            double s = (t < 8) ? red[t] : 0.0;
            s = warp_sum(s);
            if (t == 0) inv_s = inv_rms(s, a.K, a.eps);
        }
        __syncthreads();
        const float inv = inv_s;
        for (int v = t; v < a.nvec; v += kLmThreads) {
            float f[8];
            unpack8(scale_row_vec(__ldg(a.x + v), __ldg(a.norm_w + v), inv), f);   /* rounded to FP16, then widened */
#pragma unroll
            for (int e = 0; e < 8; e++) xs[v * 8 + e] = f[e];
        }
    } else {
        for (int v = t; v < a.nvec; v += kLmThreads) {
            float f[8];
            unpack8(__ldg(a.x + v), f);
#pragma unroll
            for (int e = 0; e < 8; e++) xs[v * 8 + e] = f[e];
        }
    }
    __syncthreads();

    Best best{-FLT_MAX, 0x7fffffff};
    /* the CTA's 8 warps take row pairs of its block round-robin */
    for (int r0 = cta_lo + 2 * warp; r0 < cta_hi; r0 += 2 * (kLmThreads / 32)) {
        const int r1 = r0 + 1;
        const bool two = r1 < cta_hi;
        const vec16* w0 = a.W + (size_t)r0 * (size_t)a.nvec;
        const vec16* w1 = a.W + (size_t)(two ? r1 : r0) * (size_t)a.nvec;
        float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll 7
        for (int v = lane; v < a.nvec; v += 32) {
            const vec16 p0 = ld_stream(w0 + v);
            const vec16 p1 = ld_stream(w1 + v);
            const float4 xa = *reinterpret_cast<const float4*>(xs + v * 8);
            const float4 xb = *reinterpret_cast<const float4*>(xs + v * 8 + 4);
            float f0[8], f1[8];
            unpack8(p0, f0);
            unpack8(p1, f1);
            const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
            for (int e = 0; e < 8; e++) {
                acc0 = fmaf(f0[e], xv[e], acc0);
                acc1 = fmaf(f1[e], xv[e], acc1);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            acc0 += __shfl_xor_sync(0xffffffffu, acc0, o);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, o);
        }
        if (lane == 0) {
            if (a.logits) {
                a.logits[r0] = acc0;
                if (two) a.logits[r1] = acc1;
            }
            best = better(best, Best{acc0, r0});
            if (two) best = better(best, Best{acc1, r1});
        }
    }
    if (a.part_v == nullptr) return;
    if (lane == 0) cta_best[warp] = best;
    __syncthreads();
    if (t == 0) {
        Best b = cta_best[0];
#pragma unroll
        for (int w = 1; w < 8; w++) b = better(b, cta_best[w]);
        a.part_v[blockIdx.x] = b.v;
        a.part_i[blockIdx.x] = b.i;
    }
}

/* Any K / alignment: one warp per row, scalar halves, x from global memory. */
__global__ void __launch_bounds__(256)
lm_head_scalar_kernel(const __half* x, const __half* W, float* logits, int V, int K) {
    pdl_wait();
    pdl_trigger();
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= V) return;
    const int lane = threadIdx.x & 31;
    const __half* w = W + (size_t)row * (size_t)K;
    float acc = 0.0f;
    for (int k = lane; k < K; k += 32) acc = fmaf(__half2float(w[k]), __half2float(x[k]), acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) logits[row] = acc;
}

/* Stage 1 of the stand-alone argmax: gridDim.x partials over FP32 logits. */
__global__ void __launch_bounds__(256)
argmax_logits_kernel(const float* __restrict__ logits, int V, float* part_v, int* part_i) {
    pdl_wait();
    pdl_trigger();
    __shared__ Best wb[8];
    Best best{-FLT_MAX, 0x7fffffff};
    for (int i = blockIdx.x * 256 + threadIdx.x; i < V; i += gridDim.x * 256)
        best = better(best, Best{logits[i], i});
    best = warp_best(best);
    if ((threadIdx.x & 31) == 0) wb[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        Best b = wb[0];
#pragma unroll
        for (int w = 1; w < 8; w++) b = better(b, wb[w]);
        part_v[blockIdx.x] = b.v;
        part_i[blockIdx.x] = b.i;
    }
}

/* Final stage: one CTA over n partials. An index of 0x7fffffff (no candidate
 * beat -FLT_MAX) is reported as 0, like the reference's initial value. */
__global__ void __launch_bounds__(1024)
argmax_reduce_kernel(const float* part_v, const int* part_i, int n, int* out_token, float* out_value) {
    pdl_wait();
    pdl_trigger();
    __shared__ Best wb[32];
    Best best{-FLT_MAX, 0x7fffffff};
    for (int i = threadIdx.x; i < n; i += 1024) best = better(best, Best{part_v[i], part_i[i]});
    best = warp_best(best);
    if ((threadIdx.x & 31) == 0) wb[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x < 32) {
        Best b = wb[threadIdx.x];
        b = warp_best(b);
        if (threadIdx.x == 0) {
            *out_token = (b.i == 0x7fffffff) ? 0 : b.i;
            if (out_value) *out_value = b.v;
        }
    }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace vvb

using namespace vvb;

/* Upper bound on the number of CTAs (= argmax partials) a launch over V rows uses. */
extern "C" int vvbk_lm_head_partials(int V) { return (V + kLmMinRowsPerCta - 1) / kLmMinRowsPerCta; }

/* CTAs of lm_head_kernel<NORM> resident at once on the current device for
 * `smem` bytes of dynamic shared memory. The answer is cached per host thread
 * (keyed by device, variant and size), so the one-row decode path -- where
 * this launch is latency-sensitive and runs once per token -- makes no runtime
 * query after its first call. A query that fails falls back to one CTA per SM
 * of a 148-SM part and clears the runtime's last-error slot, so that the
 * launch that follows is not reported as failed. */
template <bool NORM>
static int lm_head_resident_ctas(size_t smem) {
    static thread_local int c_dev = -1, c_ctas = 0;
    static thread_local size_t c_smem = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return 148;
    }
    if (dev == c_dev && smem == c_smem && c_ctas > 0) return c_ctas;
    int sms = 148, per_sm = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
        (void)cudaGetLastError();
        sms = 148;
    }
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lm_head_kernel<NORM>, kLmThreads, smem) != cudaSuccess ||
        per_sm < 1) {
        (void)cudaGetLastError();
        per_sm = 1;
    }
    c_dev = dev;
    c_smem = smem;
    c_ctas = sms * per_sm;
    return c_ctas;
}

/* logits (may be NULL) and/or per-CTA argmax partials (part_v/part_i, may be
 * NULL; at most vvbk_lm_head_partials(V) entries each, the number written
 * comes back in *n_partials). norm_w != NULL: x is the
 * hidden row and the final RMSNorm is applied first. Returns
 * cudaErrorNotSupported when the fast form does not fit and partials or the
 * norm were asked for (the scalar form only writes logits). */
extern "C" int vvbk_lm_head(const void* x, const void* norm_w, float eps, const void* W, float* logits,
                            float* part_v, int* part_i, int* n_partials, int V, int K, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    if (n_partials) *n_partials = 0;
    const bool fast = K % 8 == 0 && K <= 11264 &&   /* K floats of shared memory, under 48 KB with the statics */
                      aligned16(x) && aligned16(W) && aligned16(norm_w);
    if (!fast) {
        if (part_v || norm_w || !logits) return (int)cudaErrorNotSupported;
        launch_pdl(lm_head_scalar_kernel, dim3((V + 7) / 8), dim3(256), 0, s, (const __half*)x, (const __half*)W, logits, V, K);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return (int)cudaGetLastError();
    }
    const size_t smem = (size_t)K * sizeof(float);
    /* equal blocks of rows over the CTAs that are resident at once, never fewer than 32 rows each */
    const int resident = norm_w ? lm_head_resident_ctas<true>(smem) : lm_head_resident_ctas<false>(smem);
    int rows_per_cta = (V + resident - 1) / resident;
    if (rows_per_cta < kLmMinRowsPerCta) rows_per_cta = kLmMinRowsPerCta;
    rows_per_cta += rows_per_cta & 1;
    const int grid = (V + rows_per_cta - 1) / rows_per_cta;
    if (n_partials) *n_partials = grid;      /* entries of part_v / part_i this launch writes */
    LmHeadArgs a{(const vec16*)x, (const vec16*)norm_w, (const vec16*)W, logits, part_v, part_i,
                 V, K, K / 8, rows_per_cta, eps};
    if (norm_w) launch_pdl(lm_head_kernel<true>, dim3(grid), dim3(kLmThreads), smem, s, a);
    else launch_pdl(lm_head_kernel<false>, dim3(grid), dim3(kLmThreads), smem, s, a);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

extern "C" int vvbk_argmax_logits(const float* logits, int V, float* part_v, int* part_i, int nparts, void* stream) {
    launch_pdl(argmax_logits_kernel, dim3(nparts), dim3(256), 0, (cudaStream_t)stream, logits, V, part_v, part_i);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

extern "C" int vvbk_argmax_reduce(const float* part_v, const int* part_i, int n, int* out_token, float* out_value,
                                  void* stream) {
    launch_pdl(argmax_reduce_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, part_v, part_i, n, out_token, out_value);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

/* ------------------------------------------------------------------------
 * The same final norm + head + argmax for callers that have no device memory
 * to give and no way to get any.
 *
 * Who that is: a decode loop whose engine carved its whole device budget into
 * one workspace when the model was loaded and hands each op nothing but input
 * and output pointers (the reference sizes every buffer once at start-up and
 * never allocates while a token is in flight), or a host application that
 * embeds this library behind a callback and keeps its allocator out of reach.
 * Asking the CUDA runtime for memory from such a place is not an option: the
 * budget may already be spent, and cudaMalloc / cudaFree stall every stream of
 * the device while they run, in the middle of a token.
 *
 * So the argmax partials live in the array below, which is part of the
 * library image: every GPU that loads the library sets aside these 64 KB until
 * the process exits. That bounds the head this entry point accepts to
 * VVB_LM_HEAD_STATIC_MAX_V rows (8192 partials of 32 rows); taller heads are
 * refused with VV_ERR_OVERFLOW and belong to vvb_lm_head_argmax_dev.
 *
 * In host code `g_lm_head_partials` is only a handle for the symbol, not a
 * device address, so the address is looked up with cudaGetSymbolAddress -- once
 * per device, by the first call made while that device is current, and kept in
 * a table indexed by device. That first call talks to the runtime beyond a
 * plain launch, so make it during start-up, before any stream capture. The
 * table is never refreshed: the library must not be kept across a
 * cudaDeviceReset (or any other teardown of the device's primary context),
 * after which the array lives at an address the table no longer knows.
 *
 * Every call on a device writes into the one array. Nothing in it has to
 * start at zero (each launch overwrites exactly the entries its reduce step
 * reads), but two calls that overlap on the same GPU -- different streams, or
 * different host threads -- race on it and can return each other's winner. Run
 * them on one stream, or give all but one of them their own scratch through
 * vvb_lm_head_argmax_dev.
 */
#include "vvb200.h"

namespace vvb {
constexpr int kStaticPartials = VVB_LM_HEAD_STATIC_MAX_V / kLmMinRowsPerCta;          /* 8192 */
static __device__ __align__(256) unsigned char g_lm_head_partials[kStaticPartials * (sizeof(float) + sizeof(int))];

constexpr int kMaxDevices = 64;
static std::atomic<void*> g_lm_head_partials_addr[kMaxDevices];   /* device address of the array, per device */

/* Device address of the static array on the CURRENT device (looked up once). */
static cudaError_t static_partials(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    void* p = g_lm_head_partials_addr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        e = cudaGetSymbolAddress(&p, g_lm_head_partials);
        if (e != cudaSuccess) return e;
        g_lm_head_partials_addr[dev].store(p, std::memory_order_release);   /* racing first calls store the same value */
    }
    *out = p;
    return cudaSuccess;
}
}  // namespace vvb

extern "C" vv_status_t vvb_lm_head_argmax_static_dev(const void* x, const void* final_norm_w, float eps,
                                                     const void* W, int V, int K, void* logits,
                                                     int32_t* out_token, float* out_value, void* stream) {
    if (!x || !W || !out_token) return VV_ERR_NULL_PTR;
    if (V <= 0 || K <= 0) return VV_ERR_INVALID_ARG;
    if (V > VVB_LM_HEAD_STATIC_MAX_V) return VV_ERR_OVERFLOW;       /* more partials than the array holds */
    void* scratch = nullptr;
    if (static_partials(&scratch) != cudaSuccess || scratch == nullptr) return VV_ERR_CUDA;
    float* part_v = (float*)scratch;
    int* part_i = (int*)(part_v + kStaticPartials);
    int n = 0;
    int err = vvbk_lm_head(x, final_norm_w, eps, W, (float*)logits, part_v, part_i, &n, V, K, stream);
    if (err == (int)cudaErrorNotSupported) return VV_ERR_UNSUPPORTED;   /* K % 8, K > 11264 or alignment */
    if (err == 0) err = vvbk_argmax_reduce(part_v, part_i, n, (int*)out_token, out_value, stream);
    return err == 0 ? VV_OK : VV_ERR_CUDA_LAUNCH;
}
