/*
 * swiglu_bulk.cu -- EXPERIMENT, compiled only with -DVVB_TUNING: SwiGLU with
 * its loads staged through shared memory by the bulk-copy engine
 * (cp.async.bulk global -> shared, completion on an mbarrier), to measure that
 * form against the 16-byte LDG stream of swiglu.cu on the same inputs.
 *
 * Result on B200 (graph replay, [14449, 18944] in place, bit-identical
 * outputs): the LDG stream 230.4 us = 7128 GB/s; this kernel, best of six
 * (vectors per thread x stages) shapes, 273.5 us = 6005 GB/s ([4096, 18944]:
 * 66.4 against 78.6 us). The shipped library therefore keeps the LDG stream and
 * this file stays out of the product build. To repeat: build with
 * EXTRA_NVCCFLAGS=-DVVB_TUNING and set VVB_TUNE_SWIGLU_BULK to 10 x vectors
 * per thread + stages (43, 42, 24, 26, 18, 84), then time vv_swiglu_dev.
 *
 * Persistent CTAs (grid = CTAs resident at once) walk tiles of kTileVecs
 * 16-byte vectors of gate and of up; a ring of kStages stages per CTA; thread 0
 * is the producer (arrive.expect_tx + two bulk copies per tile), every thread
 * consumes: wait on the stage's barrier, read its vectors from shared memory,
 * __syncthreads (the stage is free again), thread 0 refills it with the tile
 * kStages ahead, then compute and store with st.global.cs. Every wait is
 * bounded: after kSpinLimit failed polls a thread raises g_bulk_error and the
 * CTA leaves through a bounded drain of the copies still in flight.
 */
#ifdef VVB_TUNING
#include "swiglu.cuh"
#include "vvb_launch.h"

#include <atomic>

namespace vvb {

extern std::atomic<uint64_t> g_launches;

constexpr int kBulkThreads = 256;
constexpr unsigned kSpinLimit = 1u << 20;   /* try_wait suspends for a while per poll */

__device__ unsigned int g_bulk_error = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
/* Bounded wait; false when it gave up. */
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
    for (unsigned i = 0; i < kSpinLimit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src_gmem, unsigned bytes, uint64_t* bar, uint64_t pol) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(pol) : "memory");
}

template <int kBulkVecsPerThread, int kStages>
__global__ void __launch_bounds__(kBulkThreads)
swiglu_bulk_kernel(const vec16* gate, const vec16* up, vec16* out, size_t nvec) {
    constexpr int kTileVecs = kBulkThreads * kBulkVecsPerThread;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    vec16* g_s = reinterpret_cast<vec16*>(smem_raw);                       /* [kStages][kTileVecs] */
    vec16* u_s = g_s + kStages * kTileVecs;
    __shared__ __align__(8) uint64_t full[kStages];
    pdl_wait();
    pdl_trigger();
    const int t = threadIdx.x;
    const uint64_t pol = policy_evict_first();
    const size_t ntiles = (nvec + kTileVecs - 1) / kTileVecs;
    if (t == 0) {
        for (int s = 0; s < kStages; s++) mbar_init(&full[s], 1);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   /* the init, seen by the copy engine */
    }
    __syncthreads();

    auto issue = [&](size_t tile, int s) {
        const size_t v0 = tile * kTileVecs;
        const unsigned nv = (unsigned)((nvec - v0 < (size_t)kTileVecs) ? (nvec - v0) : (size_t)kTileVecs);
        mbar_expect_tx(&full[s], nv * 32u);
        bulk_load(g_s + s * kTileVecs, gate + v0, nv * 16u, &full[s], pol);
        bulk_load(u_s + s * kTileVecs, up + v0, nv * 16u, &full[s], pol);
    };

    /* prologue: fill the ring */
    int issued = 0;                       /* tiles this CTA has requested (thread 0's count) */
    if (t == 0) {
        for (int s = 0; s < kStages; s++) {
            const size_t tile = (size_t)blockIdx.x + (size_t)s * gridDim.x;
            if (tile < ntiles) { issue(tile, s); issued++; }
        }
    }

    int k = 0;                            /* tiles this CTA has consumed */
    bool failed = false;
    for (size_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, k++) {
        const int s = k % kStages;
        const unsigned parity = (unsigned)(k / kStages) & 1u;
        if (!mbar_wait(&full[s], parity)) { failed = true; break; }
        const size_t v0 = tile * kTileVecs;
        vec16 gv[kBulkVecsPerThread], uv[kBulkVecsPerThread];
#pragma unroll
        for (int j = 0; j < kBulkVecsPerThread; j++) {
            gv[j] = g_s[s * kTileVecs + t + j * kBulkThreads];
            uv[j] = u_s[s * kTileVecs + t + j * kBulkThreads];
        }
        __syncthreads();                  /* every thread has read stage s */
        if (t == 0) {
            const size_t next = tile + (size_t)kStages * gridDim.x;
            if (next < ntiles) { issue(next, s); issued++; }
        }
#pragma unroll
        for (int j = 0; j < kBulkVecsPerThread; j++) {
            const size_t v = v0 + t + (size_t)j * kBulkThreads;
            if (v < nvec) st_stream(out + v, silu_mul_vec(gv[j], uv[j]));
        }
    }
    if (failed) {
        atomicExch(&g_bulk_error, 1u);
        /* bounded drain: the copies already requested still target this CTA's
         * shared memory; give each outstanding stage one more bounded wait */
        __syncthreads();
        if (t == 0) {
            for (int j = k; j < issued; j++) mbar_wait(&full[j % kStages], (unsigned)(j / kStages) & 1u);
        }
        __syncthreads();
    }
}

}  // namespace vvb

using namespace vvb;

template <int VPT, int STAGES>
static int launch_bulk(const void* gate, const void* up, void* out, size_t nvec, void* stream) {
    static int resident = 0;
    constexpr int kTileVecs = kBulkThreads * VPT;
    const size_t smem = (size_t)2 * STAGES * kTileVecs * sizeof(vec16);
    if (resident == 0) {
        if (cudaFuncSetAttribute(swiglu_bulk_kernel<VPT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        int per_sm = 0, dev = 0, sms = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, swiglu_bulk_kernel<VPT, STAGES>, kBulkThreads, smem);
        resident = (per_sm > 0 ? per_sm : 1) * (sms > 0 ? sms : 148);
    }
    const size_t ntiles = (nvec + kTileVecs - 1) / kTileVecs;
    const unsigned grid = (unsigned)(ntiles < (size_t)resident ? ntiles : (size_t)resident);
    launch_pdl(swiglu_bulk_kernel<VPT, STAGES>, dim3(grid), dim3(kBulkThreads), smem, (cudaStream_t)stream,
               (const vec16*)gate, (const vec16*)up, (vec16*)out, nvec);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

/* variant = 10 * vectors per thread + stages */
extern "C" int vvbk_swiglu_bulk(const void* gate, const void* up, void* out, size_t nvec, void* stream, int variant) {
    switch (variant) {
        case 42: return launch_bulk<4, 2>(gate, up, out, nvec, stream);
        case 24: return launch_bulk<2, 4>(gate, up, out, nvec, stream);
        case 26: return launch_bulk<2, 6>(gate, up, out, nvec, stream);
        case 18: return launch_bulk<1, 8>(gate, up, out, nvec, stream);
        case 84: return launch_bulk<8, 3>(gate, up, out, nvec, stream);
        default: return launch_bulk<4, 3>(gate, up, out, nvec, stream);
    }
}

/* Test hook: 1 when any wait of the bulk kernel has ever given up. Synchronises. */
extern "C" int vvbk_swiglu_bulk_error(void) {
    unsigned v = 0;
    if (cudaMemcpyFromSymbol(&v, g_bulk_error, sizeof v) != cudaSuccess) return -1;
    return (int)v;
}
#endif  /* VVB_TUNING */
