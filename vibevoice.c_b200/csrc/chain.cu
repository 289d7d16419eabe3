/*
 * chain.cu -- one decoder layer's elementwise chain as ONE launch.
 *
 * The three operations of the chain (residual add + RMSNorm on the hidden
 * state, RoPE on Q and K, SwiGLU on gate/up) touch disjoint tensors, so nothing
 * orders them: a single grid carries the CTAs of all three, block index ranges
 * selecting the work ([norm | rope | swiglu]). Compared with three launches this
 * removes two launch ramps and two drains per step -- about 2 us each, which is
 * a tenth of a step when a 14449-token prompt is sharded over eight GPUs
 * (1807 rows, ~45 us per GPU) -- because CTAs of the next operation start on an
 * SM as soon as CTAs of the previous one retire. Every CTA runs exactly the
 * device body the separate kernels run (row_norm.cuh, rope.cuh, swiglu.cuh), so
 * results are byte-identical to the three-launch path.
 *
 * CTAs are 256 threads: two rows of the norm (two 128-thread groups with a
 * named barrier each), one RoPE tile, or 4 x 256 SwiGLU vectors.
 */
#include "rope.cuh"
#include "row_norm.cuh"
#include "swiglu.cuh"
#include "vvb_launch.h"

#include <atomic>

namespace vvb {

extern std::atomic<uint64_t> g_launches;

#ifndef VVB_CHAIN_THREADS
#define VVB_CHAIN_THREADS 256
#endif
constexpr int kChainThreads = VVB_CHAIN_THREADS;
constexpr int kChainNormGroup = 128;     /* threads per row */
constexpr int kChainNormVPT = 4;         /* => hidden <= 128 * 4 * 8 = 4096 */
/* Build-time shape choices (the defaults are the measured best):
 * VVB_CHAIN_SWIGLU_UNROLL  vectors of gate (and of up) per thread of a SwiGLU CTA;
 * VVB_CHAIN_ORDER          block-index order of the three kinds of CTA:
 *                          0 [norm | rope | swiglu], 1 [swiglu | norm | rope],
 *                          2 [swiglu | rope | norm]. */
#ifndef VVB_CHAIN_SWIGLU_UNROLL
#define VVB_CHAIN_SWIGLU_UNROLL 4
#endif
#ifndef VVB_CHAIN_ORDER
#define VVB_CHAIN_ORDER 0
#endif
/* VVB_CHAIN_TAIL_UNROLL  0: off. Otherwise the last wave's worth of SwiGLU vectors goes out in
 *                        CTAs of this many vectors per thread (smaller than the bulk's), so that
 *                        the grid drains in shorter steps. Order 0 only. */
#ifndef VVB_CHAIN_TAIL_UNROLL
#define VVB_CHAIN_TAIL_UNROLL 0
#endif
constexpr int kChainSwigluUnroll = VVB_CHAIN_SWIGLU_UNROLL;

/* CTAs per SM the kernel is compiled for. At 4 the register cap is 64 and the
 * kernel spills a few words (328.6 us per step at 14449 rows); at 3 it takes 75
 * registers, spills nothing and runs 326.0 us (45.1 us at 1807 rows either way). */
#ifndef VVB_CHAIN_CTAS
#define VVB_CHAIN_CTAS 3
#endif

struct ChainArgs {
    RowNormArgs norm;
    RopeArgs rope;
    const vec16* gate;
    const vec16* up;
    vec16* out;
    size_t swiglu_vecs;
    unsigned norm_ctas, rope_gx, rope_ctas, swiglu_ctas, swiglu_bulk_ctas;
};

template <int NORM_GUARD>
__global__ void __launch_bounds__(kChainThreads, VVB_CHAIN_CTAS)
layer_chain_kernel(const __grid_constant__ ChainArgs a) {
    pdl_wait();
    pdl_trigger();
    unsigned b = blockIdx.x;
    const int t = threadIdx.x;
#if VVB_CHAIN_ORDER != 0
    if (b < a.swiglu_ctas) {
        swiglu_stream_body<kChainSwigluUnroll, kChainThreads>(a.gate, a.up, a.out, a.swiglu_vecs, b, t);
        return;
    }
    b -= a.swiglu_ctas;
#endif
#if VVB_CHAIN_ORDER == 2
    if (b < a.rope_ctas) {
        rope_tile_body<kChainThreads>(a.rope, (int)(b % a.rope_gx), (int)(b / a.rope_gx));
        return;
    }
    b -= a.rope_ctas;
#endif
    if (b < a.norm_ctas) {
        const int grp = t / kChainNormGroup;
        row_norm_body<kChainNormVPT, kChainThreads / kChainNormGroup, NORM_GUARD>(
            a.norm, (int)(b * (kChainThreads / kChainNormGroup)) + grp, t - grp * kChainNormGroup,
            kChainNormGroup, grp);
        return;
    }
#if VVB_CHAIN_ORDER != 2
    b -= a.norm_ctas;
    if (b < a.rope_ctas) {
        rope_tile_body<kChainThreads>(a.rope, (int)(b % a.rope_gx), (int)(b / a.rope_gx));
        return;
    }
#endif
#if VVB_CHAIN_ORDER == 0
    b -= a.rope_ctas;
#if VVB_CHAIN_TAIL_UNROLL > 0
    if (b >= a.swiglu_bulk_ctas) {
        const size_t done = (size_t)a.swiglu_bulk_ctas * (size_t)(kChainThreads * kChainSwigluUnroll);
        swiglu_stream_body<VVB_CHAIN_TAIL_UNROLL, kChainThreads>(a.gate + done, a.up + done, a.out + done,
                                                                 a.swiglu_vecs - done, b - a.swiglu_bulk_ctas, t);
        return;
    }
    swiglu_stream_body<kChainSwigluUnroll, kChainThreads>(
        a.gate, a.up, a.out, (size_t)a.swiglu_bulk_ctas * (size_t)(kChainThreads * kChainSwigluUnroll), b, t);
#else
    swiglu_stream_body<kChainSwigluUnroll, kChainThreads>(a.gate, a.up, a.out, a.swiglu_vecs, b, t);
#endif
#endif
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace vvb

using namespace vvb;

/* Returns cudaErrorNotSupported (without launching) when the shapes do not fit
 * the single-launch form; the caller then issues the three launches. */
extern "C" int vvbk_layer_chain(void* hidden, const void* delta, const void* weight, void* normed,
                                void* q, void* k, void* gate, const void* up,
                                int rows, int hidden_size, int n_q_heads, int n_kv_heads, int head_dim,
                                int inter, int position_offset, const float* inv_freq, float eps,
                                void* stream) {
    const int nvec = hidden_size / 8;
    const size_t n = (size_t)rows * (size_t)inter;
    const bool fits = rows > 0 && hidden_size > 0 && hidden_size % 8 == 0 &&
                      nvec <= kChainNormGroup * kChainNormVPT && delta != nullptr &&
                      head_dim >= 16 && head_dim % 16 == 0 && head_dim / 2 <= VVB_ROPE_MAX_HALF &&
                      n_q_heads + n_kv_heads > 0 && n > 0 && n % 8 == 0 &&
                      aligned16(hidden) && aligned16(delta) && aligned16(weight) && aligned16(normed) &&
                      aligned16(q) && aligned16(k) && aligned16(gate) && aligned16(up);
    if (!fits) return (int)cudaErrorNotSupported;

    ChainArgs a;
    a.norm = make_row_norm_args(hidden, delta, nullptr, hidden, weight, normed, rows, hidden_size, 0, eps);
    unsigned gx, gy;
    rope_plan(a.rope, q, k, rows, n_q_heads, n_kv_heads, head_dim, position_offset, nullptr, inv_freq,
              kRopeMaxRowsPerThread, &gx, &gy, kChainThreads);
    a.gate = (const vec16*)gate;
    a.up = (const vec16*)up;
    a.out = (vec16*)gate;
    a.swiglu_vecs = n / 8;
    const unsigned rows_per_cta = kChainThreads / kChainNormGroup;
    a.norm_ctas = ((unsigned)rows + rows_per_cta - 1) / rows_per_cta;
    a.rope_gx = gx;
    a.rope_ctas = gx * gy;
    const size_t per_cta = (size_t)kChainThreads * kChainSwigluUnroll;
#if VVB_CHAIN_TAIL_UNROLL > 0
    /* bulk CTAs for all but the last resident wave's worth of vectors, small CTAs for the rest */
    const size_t wave = (size_t)148 * VVB_CHAIN_CTAS;
    size_t bulk = a.swiglu_vecs / per_cta;
    bulk = bulk > wave ? bulk - wave : 0;
    const size_t per_tail = (size_t)kChainThreads * VVB_CHAIN_TAIL_UNROLL;
    const size_t swiglu_ctas = bulk + (a.swiglu_vecs - bulk * per_cta + per_tail - 1) / per_tail;
    a.swiglu_bulk_ctas = (unsigned)bulk;
#else
    const size_t swiglu_ctas = (a.swiglu_vecs + per_cta - 1) / per_cta;
    a.swiglu_bulk_ctas = 0;
#endif
    const size_t total = (size_t)a.norm_ctas + a.rope_ctas + swiglu_ctas;
    if (total > 0x7fffffffu) return (int)cudaErrorNotSupported;
    a.swiglu_ctas = (unsigned)swiglu_ctas;
    const int guard = row_guard_mode(nvec, kChainNormGroup, kChainNormVPT);
    if (guard == GUARD_NONE)
        launch_pdl(layer_chain_kernel<GUARD_NONE>, dim3((unsigned)total), dim3(kChainThreads), 0, (cudaStream_t)stream, a);
    else if (guard == GUARD_LAST)
        launch_pdl(layer_chain_kernel<GUARD_LAST>, dim3((unsigned)total), dim3(kChainThreads), 0, (cudaStream_t)stream, a);
    else
        launch_pdl(layer_chain_kernel<GUARD_ALL>, dim3((unsigned)total), dim3(kChainThreads), 0, (cudaStream_t)stream, a);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}
