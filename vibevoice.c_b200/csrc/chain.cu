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

constexpr int kChainThreads = 256;
constexpr int kChainNormGroup = 128;     /* threads per row */
constexpr int kChainNormVPT = 4;         /* => hidden <= 128 * 4 * 8 = 4096 */
/* Vectors of gate (and of up) per thread of a SwiGLU CTA. Inside this kernel
 * (three 256-thread CTAs per SM) four is the measured best: 324 us per step at
 * 14449 rows and 45.1 us at 1807 against 360 / 49.1 with two and 448 / 59.4 with
 * one, which leave too few bytes in flight per SM. */
#ifndef VVB_CHAIN_SWIGLU_UNROLL
#define VVB_CHAIN_SWIGLU_UNROLL 4
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
    unsigned norm_ctas, rope_gx, rope_ctas;
};

template <int NORM_GUARD>
__global__ void __launch_bounds__(kChainThreads, VVB_CHAIN_CTAS)
layer_chain_kernel(const __grid_constant__ ChainArgs a) {
    pdl_wait();
    pdl_trigger();
    unsigned b = blockIdx.x;
    const int t = threadIdx.x;
    if (b < a.norm_ctas) {
        const int grp = t / kChainNormGroup;
        row_norm_body<kChainNormVPT, kChainThreads / kChainNormGroup, NORM_GUARD>(
            a.norm, (int)(b * (kChainThreads / kChainNormGroup)) + grp, t - grp * kChainNormGroup,
            kChainNormGroup, grp);
        return;
    }
    b -= a.norm_ctas;
    if (b < a.rope_ctas) {
        rope_tile_body(a.rope, (int)(b % a.rope_gx), (int)(b / a.rope_gx));
        return;
    }
    b -= a.rope_ctas;
    swiglu_stream_body<kChainSwigluUnroll, kChainThreads>(a.gate, a.up, a.out, a.swiglu_vecs, b, t);
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
              kRopeMaxRowsPerThread, &gx, &gy);
    a.gate = (const vec16*)gate;
    a.up = (const vec16*)up;
    a.out = (vec16*)gate;
    a.swiglu_vecs = n / 8;
    const unsigned rows_per_cta = kChainThreads / kChainNormGroup;
    a.norm_ctas = ((unsigned)rows + rows_per_cta - 1) / rows_per_cta;
    a.rope_gx = gx;
    a.rope_ctas = gx * gy;
    const size_t per_cta = (size_t)kChainThreads * kChainSwigluUnroll;
    const size_t swiglu_ctas = (a.swiglu_vecs + per_cta - 1) / per_cta;
    const size_t total = (size_t)a.norm_ctas + a.rope_ctas + swiglu_ctas;
    if (total > 0x7fffffffu) return (int)cudaErrorNotSupported;
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
