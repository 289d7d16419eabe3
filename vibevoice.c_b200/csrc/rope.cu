/*
 * rope.cu -- rotary position embedding, in place, on Q and K in one launch.
 * sm_100a, HBM-bound.
 *
 * Layout: x[rows, n_heads, head_dim] FP16; pairs (i, i + head_dim/2)
 * (rotate_half). The work of one row is (n_q + n_kv) heads x head_dim/16
 * "items"; an item is one 16-byte vector from the low half of a head and its
 * partner vector from the high half (8 pairs). A thread owns ONE item column
 * (head, vector) and walks up to four rows of it, so all index arithmetic is
 * done once per thread and the row loop only adds a stride. A CTA of 256
 * threads covers 256 columns -- the whole 7B row (32 heads x 8 vectors) -- of
 * up to four rows: every thread first puts eight 16-byte loads in flight, then
 * the CTA computes its cos/sin table ONCE per (row, frequency) into shared
 * memory while the loads travel, and all 32 heads reuse it. (The reference
 * recomputes powf/cosf/sinf for each head: src/cuda/rope.cu:54-57.)
 *
 * Arithmetic, chosen to land on the reference CPU kernel's bits
 * (src/cpu/cpu_kernels.c:1466-1474):
 *   freq_i   powf(theta, -2i/head_dim) evaluated by the HOST libm and passed
 *            by value in the kernel parameters -- one float ulp of error in
 *            freq_i is several FP16 ulps in the result at positions ~1e4, and
 *            a device powf is not bit-identical to glibc's;
 *   ang      (float)pos * freq_i, one float multiply, as on the CPU;
 *   cos/sin  evaluated in DOUBLE on the float angle (three-term Cody-Waite
 *            reduction by pi/2 with fused multiply-adds, then Taylor
 *            polynomials on [-pi/4, pi/4], absolute error < 1e-14) and rounded
 *            to float: the correctly rounded value, which is what glibc's
 *            cosf/sinf return in all but rare cases;
 *   rotate   a*c - b*s and a*s + b*c with four separately rounded products
 *            (no FMA contraction, as in the reference's default CPU build).
 * No global or file-scope state: the launch is re-entrant and capturable, and
 * a replayed graph follows *d_position.
 */
#include "rope.cuh"

#include <atomic>

/* CTAs per SM the tile kernel is compiled for: 3 (75 registers, no spills)
 * measures 36.5 us at 14449 rows and 11.9 at 4096 against 36.9 and 12.1 at 4
 * (register cap 64, a few spilled words). */
#ifndef VVB_ROPE_CTAS
#define VVB_ROPE_CTAS 3
#endif

namespace vvb {

extern std::atomic<uint64_t> g_launches;

__global__ void __launch_bounds__(kRopeThreads, VVB_ROPE_CTAS)
rope_tile_kernel(const __grid_constant__ RopeArgs a) {
    pdl_wait();
    pdl_trigger();
    rope_tile_body(a, blockIdx.x, blockIdx.y);
}

/* Any head_dim / alignment: one thread per pair, its own cos/sin. */
struct RopeScalarArgs {
    __half* q;
    __half* k;
    const int* d_position;
    int rows, n_q, n_kv, head_dim, half, position_offset;
    float inv_freq[VVB_ROPE_MAX_HALF];
};

__global__ void __launch_bounds__(256)
rope_scalar_kernel(const __grid_constant__ RopeScalarArgs a) {
    pdl_wait();
    pdl_trigger();
    const size_t pairs_per_row = (size_t)(a.n_q + a.n_kv) * (size_t)a.half;
    const size_t total = (size_t)a.rows * pairs_per_row;
    const int pos_base = (a.d_position != nullptr ? *a.d_position : a.position_offset);
    for (size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * 256) {
        const int row = (int)(idx / pairs_per_row);
        const int rem = (int)(idx - (size_t)row * pairs_per_row);
        const int head = rem / a.half;
        const int i = rem - head * a.half;
        __half* v = (head < a.n_q)
            ? a.q + ((size_t)row * (size_t)a.n_q + (size_t)head) * (size_t)a.head_dim
            : a.k + ((size_t)row * (size_t)a.n_kv + (size_t)(head - a.n_q)) * (size_t)a.head_dim;
        const float ang = __fmul_rn((float)(pos_base + row), a.inv_freq[i]);
        float s, c;
        sincos_f64(ang, &s, &c);
        const float x0 = __half2float(v[i]), x1 = __half2float(v[i + a.half]);
        v[i] = __float2half_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)));
        v[i + a.half] = __float2half_rn(__fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)));
    }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace vvb

using namespace vvb;

extern "C" int vvbk_rope(void* q, void* k, int rows, int n_q_heads, int n_kv_heads, int head_dim,
                         int position_offset, const int* d_position, const float* inv_freq,
                         void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    const int half = head_dim / 2;
    const int heads = n_q_heads + n_kv_heads;
    if (rows <= 0 || heads <= 0 || half <= 0) return (int)cudaSuccess;

    if (head_dim % 16 == 0 && aligned16(q) && aligned16(k)) {
        RopeArgs a;
        const int max_passes = kRopeMaxRowsPerThread;
        unsigned gx, gy;
        rope_plan(a, q, k, rows, n_q_heads, n_kv_heads, head_dim, position_offset, d_position, inv_freq,
                  max_passes, &gx, &gy);
        if (gy > 65535u) return (int)cudaErrorInvalidValue;
        launch_pdl(rope_tile_kernel, dim3(gx, gy), dim3(kRopeThreads), 0, s, a);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return (int)cudaGetLastError();
    }

    RopeScalarArgs a;
    a.q = (__half*)q;
    a.k = (__half*)k;
    a.d_position = d_position;
    a.rows = rows;
    a.n_q = n_q_heads;
    a.n_kv = n_kv_heads;
    a.head_dim = head_dim;
    a.half = half;
    a.position_offset = position_offset;
    for (int i = 0; i < half; i++) a.inv_freq[i] = inv_freq[i];
    const size_t total = (size_t)rows * (size_t)heads * (size_t)half;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148u * 32u) blocks = 148u * 32u;
    launch_pdl(rope_scalar_kernel, dim3((unsigned)blocks), dim3(256), 0, s, a);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}
