/*
 * rope.cu -- rotary position embedding, in place, on Q and K in one launch.
 * sm_100a, HBM-bound.
 *
 * Layout: x[rows, n_heads, head_dim] FP16; pairs (i, i + head_dim/2)
 * (rotate_half). The work of one row is (n_q + n_kv) heads x head_dim/16
 * "items"; an item is one 16-byte vector from the low half of a head and its
 * partner vector from the high half (8 pairs). A CTA of 256 threads takes a
 * tile of up to 1024 items -- four rows of the 7B shape (32 heads x 8 items) --
 * so every thread first puts eight 16-byte loads in flight, then the CTA
 * computes the tile's cos/sin table ONCE per (row, frequency) into shared
 * memory while those loads travel, and every head of the row reuses it. (The
 * reference recomputes powf/cosf/sinf for each of the 32 heads:
 * src/cuda/rope.cu:54-57.)
 *
 * Arithmetic, chosen to land on the reference CPU kernel's bits
 * (src/cpu/cpu_kernels.c:1466-1474):
 *   freq_i   powf(theta, -2i/head_dim) evaluated by the HOST libm and passed
 *            by value in the kernel parameters -- one float ulp of error in
 *            freq_i is several FP16 ulps in the result at positions ~1e4, and
 *            a device powf is not bit-identical to glibc's;
 *   ang      (float)pos * freq_i, one float multiply, as on the CPU;
 *   cos/sin  evaluated in DOUBLE on the float angle and rounded to float: the
 *            correctly rounded value, which is what glibc's cosf/sinf return
 *            in all but rare cases (64 evaluations per row, negligible);
 *   rotate   a*c - b*s and a*s + b*c with four separately rounded products
 *            (no FMA contraction, as in the reference's default CPU build).
 * No global or file-scope state: the launch is re-entrant and capturable, and
 * a replayed graph follows *d_position.
 */
#include "vvb_device.cuh"
#include "vvb_launch.h"

#include <atomic>

namespace vvb {

extern std::atomic<uint64_t> g_launches;

constexpr int kRopeThreads = 256;
constexpr int kRopeItemsPerThread = 4;
constexpr int kRopeTileItems = kRopeThreads * kRopeItemsPerThread; /* 1024 */
constexpr int kRopeTableEntries = 1024;                            /* rows_per_tile * half <= this */

struct RopeArgs {
    vec16* q;
    vec16* k;
    const int* d_position;
    int rows, n_q, n_kv;
    int half;            /* head_dim / 2 */
    int hvn;             /* half / 8: vectors per half head */
    int items_per_row;   /* (n_q + n_kv) * hvn */
    int rows_per_tile;   /* R */
    int chunk_items;     /* items of one row a CTA covers (== items_per_row unless the row is split) */
    int position_offset;
    float inv_freq[VVB_ROPE_MAX_HALF];
};

__device__ __forceinline__ vec16* item_ptr(const RopeArgs& a, int row, int c) {
    const int head = c / a.hvn;
    const int vec = c - head * a.hvn;
    const size_t vecs_per_head = (size_t)(2 * a.hvn);
    if (head < a.n_q)
        return a.q + ((size_t)row * (size_t)a.n_q + (size_t)head) * vecs_per_head + vec;
    return a.k + ((size_t)row * (size_t)a.n_kv + (size_t)(head - a.n_q)) * vecs_per_head + vec;
}

__global__ void __launch_bounds__(kRopeThreads)
rope_tile_kernel(const __grid_constant__ RopeArgs a) {
    __shared__ __align__(16) float cos_s[kRopeTableEntries];
    __shared__ __align__(16) float sin_s[kRopeTableEntries];

    const int t = threadIdx.x;
    const int row0 = blockIdx.x * a.rows_per_tile;
    const int c0 = blockIdx.y * a.chunk_items;
    const int nrows = min(a.rows_per_tile, a.rows - row0);
    const int ncols = min(a.chunk_items, a.items_per_row - c0);
    const int nitems = nrows * ncols;

    /* Phase A: put this thread's loads in flight. */
    vec16 lo[kRopeItemsPerThread], hi[kRopeItemsPerThread];
    vec16* ptr[kRopeItemsPerThread];
    int tab[kRopeItemsPerThread];   /* index of the item's first cos/sin entry */
#pragma unroll
    for (int m = 0; m < kRopeItemsPerThread; m++) {
        const int it = t + m * kRopeThreads;
        ptr[m] = nullptr;
        tab[m] = 0;
        if (it < nitems) {
            const int rl = it / ncols;
            const int c = c0 + (it - rl * ncols);
            vec16* p = item_ptr(a, row0 + rl, c);
            ptr[m] = p;
            tab[m] = rl * a.half + (c % a.hvn) * 8;
            lo[m] = ld_stream(p);
            hi[m] = ld_stream(p + a.hvn);
        }
    }

    /* Phase B: the tile's cos/sin, once per (row, frequency). */
    const int pos0 = (a.d_position != nullptr ? *a.d_position : a.position_offset) + row0;
    for (int e = t; e < nrows * a.half; e += kRopeThreads) {
        const int rl = e / a.half;
        const int i = e - rl * a.half;
        const float ang = __fmul_rn((float)(pos0 + rl), a.inv_freq[i]);
        double s, c;
        sincos((double)ang, &s, &c);
        cos_s[e] = (float)c;
        sin_s[e] = (float)s;
    }
    __syncthreads();

    /* Phase C: rotate and store. */
#pragma unroll
    for (int m = 0; m < kRopeItemsPerThread; m++) {
        if (ptr[m] == nullptr) continue;
        float x0[8], x1[8], c[8], s[8];
        unpack8(lo[m], x0);
        unpack8(hi[m], x1);
        *reinterpret_cast<float4*>(&c[0]) = *reinterpret_cast<const float4*>(&cos_s[tab[m]]);
        *reinterpret_cast<float4*>(&c[4]) = *reinterpret_cast<const float4*>(&cos_s[tab[m] + 4]);
        *reinterpret_cast<float4*>(&s[0]) = *reinterpret_cast<const float4*>(&sin_s[tab[m]]);
        *reinterpret_cast<float4*>(&s[4]) = *reinterpret_cast<const float4*>(&sin_s[tab[m] + 4]);
        float y0[8], y1[8];
#pragma unroll
        for (int e = 0; e < 8; e++) {
            y0[e] = __fsub_rn(__fmul_rn(x0[e], c[e]), __fmul_rn(x1[e], s[e]));
            y1[e] = __fadd_rn(__fmul_rn(x0[e], s[e]), __fmul_rn(x1[e], c[e]));
        }
        st_stream(ptr[m], pack8(y0));
        st_stream(ptr[m] + a.hvn, pack8(y1));
    }
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
        double sd, cd;
        sincos((double)ang, &sd, &cd);
        const float c = (float)cd, s = (float)sd;
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
        a.q = (vec16*)q;
        a.k = (vec16*)k;
        a.d_position = d_position;
        a.rows = rows;
        a.n_q = n_q_heads;
        a.n_kv = n_kv_heads;
        a.half = half;
        a.hvn = half / 8;
        a.items_per_row = heads * a.hvn;
        a.position_offset = position_offset;
        for (int i = 0; i < half; i++) a.inv_freq[i] = inv_freq[i];
        unsigned grid_y = 1;
        if (a.items_per_row <= kRopeTileItems) {
            int r = kRopeTileItems / a.items_per_row;
            const int table_rows = kRopeTableEntries / half;
            if (r > table_rows) r = table_rows;
            if (r > rows) r = rows;
            a.rows_per_tile = r;
            a.chunk_items = a.items_per_row;
        } else {
            a.rows_per_tile = 1;
            a.chunk_items = kRopeTileItems;
            grid_y = (unsigned)((a.items_per_row + kRopeTileItems - 1) / kRopeTileItems);
        }
        dim3 grid((unsigned)((rows + a.rows_per_tile - 1) / a.rows_per_tile), grid_y);
        rope_tile_kernel<<<grid, kRopeThreads, 0, s>>>(a);
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
    rope_scalar_kernel<<<(unsigned)blocks, 256, 0, s>>>(a);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}
