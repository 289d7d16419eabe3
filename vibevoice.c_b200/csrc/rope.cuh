/*
 * rope.cuh -- arguments and the per-CTA device body of the RoPE tile kernel,
 * shared by rope.cu and the single-launch layer chain (chain.cu). The design
 * and the arithmetic are documented at the top of rope.cu.
 */
#pragma once
#include "vvb_device.cuh"
#include "vvb_launch.h"

namespace vvb {

constexpr int kRopeThreads = 256;
constexpr int kRopeMaxRowsPerThread = 4;
constexpr int kRopeTableEntries = 1024;   /* rows_per_cta * half <= this */
constexpr unsigned kRopeOneWave = 3u * 148u;   /* CTAs resident at once on a 148-SM part */

struct RopeArgs {
    vec16* q;
    vec16* k;
    const int* d_position;
    int rows, n_q, n_kv;
    int half;              /* head_dim / 2 */
    int hvn;               /* half / 8: vectors per half head */
    int items_per_row;     /* (n_q + n_kv) * hvn */
    int cols_per_cta;      /* min(items_per_row, 256) */
    int row_slots;         /* 256 / cols_per_cta: rows a CTA touches per pass */
    int passes;            /* rows per thread, 1..4 */
    int position_offset;
    float inv_freq[VVB_ROPE_MAX_HALF];
};

/* sin and cos of a float angle, evaluated in double and rounded to float.
 * k = nearest integer to x*2/pi (|k| < 2^31 for every |x| <= 2^31);
 * r = x - k*pi/2 with pi/2 = P1 + P2 + P3, each product exact inside the FMA. */
__device__ __forceinline__ void sincos_f64(float angle, float* s_out, float* c_out) {
    const double x = (double)angle;
    const double kShift = 6755399441055744.0;                 /* 1.5 * 2^52 */
    const double t = fma(x, 0.63661977236758134308, kShift);  /* 2/pi */
    const int q = __double2loint(t);
    const double k = t - kShift;
    double r = fma(-k, 1.57079632679489655800e+00, x);
    r = fma(-k, 6.12323399573676603587e-17, r);
    r = fma(-k, -1.49738490485916983294e-33, r);
    const double r2 = r * r;
    /* sin r = r + r^3 * (-1/3! + r^2/5! - ... + r^12/15!) */
    double ps = 1.0 / 1307674368000.0;
    ps = fma(ps, r2, -1.0 / 6227020800.0);
    ps = fma(ps, r2, 1.0 / 39916800.0);
    ps = fma(ps, r2, -1.0 / 362880.0);
    ps = fma(ps, r2, 1.0 / 5040.0);
    ps = fma(ps, r2, -1.0 / 120.0);
    ps = fma(ps, r2, 1.0 / 6.0);
    const double sn = fma(-ps * r2, r, r);
    /* cos r = 1 - r^2/2! + r^4/4! - ... + r^16/16! */
    double pc = 1.0 / 20922789888000.0;
    pc = fma(pc, r2, -1.0 / 87178291200.0);
    pc = fma(pc, r2, 1.0 / 479001600.0);
    pc = fma(pc, r2, -1.0 / 3628800.0);
    pc = fma(pc, r2, 1.0 / 40320.0);
    pc = fma(pc, r2, -1.0 / 720.0);
    pc = fma(pc, r2, 1.0 / 24.0);
    pc = fma(pc, r2, -0.5);
    const double cs = fma(pc, r2, 1.0);
    const float sf = (float)sn, cf = (float)cs;
    const float s1 = (q & 1) ? cf : sf;      /* quadrant: 0:(s,c) 1:(c,-s) 2:(-s,-c) 3:(-c,s) */
    const float c1 = (q & 1) ? sf : cf;
    *s_out = (q & 2) ? -s1 : s1;
    *c_out = ((q + 1) & 2) ? -c1 : c1;
}

/* One CTA's tile: block (bx, by) of the (row tiles, column chunks) grid. */
__device__ __forceinline__ void rope_tile_body(const RopeArgs& a, int bx, int by) {
    __shared__ __align__(16) float cos_s[kRopeTableEntries];
    __shared__ __align__(16) float sin_s[kRopeTableEntries];

    const int t = threadIdx.x;
    const int rows_per_cta = a.row_slots * a.passes;
    const int row0 = bx * rows_per_cta;
    const int nrows = min(rows_per_cta, a.rows - row0);

    /* This thread's column, fixed for all its rows. */
    const int slot = t / a.cols_per_cta;
    const int cl = t - slot * a.cols_per_cta;
    const int c = by * kRopeThreads + cl;
    const bool col_ok = (slot < a.row_slots) && (c < a.items_per_row);
    const int head = c / a.hvn;
    const int vec = c - head * a.hvn;
    const size_t vph = (size_t)(2 * a.hvn);               /* vectors per head */
    vec16* base;
    size_t row_stride;                                     /* vectors between consecutive rows */
    if (head < a.n_q) {
        row_stride = (size_t)a.n_q * vph;
        base = a.q + (size_t)head * vph + vec;
    } else {
        row_stride = (size_t)a.n_kv * vph;
        base = a.k + (size_t)(head - a.n_q) * vph + vec;
    }

    /* Phase A: put this thread's loads in flight. */
    vec16 lo[kRopeMaxRowsPerThread], hi[kRopeMaxRowsPerThread];
    vec16* ptr[kRopeMaxRowsPerThread];
#pragma unroll
    for (int m = 0; m < kRopeMaxRowsPerThread; m++) {
        const int rl = slot + m * a.row_slots;
        ptr[m] = nullptr;
        if (col_ok && m < a.passes && rl < nrows) {
            vec16* p = base + (size_t)(row0 + rl) * row_stride;
            ptr[m] = p;
            lo[m] = ld_stream(p);
            hi[m] = ld_stream(p + a.hvn);
        }
    }

    /* Phase B: the CTA's cos/sin, once per (row, frequency). */
    const int pos0 = (a.d_position != nullptr ? *a.d_position : a.position_offset) + row0;
    for (int e = t; e < nrows * a.half; e += kRopeThreads) {
        const int rl = e / a.half;
        const int i = e - rl * a.half;
        const float ang = __fmul_rn((float)(pos0 + rl), a.inv_freq[i]);
        sincos_f64(ang, &sin_s[e], &cos_s[e]);
    }
    __syncthreads();

    /* Phase C: rotate and store. */
#pragma unroll
    for (int m = 0; m < kRopeMaxRowsPerThread; m++) {
        if (ptr[m] == nullptr) continue;
        const int tab = (slot + m * a.row_slots) * a.half + vec * 8;
        float x0[8], x1[8], c8[8], s8[8];
        unpack8(lo[m], x0);
        unpack8(hi[m], x1);
        *reinterpret_cast<float4*>(&c8[0]) = *reinterpret_cast<const float4*>(&cos_s[tab]);
        *reinterpret_cast<float4*>(&c8[4]) = *reinterpret_cast<const float4*>(&cos_s[tab + 4]);
        *reinterpret_cast<float4*>(&s8[0]) = *reinterpret_cast<const float4*>(&sin_s[tab]);
        *reinterpret_cast<float4*>(&s8[4]) = *reinterpret_cast<const float4*>(&sin_s[tab + 4]);
        float y0[8], y1[8];
#pragma unroll
        for (int e = 0; e < 8; e++) {
            y0[e] = __fsub_rn(__fmul_rn(x0[e], c8[e]), __fmul_rn(x1[e], s8[e]));
            y1[e] = __fadd_rn(__fmul_rn(x0[e], s8[e]), __fmul_rn(x1[e], c8[e]));
        }
        st_stream(ptr[m], pack8(y0));
        st_stream(ptr[m] + a.hvn, pack8(y1));
    }
}

/* Host side: fill the tile plan for a [rows, n_q + n_kv heads, head_dim]
 * problem (head_dim a multiple of 16) and return the (x, y) grid. */
static inline void rope_plan(RopeArgs& a, void* q, void* k, int rows, int n_q_heads, int n_kv_heads,
                             int head_dim, int position_offset, const int* d_position,
                             const float* inv_freq, int max_passes, unsigned* gx, unsigned* gy) {
    const int half = head_dim / 2;
    a.q = (vec16*)q;
    a.k = (vec16*)k;
    a.d_position = d_position;
    a.rows = rows;
    a.n_q = n_q_heads;
    a.n_kv = n_kv_heads;
    a.half = half;
    a.hvn = half / 8;
    a.items_per_row = (n_q_heads + n_kv_heads) * a.hvn;
    a.position_offset = position_offset;
    for (int i = 0; i < half; i++) a.inv_freq[i] = inv_freq[i];
    a.cols_per_cta = a.items_per_row < kRopeThreads ? a.items_per_row : kRopeThreads;
    a.row_slots = kRopeThreads / a.cols_per_cta;
    /* rows per CTA = row_slots * passes, bounded by the cos/sin table */
    int passes = kRopeTableEntries / (half * a.row_slots);
    if (passes > max_passes) passes = max_passes;
    if (passes < 1) {                       /* narrow rows of a wide head: fewer row slots */
        a.row_slots = kRopeTableEntries / half;
        passes = 1;
    }
    /* Deep grids take the most rows per thread (36.4 us at 14449 rows with 4
     * against 37.7 with 3, 40.8 with 2 and 55.6 with 1; 11.9 / 12.1 / 13.1 us at
     * 4096 rows, where the grid is 2.3 waves: fewer rows per thread to even out
     * the waves costs more than the uneven last wave does). A grid that fits the SMs in one wave
     * is a latency problem instead: it takes the fewest rows per thread that
     * still fit one wave (1.86 against 2.48 us at 64 rows, 4.43 against 5.08 at
     * 1024). kRopeOneWave = 3 CTAs on each of 148 SMs. */
    const unsigned gy_ = (unsigned)((a.items_per_row + kRopeThreads - 1) / kRopeThreads);
    for (int p = 1; p < passes; p++) {
        const unsigned ctas = (unsigned)((rows + a.row_slots * p - 1) / (a.row_slots * p)) * gy_;
        if (ctas <= kRopeOneWave) { passes = p; break; }
    }
    a.passes = passes;
    const int rows_per_cta = a.row_slots * a.passes;
    *gx = (unsigned)((rows + rows_per_cta - 1) / rows_per_cta);
    *gy = gy_;
}

}  // namespace vvb
