/*
 * row_norm.cuh -- arguments and the per-row device body of the RMSNorm family
 * (RMSNorm, residual add + RMSNorm, gather + RMSNorm), shared by the row
 * kernel (row_norm.cu) and the single-launch layer chain (chain.cu).
 * The arithmetic is documented at the top of row_norm.cu.
 */
#pragma once
#include "vvb_device.cuh"

namespace vvb {

struct RowNormArgs {
    const vec16* src;     /* rows or table */
    const vec16* delta;   /* may be null */
    const int32_t* ids;   /* may be null */
    vec16* row_out;       /* may be null */
    const vec16* weight;
    vec16* normed;        /* never null in the norm kernel */
    int rows;
    int nvec;             /* hidden / 8 */
    int hidden;
    int vocab;
    float eps;
    double inv_hidden;    /* 1.0 / hidden, rounded by the host's division */
};

static inline RowNormArgs make_row_norm_args(const void* src, const void* delta, const int32_t* ids, void* row_out,
                                             const void* weight, void* normed, int rows, int hidden, int vocab,
                                             float eps) {
    return RowNormArgs{(const vec16*)src, (const vec16*)delta, ids, (vec16*)row_out, (const vec16*)weight,
                       (vec16*)normed, rows, hidden / 8, hidden, vocab, eps, 1.0 / (double)hidden};
}

/* Launch shape of the one-CTA-per-row kernels (row norm, int8 quantizers):
 * threads per row and 16-byte vectors per thread (1, 2 or 4). Deep grids take
 * four vectors per thread; grids of at most kLatencyRows rows (about one wave
 * on a 148-SM part) are bound by one row's latency and take one vector per
 * thread when the row fits a CTA that way. */
constexpr int kLatencyRows = 592;
static inline void row_launch_shape(int rows, int nvec, int* threads, int* vpt) {
    const int per_thread = (rows <= kLatencyRows && nvec <= 1024) ? 1 : 4;
    int t = (((nvec + per_thread - 1) / per_thread) + 31) / 32 * 32;
    if (t > 1024) t = 1024;
    int v = (nvec + t - 1) / t;
    if (v == 3) v = 4;
    *threads = t;
    *vpt = v;
}
/* How much of the "is this vector inside the row" test a kernel instance
 * carries: every vector, only a thread's last one (true whenever
 * (VPT - 1) * threads < nvec: all earlier vectors are inside for every thread),
 * or none (VPT * threads == nvec). The test costs a compare, a branch and the
 * zeroing of four registers per vector, which the issue-bound kernels feel. */
enum { GUARD_ALL = 0, GUARD_LAST = 1, GUARD_NONE = 2 };
static inline int row_guard_mode(int nvec, int threads, int vpt) {
    if ((long long)vpt * threads == nvec) return GUARD_NONE;
    if ((long long)(vpt - 1) * threads < nvec) return GUARD_LAST;
    return GUARD_ALL;
}
template <int VPT, int GUARD>
__device__ __forceinline__ bool vec_inside(int j, int v, int nvec) {
    if (GUARD == GUARD_NONE) return true;
    if (GUARD == GUARD_LAST && j < VPT - 1) return true;
    return v < nvec;
}

/* A gathered row's address depends on a load (its id), so a gather CTA begins
 * with two DRAM round trips in sequence. The CTA of row r therefore also pulls
 * the table row of row r + kGatherAhead into L2 -- that id load is off its own
 * critical path -- and by the time the later CTA runs, its row is an L2 hit.
 * kGatherAhead is about twice the CTAs resident at once (8 per SM): 2048 rows
 * of 7 KB are 15 MB of the 126 MB L2. Only addresses inside the row are named. */
constexpr int kGatherAhead = 2048;
/* Step 1, next to the CTA's own id load: the far row's id, or -1. */
__device__ __forceinline__ int gather_far_id(const int32_t* ids, int row, int rows, int vocab) {
    const int far = row + kGatherAhead;
    if (far >= rows) return -1;
    int id = __ldg(ids + far);
    if (vocab > 0) id = min(max(id, 0), vocab - 1);
    return id;
}
/* Step 2, after the CTA's own row loads have been issued (a warp issues in
 * order: waiting for the far id any earlier would hold those loads back). */
__device__ __forceinline__ void gather_prefetch(const vec16* table, int far_id, int nvec, int t, int nthreads) {
    if (far_id < 0) return;
    const char* p = reinterpret_cast<const char*>(table + (size_t)far_id * (size_t)nvec);
    const int bytes = nvec * (int)sizeof(vec16);
    for (int off = t * 128; off < bytes; off += nthreads * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p + off));
}

__device__ __forceinline__ float inv_rms(double ss, int hidden, float eps) {
    const float mean = (float)(ss / (double)hidden);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
}

/* ss / n, correctly rounded, without the division sequence (some thirty
 * dependent instructions that every row waits for): q = ss * fl(1/n) is within
 * two ulps of the quotient, and a step q += (ss - q*n) * fl(1/n), whose residual
 * is exact inside the fused multiply-add, lands on the correctly rounded
 * quotient from a start within one ulp (Markstein's theorem for division by
 * reciprocal); two steps cover the two-ulp start. An infinite or NaN sum (a row
 * holding one) takes the division itself, which the residual would turn to NaN. */
__device__ __forceinline__ double div_rn_by_count(double ss, int hidden, double inv_hidden) {
    const double n = (double)hidden;
    double q = ss * inv_hidden;
    q = fma(fma(-q, n, ss), inv_hidden, q);
    q = fma(fma(-q, n, ss), inv_hidden, q);
    if (!(fabs(ss) <= 1.7976931348623157e308)) q = ss / n;
    return q;
}
__device__ __forceinline__ float inv_rms(double ss, int hidden, double inv_hidden, float eps) {
    const float mean = (float)div_rn_by_count(ss, hidden, inv_hidden);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
}

/* (h * inv) * w for the eight elements of a vector. */
__device__ __forceinline__ vec16 scale_row_vec(const vec16& h, const vec16& w, float inv) {
    const float2 i2 = splat2(inv);
    vec16 r;
    r.x = pack2(mul2(mul2(unpack2(h.x), i2), unpack2(w.x)));
    r.y = pack2(mul2(mul2(unpack2(h.y), i2), unpack2(w.y)));
    r.z = pack2(mul2(mul2(unpack2(h.z), i2), unpack2(w.z)));
    r.w = pack2(mul2(mul2(unpack2(h.w), i2), unpack2(w.w)));
    return r;
}

/* ------------------------------------------------------------ one row, one group
 * GROUPS groups of `G` threads share a CTA, one row each (GROUPS == 1: the
 * group is the whole CTA). t = thread index within the group. */
/* Phase 1: loads the row (and addend, gamma), stores the updated row if asked,
 * reduces the sum of squares and leaves the NORMALISED row, rounded to FP16, in
 * yv[] (vector v = t + j*G in yv[j]; zeros beyond the row). LATEW: gamma is
 * fetched when it is used, after the reduction (it stays in L1), instead of
 * riding in registers next to the row: for instances with many vectors per
 * thread. (Keeping the row widened to float across the reduction, to save the
 * second widening, was measured: same registers after the compiler's own
 * choices, same time.) */
template <int VPT, int GROUPS, int GUARD, bool LATEW = false, int DELTA = 2>
__device__ __forceinline__ void row_norm_produce(const RowNormArgs& a, int row, int t, int G, int grp,
                                                 vec16 (&yv)[VPT]) {
    __shared__ double red[GROUPS][32];
    __shared__ float inv_s[GROUPS];
    /* one group per CTA: the grid is exactly the rows, so the group has one */
    const bool have = (GROUPS == 1) || (row < a.rows);
    const size_t roff = (size_t)(have ? row : 0) * (size_t)a.nvec;
    const int nvec = a.nvec;
    /* a group without a row loads and stores nothing */
#define VVB_ROW_IN(j) (have && vec_inside<VPT, GUARD>(j, t + (j) * G, nvec))

    size_t srow = (size_t)(have ? row : 0);
    int far_id = -1;
    if (have && a.ids != nullptr) {
        int id = a.ids[row];
        far_id = gather_far_id(a.ids, row, a.rows, a.vocab);
        if (a.vocab > 0) id = min(max(id, 0), a.vocab - 1);
        srow = (size_t)id;
    }
    const vec16* sp = a.src + srow * (size_t)a.nvec + t;
    /* DELTA: 0 no addend (its registers are not even reserved), 1 an addend, 2 decided by the argument */
    const bool has_delta = (DELTA == 2) ? (a.delta != nullptr) : (DELTA == 1);

    /* Every load of the row, the addend and gamma goes out before any is used. */
    vec16 hv[VPT], dv[VPT], wv[VPT];
#pragma unroll
    for (int j = 0; j < VPT; j++) hv[j] = VVB_ROW_IN(j) ? ld_stream(sp + j * G) : make_uint4(0, 0, 0, 0);
    if (has_delta) {
        const vec16* dp = a.delta + roff + t;
#pragma unroll
        for (int j = 0; j < VPT; j++) dv[j] = VVB_ROW_IN(j) ? ld_stream(dp + j * G) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int j = 0; j < VPT; j++)
        if (!LATEW) wv[j] = VVB_ROW_IN(j) ? __ldg(a.weight + t + j * G) : make_uint4(0, 0, 0, 0);
    gather_prefetch(a.src, far_id, a.nvec, t, G);
    /* (The same look-ahead on the streaming rows of the plain norm was measured
     * and does not pay: 62.5 against 62.2 us, the chain 328.2 against 326.1 --
     * their addresses are known at once, so the loads are already in flight.) */

    double ss = 0.0, ss1 = 0.0;
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        uint32_t* hw = reinterpret_cast<uint32_t*>(&hv[j]);
        const uint32_t* dw = reinterpret_cast<const uint32_t*>(&dv[j]);
#pragma unroll
        for (int e = 0; e < 4; e++) {
            if (has_delta) hw[e] = hadd2_bits(hw[e], dw[e]);
            /* half -> double in ONE conversion each (exact either way; the detour
             * through float cost an instruction per element: rmsnorm_q8 36.2 -> 35.1 us) */
            double dx, dy;
            asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.f64.f16 %0, lo;\n\tcvt.f64.f16 %1, hi;\n\t}"
                : "=d"(dx), "=d"(dy) : "r"(hw[e]));
            ss = fma(dx, dx, ss);
            ss1 = fma(dy, dy, ss1);
        }
    }
    if (a.row_out != nullptr) {
        vec16* rp = a.row_out + roff + t;
#pragma unroll
        for (int j = 0; j < VPT; j++)
            if (VVB_ROW_IN(j)) st_stream(rp + j * G, hv[j]);
    }
#undef VVB_ROW_IN
    ss += ss1;

    ss = warp_sum(ss);
    if ((t & 31) == 0) red[grp][t >> 5] = ss;
    if (GROUPS == 1) {
        __syncthreads();
    } else {
        asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "r"(G) : "memory");
    }
    /* The scalar tail (the mean, a square root and a float division: some forty
     * dependent instructions) is issued by ONE warp of the group, not by all of
     * them. */
    if (t < 32) {
        double s = (t < (G >> 5)) ? red[grp][t] : 0.0;
        s = warp_sum(s);
        if (t == 0) inv_s[grp] = inv_rms(s, a.hidden, a.inv_hidden, a.eps);
    }
    if (GROUPS == 1) {
        __syncthreads();
    } else {
        asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "r"(G) : "memory");
    }
    const float inv = inv_s[grp];
#pragma unroll
    for (int j = 0; j < VPT; j++) {
        if (LATEW) wv[j] = vec_inside<VPT, GUARD>(j, t + j * G, nvec) ? __ldg(a.weight + t + j * G) : make_uint4(0, 0, 0, 0);
        yv[j] = scale_row_vec(hv[j], wv[j], inv);
    }
}

/* One row: produce, then stream the normalised row out. */
template <int VPT, int GROUPS, int GUARD, bool LATEW = false, int DELTA = 2>
__device__ __forceinline__ void row_norm_body(const RowNormArgs& a, int row, int t, int G, int grp) {
    vec16 yv[VPT];
    row_norm_produce<VPT, GROUPS, GUARD, LATEW, DELTA>(a, row, t, G, grp, yv);
    if (GROUPS > 1 && row >= a.rows) return;
    vec16* np_ = a.normed + (size_t)row * (size_t)a.nvec + t;
#pragma unroll
    for (int j = 0; j < VPT; j++)
        if (vec_inside<VPT, GUARD>(j, t + j * G, a.nvec)) st_stream(np_ + j * G, yv[j]);
}

}  // namespace vvb
