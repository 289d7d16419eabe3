/*
 * rope_append.cu -- q/k/v bias add, RoPE on Q and K, and the KV-cache append,
 * in one launch. sm_100a, HBM-bound.
 *
 * The reference does this in up to six passes per layer
 * (src/inference/decoder.c:463-464 vv_bias_add_dev on q, k, v; :850-855
 * vv_rope_dev on Q then K; src/inference/kv_cache.c:229-246 two device copies
 * of K and V into the layer's cache). Here one grid carries RoPE tiles
 * (rope.cuh) over the Q and K columns and, as its first CTAs, flat copy CTAs
 * for V:
 *   Q head   x = f16(q + bias_q), rotate, store in place
 *   K head   x = f16(k + bias_k), rotate, store INTO THE CACHE row
 *            (cache_offset + r); also in place when the caller keeps K
 *   V head   x = f16(v + bias_v), store into the cache row (no rotation)
 * so K and V are read once and written once (RoPE applied while K is
 * written), and Q is read and written once. Per 7B token: 18 432 bytes against
 * 20 480 without biases and 38 912 with them.
 *
 * Arithmetic is that of the separate ops, step by step: the bias sum is
 * rounded to FP16 before the rotation sees it (src/cuda/conv_vae.cu:54-66),
 * the rotation is rope.cuh's, the append is a bit copy. The cache is the
 * reference's raw FP16 layout: one [max_len, n_kv_heads * head_dim] array per
 * layer for K and one for V (src/inference/kv_cache.c:229-232).
 *
 * FP8 caches (template FMT = KV_E4M3 / KV_E5M2): the same launch, but what is
 * stored is the reference's software FP8 byte of each value (fp8_kv.cuh), one
 * byte per element in the same [max_len, n_kv_heads * head_dim] order
 * (src/cuda/kv_quant.cu:60-83 with a null page table). K is rounded to FP16
 * after the rotation, as the separate vv_rope_dev would have stored it, has
 * the layer's reference key subtracted in float when the cache keeps one
 * (kv_quant.cu:68-73), and is encoded; V is encoded as it is. The cache write
 * shrinks from 4096 to 2048 bytes per 7B token.
 *
 * TurboQuant caches (template FMT = KV_TQ4 .. KV_TQ1_5, head_dim 128 only): what
 * is stored is the reference's rotated and quantized form of each head vector
 * (tq_kv.cuh; src/cuda/kv_quant.cu:85-120): bytes_per_vec bytes of codes in
 * [max_len, n_kv_heads * bytes_per_vec] plus one FP16 RMS per vector in
 * [max_len, n_kv_heads]. A head vector is a warp's work, so the rotated K tile of
 * a CTA goes through shared memory (as for FP8) and its warps take the tile's
 * (row, head) vectors in turn; the V CTAs walk their rows a head vector per
 * warp. Per 7B token the cache write shrinks from 4096 bytes to 528 (4-bit) ..
 * 208 (1.5-bit).
 *
 * Paged caches (template PAGED): logical position t = cache_offset + r lands in
 * row page_table[t / 64] * 64 + t % 64 of the pool (cache_row below), for every
 * format; the contiguous instantiations carry no trace of the mapping.
 */
#include "fp8_kv.cuh"
#include "rope.cuh"
#include "tq_kv.cuh"

#include <atomic>

namespace vvb {

extern std::atomic<uint64_t> g_launches;

constexpr int kVRowsPerCta = 32;

/* CTAs per SM the FP16 variant is compiled for (the FP8 variants take 3: at 4
 * they spill and run 61.7 instead of 48.0 us; the FP16 variant measures 43.8 us
 * at 3 without spills against 44.3 at 4 with 124 bytes of spill loads). */
#ifndef VVB_ROPE_APPEND_RAW_CTAS
#define VVB_ROPE_APPEND_RAW_CTAS 3
#endif

struct RopeAppendArgs {
    RopeArgs r;               /* tile plan over the n_q + n_kv rotated heads */
    const vec16* v;
    vec16* k_cache;
    vec16* v_cache;
    const vec16* q_bias;      /* each may be null */
    const vec16* k_bias;
    const vec16* v_bias;
    const vec16* k_ref;       /* FP8 / TurboQuant: [n_kv_heads * head_dim] FP16 subtracted from K; may be null */
    __half* k_meta;           /* TurboQuant: [max_len, n_kv_heads] FP16 RMS of each stored K vector */
    __half* v_meta;
    const int* page_table;    /* may be null: logical position t lives in cache row t */
    int cache_offset;         /* cache row of row 0 (when r.d_position is null) */
    int keep_k;               /* also write the rotated K back in place */
    int v_ctas;               /* the grid's first v_ctas CTAs carry V, the rest are RoPE tiles ... */
    int row_tiles;            /* ... numbered row tile first: tile = chunk * row_tiles + row_tile */
};

/* Cache row of logical position t. A paged cache (the server's slots share one
 * pool of 64-position pages, include/vibevoice/kv_quant.h:47-53) maps page
 * t / 64 through the context's table and keeps the offset inside the page
 * (src/cuda/kv_codec.cuh:29-36). */
constexpr int kKvPageShift = 6;
__device__ __forceinline__ size_t cache_row(const int* page_table, int t) {
    if (page_table == nullptr) return (size_t)t;
    return ((size_t)__ldg(page_table + (t >> kKvPageShift)) << kKvPageShift) + (size_t)(t & ((1 << kKvPageShift) - 1));
}

__device__ __forceinline__ vec16 add_bias_vec(const vec16& x, const vec16& b) {
    return hadd8(x, b);      /* == widen, add, round to FP16 (vvb_device.cuh) */
}

template <int FMT, bool PAGED>
__global__ void __launch_bounds__(kRopeThreads, FMT == KV_RAW ? VVB_ROPE_APPEND_RAW_CTAS : 3)
rope_append_kernel(const __grid_constant__ RopeAppendArgs A) {
    __shared__ __align__(16) float cos_s[kRopeTableEntries];
    __shared__ __align__(16) float sin_s[kRopeTableEntries];
    const RopeArgs& a = A.r;
    const int t = threadIdx.x;
    pdl_wait();
    pdl_trigger();
    __shared__ TqCells tq_cells[1];
    if constexpr (TqUsesCells<FMT>::value) tq_cells_fill<FMT>(tq_cells[0], t);

    /* The FIRST CTAs of the grid (blockIdx.x < v_ctas) carry V: no rotation, so no table
     * and no barrier -- a flat copy (+ bias, + FP8 encoding) of kVRowsPerCta
     * rows per CTA into the cache. These CTAs are the longest of the grid (each
     * walks 32 rows), so they are dispatched first and the short RoPE tiles
     * fill in behind them instead of waiting for a tail of V copies; four
     * loads per thread are in flight at a time. */
    if ((int)blockIdx.x < A.v_ctas) {
        const int cols_v = a.n_kv * 2 * a.hvn;                 /* vectors per V row */
        const int row0v = blockIdx.x * kVRowsPerCta;
        if (row0v >= a.rows) return;
        const int items = min(kVRowsPerCta, a.rows - row0v) * cols_v;
        const int cache_first_v = (a.d_position != nullptr) ? *a.d_position : A.cache_offset;
        if constexpr (kv_is_tq(FMT)) {
            /* eight lanes to a head vector (tq_store16): a warp takes four consecutive vectors a
             * step, each lane two 16-byte pieces of its vector, and has two steps' loads in flight */
            constexpr int BPV = tq_bytes_per_vec(FMT);
            constexpr int kU = 2;
            constexpr int kWarps = kRopeThreads / 32;
            const int warp = t >> 5, lane = t & 31, sub = lane & 7;
            const int nvecs = min(kVRowsPerCta, a.rows - row0v) * a.n_kv;
            if constexpr (TqUsesCells<FMT>::value) __syncthreads();       /* the cell table */
            uint32_t flip[8];
            tq_flips16(sub, flip);
            const vec16* vsrc = A.v + (size_t)row0v * a.n_kv * 16;       /* a vector is 16 pieces */
            /* (row, head) of this lane's vector idx = 4 warp + (lane >> 3) + 32 n, by stepping */
            const int step_r = (4 * kWarps) / a.n_kv, step_h = 4 * kWarps - step_r * a.n_kv;
            const int idx0 = 4 * warp + (lane >> 3);
            int rl = idx0 / a.n_kv, h = idx0 - rl * a.n_kv;
            for (int base = 4 * warp; base < nvecs; base += 4 * kWarps * kU) {      /* warp-uniform */
                vec16 x[kU][2];
#pragma unroll
                for (int j = 0; j < kU; j++) {
                    const int idx = base + j * 4 * kWarps + (lane >> 3);
                    if (idx < nvecs) {
                        x[j][0] = ld_stream(vsrc + (size_t)idx * 16 + 2 * sub);
                        x[j][1] = ld_stream(vsrc + (size_t)idx * 16 + 2 * sub + 1);
                    } else {
                        x[j][0] = x[j][1] = make_uint4(0, 0, 0, 0);
                    }
                }
#pragma unroll
                for (int j = 0; j < kU; j++) {
                    if (base + j * 4 * kWarps >= nvecs) break;                    /* warp-uniform */
                    const int idx = base + j * 4 * kWarps + (lane >> 3);
                    const bool live = idx < nvecs;
                    if (A.v_bias && live) {
                        x[j][0] = add_bias_vec(x[j][0], __ldg(A.v_bias + h * 16 + 2 * sub));
                        x[j][1] = add_bias_vec(x[j][1], __ldg(A.v_bias + h * 16 + 2 * sub + 1));
                    }
                    const uint32_t* w = reinterpret_cast<const uint32_t*>(&x[j][0]);
                    float v16[16];
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const float2 f = unpack2(w[i] ^ flip[i]);
                        v16[2 * i] = f.x;
                        v16[2 * i + 1] = f.y;
                    }
                    const size_t at = live ? cache_row(PAGED ? A.page_table : nullptr, cache_first_v + row0v + rl) * a.n_kv + h : 0;
                    tq_store16<FMT>(v16, lane, reinterpret_cast<uint8_t*>(A.v_cache) + at * BPV, A.v_meta + at, live, tq_cells);
                    h += step_h;
                    rl += step_r;
                    if (h >= a.n_kv) { h -= a.n_kv; rl++; }
                }
            }
            return;
        }
        constexpr int kVUnroll = 4;
        for (int base = t; base < items; base += kRopeThreads * kVUnroll) {
            vec16 x[kVUnroll];
#pragma unroll
            for (int j = 0; j < kVUnroll; j++) {
                const int it = base + j * kRopeThreads;
                if (it < items) x[j] = ld_stream(A.v + (size_t)row0v * cols_v + it);
            }
#pragma unroll
            for (int j = 0; j < kVUnroll; j++) {
                const int it = base + j * kRopeThreads;
                if (it >= items) continue;
                const int rl = it / cols_v;
                const int cv = it - rl * cols_v;
                if (A.v_bias) x[j] = add_bias_vec(x[j], __ldg(A.v_bias + cv));
                const size_t at = cache_row(PAGED ? A.page_table : nullptr, cache_first_v + row0v + rl) * cols_v + cv;
                if constexpr (FMT == KV_RAW) st_stream(A.v_cache + at, x[j]);
                else if constexpr (!kv_is_tq(FMT))
                    __stcs(reinterpret_cast<uint2*>(A.v_cache) + at, fp8_encode8<FMT>(x[j], nullptr));
            }
        }
        return;
    }
    const int tile = (int)blockIdx.x - A.v_ctas;
    const int by = (tile < A.row_tiles) ? 0 : tile / A.row_tiles;   /* column chunk of this RoPE tile */
    const int bx = tile - by * A.row_tiles;                    /* its block of rows */

    const int rows_per_cta = a.row_slots * a.passes;
    const int row0 = bx * rows_per_cta;
    const int nrows = min(rows_per_cta, a.rows - row0);

    /* This thread's column (tensor, head, vector), fixed for all its rows. */
    const int slot = t / a.cols_per_cta;
    const int cl = t - slot * a.cols_per_cta;
    const int c = by * kRopeThreads + cl;
    const bool col_ok = (slot < a.row_slots) && (c < a.items_per_row);
    const int head = c / a.hvn;
    const int vec = c - head * a.hvn;
    const size_t vph = (size_t)(2 * a.hvn);
    const int dev_pos = (a.d_position != nullptr) ? *a.d_position : 0;
    const int pos_first = (a.d_position != nullptr) ? dev_pos : a.position_offset;
    const int cache_first = (a.d_position != nullptr) ? dev_pos : A.cache_offset;

    /* FP8: the K columns of this CTA's column chunk are staged through shared
     * memory (phase D) when the tile fits: 4 rows x 4 heads of 128 are 256 vectors. */
    constexpr int kStageVecs = 512;
    __shared__ vec16 k_stage[FMT == KV_RAW ? 1 : kStageVecs];
    const int chunk0 = by * kRopeThreads;
    const int chunk1 = min(chunk0 + a.cols_per_cta, a.items_per_row);
    const int first_k_col = max(chunk0, a.n_q * a.hvn);
    const int kcols = max(0, chunk1 - first_k_col);
    const bool staged = (FMT != KV_RAW) && kcols > 0 && kcols * 2 * rows_per_cta <= kStageVecs;

    const vec16* src;
    vec16* dst;
    vec16* dst_keep = nullptr;
    const vec16* bias = nullptr;
    size_t stride;
    int dst_row_first = 0;
    bool to_cache = false;
    vec16 rlo = make_uint4(0, 0, 0, 0), rhi = make_uint4(0, 0, 0, 0);     /* reference key (FP8) */
    if (head < a.n_q) {
        const size_t off = (size_t)head * vph + vec;
        stride = (size_t)a.n_q * vph;
        src = a.q + off;
        dst = a.q + off;
        if (A.q_bias) bias = A.q_bias + off;
    } else {
        const size_t off = (size_t)(head - a.n_q) * vph + vec;
        stride = (size_t)a.n_kv * vph;
        src = a.k + off;
        dst = A.k_cache + off;
        dst_row_first = cache_first;
        to_cache = true;
        if (FMT != KV_RAW && !kv_is_tq(FMT) && A.k_ref != nullptr && col_ok && !staged) {
            rlo = __ldg(A.k_ref + off);
            rhi = __ldg(A.k_ref + off + a.hvn);
        }
        if (A.keep_k) dst_keep = a.k + off;
        if (A.k_bias) bias = A.k_bias + off;
    }

    /* Phase A: loads in flight. */
    vec16 lo[kRopeMaxRowsPerThread], hi[kRopeMaxRowsPerThread];
    bool live[kRopeMaxRowsPerThread];
    vec16 blo = make_uint4(0, 0, 0, 0), bhi = make_uint4(0, 0, 0, 0);
    if (col_ok && bias != nullptr) {
        blo = __ldg(bias);
        bhi = __ldg(bias + a.hvn);
    }
#pragma unroll
    for (int m = 0; m < kRopeMaxRowsPerThread; m++) {
        const int rl = slot + m * a.row_slots;
        live[m] = col_ok && m < a.passes && rl < nrows;
        if (live[m]) {
            const vec16* p = src + (size_t)(row0 + rl) * stride;
            lo[m] = ld_stream(p);
            hi[m] = ld_stream(p + a.hvn);
        }
    }

    /* Phase B: cos/sin of the CTA's rows. */
    const int pos0 = pos_first + row0;
    for (int e = t; e < nrows * a.half; e += kRopeThreads) {
        const int rl = e / a.half;
        const int i = e - rl * a.half;
        const float ang = __fmul_rn((float)(pos0 + rl), a.inv_freq[i]);
        sincos_f64(ang, &sin_s[e], &cos_s[e]);
    }
    __syncthreads();

    /* Phase C: bias, rotate, store to the destination row. */
#pragma unroll
    for (int m = 0; m < kRopeMaxRowsPerThread; m++) {
        if (!live[m]) continue;
        const int rl = slot + m * a.row_slots;
        vec16 xlo = lo[m], xhi = hi[m];
        if (bias != nullptr) {
            xlo = add_bias_vec(xlo, blo);
            xhi = add_bias_vec(xhi, bhi);
        }
        {
            const int tab = rl * a.half + vec * 8;
            float x0[8], x1[8], c8[8], s8[8], y0[8], y1[8];
            unpack8(xlo, x0);
            unpack8(xhi, x1);
            *reinterpret_cast<float4*>(&c8[0]) = *reinterpret_cast<const float4*>(&cos_s[tab]);
            *reinterpret_cast<float4*>(&c8[4]) = *reinterpret_cast<const float4*>(&cos_s[tab + 4]);
            *reinterpret_cast<float4*>(&s8[0]) = *reinterpret_cast<const float4*>(&sin_s[tab]);
            *reinterpret_cast<float4*>(&s8[4]) = *reinterpret_cast<const float4*>(&sin_s[tab + 4]);
#pragma unroll
            for (int e = 0; e < 8; e++) {
                y0[e] = __fsub_rn(__fmul_rn(x0[e], c8[e]), __fmul_rn(x1[e], s8[e]));
                y1[e] = __fadd_rn(__fmul_rn(x0[e], s8[e]), __fmul_rn(x1[e], c8[e]));
            }
            xlo = pack8(y0);
            xhi = pack8(y1);
        }
        if (FMT != KV_RAW && to_cache && staged) {
            /* hand the rotated FP16 K to the whole CTA for encoding (phase D) */
            k_stage[(rl * 2 + 0) * kcols + (c - first_k_col)] = xlo;
            k_stage[(rl * 2 + 1) * kcols + (c - first_k_col)] = xhi;
        } else if (FMT != KV_RAW && to_cache) {
            if constexpr (FMT != KV_RAW && !kv_is_tq(FMT)) {
                /* one byte per element: vector i of the row is 8 bytes at uint2 index i */
                uint2* d8 = reinterpret_cast<uint2*>(A.k_cache) +
                            (cache_row(PAGED ? A.page_table : nullptr, dst_row_first + row0 + rl) * stride + (size_t)(dst - A.k_cache));
                const bool sub = A.k_ref != nullptr;
                __stcs(d8, fp8_encode8<FMT>(xlo, sub ? &rlo : nullptr));
                __stcs(d8 + a.hvn, fp8_encode8<FMT>(xhi, sub ? &rhi : nullptr));
            }
            /* (a TurboQuant launch always stages: the launcher plans the tile to fit) */
        } else {
            const size_t drow = to_cache ? cache_row(PAGED ? A.page_table : nullptr, dst_row_first + row0 + rl)
                                         : (size_t)(row0 + rl);
            vec16* d = dst + drow * stride;
            st_stream(d, xlo);
            st_stream(d + a.hvn, xhi);
        }
        if (dst_keep != nullptr) {
            vec16* d2 = dst_keep + (size_t)(row0 + rl) * stride;
            st_stream(d2, xlo);
            st_stream(d2 + a.hvn, xhi);
        }
    }

    /* Phase D (FP8): the encoder costs several times the rotation, and the K
     * columns of a CTA sit in few of its warps (one of eight for the 7B shape),
     * which would finish long after the others. The staged K tile is therefore
     * encoded by ALL threads, one 16-byte vector (8 bytes out) at a time;
     * consecutive threads write consecutive 8-byte pieces of a cache row. */
    if constexpr (kv_is_tq(FMT)) {
        if (staged) {
            __syncthreads();
            constexpr int BPV = tq_bytes_per_vec(FMT);
            const int warp = t >> 5, lane = t & 31;
            const int heads = kcols / a.hvn;                       /* K heads of this column chunk */
            const int head0 = first_k_col / a.hvn - a.n_q;         /* first of them, as a KV head index */
            /* eight lanes to a head vector (tq_store16), four vectors per warp and step: this lane's
             * values 16 sub .. 16 sub + 15 are two 16-byte pieces of the low (sub < 4) or high half */
            const int sub = lane & 7, half_sel = sub >> 2, vsel = 2 * (sub & 3);
            constexpr int kWarps = kRopeThreads / 32;
            uint32_t flip[8];
            tq_flips16(sub, flip);
            const int total = nrows * heads;
            const int step_r = (4 * kWarps) / heads, step_h = 4 * kWarps - step_r * heads;
            const int idx0 = 4 * warp + (lane >> 3);
            int rl = idx0 / heads, hk = idx0 - rl * heads;
            for (int base = 4 * warp; base < total; base += 4 * kWarps) {          /* warp-uniform */
                const bool live = base + (lane >> 3) < total;
                const int rs = live ? rl : 0, hs = live ? hk : 0;
                const vec16* src16 = &k_stage[(rs * 2 + half_sel) * kcols + hs * a.hvn + vsel];
                const vec16 x0 = src16[0], x1 = src16[1];
                const int h = head0 + hs;
                const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&x0);
                const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&x1);
                float v16[16];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float2 f0 = unpack2(w0[i] ^ flip[i]), f1 = unpack2(w1[i] ^ flip[4 + i]);
                    v16[2 * i] = f0.x; v16[2 * i + 1] = f0.y;
                    v16[8 + 2 * i] = f1.x; v16[8 + 2 * i + 1] = f1.y;
                }
                if (A.k_ref != nullptr) {
                    /* (x - ref) * sign == x * sign - ref * sign: the reference key gets the same flips */
                    const vec16 r0 = __ldg(A.k_ref + h * 16 + 2 * sub), r1 = __ldg(A.k_ref + h * 16 + 2 * sub + 1);
                    const uint32_t* q0 = reinterpret_cast<const uint32_t*>(&r0);
                    const uint32_t* q1 = reinterpret_cast<const uint32_t*>(&r1);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float2 f0 = unpack2(q0[i] ^ flip[i]), f1 = unpack2(q1[i] ^ flip[4 + i]);
                        v16[2 * i] = __fsub_rn(v16[2 * i], f0.x); v16[2 * i + 1] = __fsub_rn(v16[2 * i + 1], f0.y);
                        v16[8 + 2 * i] = __fsub_rn(v16[8 + 2 * i], f1.x); v16[8 + 2 * i + 1] = __fsub_rn(v16[8 + 2 * i + 1], f1.y);
                    }
                }
                const size_t at = cache_row(PAGED ? A.page_table : nullptr, cache_first + row0 + rs) * a.n_kv + h;
                tq_store16<FMT>(v16, lane, reinterpret_cast<uint8_t*>(A.k_cache) + at * BPV, A.k_meta + at, live, tq_cells);
                hk += step_h;
                rl += step_r;
                if (hk >= heads) { hk -= heads; rl++; }
            }
        }
    } else if (FMT != KV_RAW && staged) {
        __syncthreads();
        const size_t stride_k = (size_t)a.n_kv * vph;
        for (int idx = t; idx < nrows * 2 * kcols; idx += kRopeThreads) {
            const int rh = idx / kcols;                    /* (row, half) */
            const int kc = idx - rh * kcols;
            const int rl = rh >> 1;
            const int ck = first_k_col + kc;
            const int hd = ck / a.hvn;
            const size_t off = (size_t)(hd - a.n_q) * vph + (size_t)(ck - hd * a.hvn) + ((rh & 1) ? (size_t)a.hvn : 0);
            uint2* d8 = reinterpret_cast<uint2*>(A.k_cache) +
                        (cache_row(PAGED ? A.page_table : nullptr, cache_first + row0 + rl) * stride_k + off);
            const vec16 x = k_stage[idx];
            if (A.k_ref != nullptr) {
                const vec16 r = __ldg(A.k_ref + off);
                __stcs(d8, fp8_encode8<FMT>(x, &r));
            } else {
                __stcs(d8, fp8_encode8<FMT>(x, nullptr));
            }
        }
    }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace vvb

using namespace vvb;

/* Returns cudaErrorNotSupported without launching when head_dim is not a
 * multiple of 16 or a pointer is not 16-byte aligned. */
extern "C" int vvbk_rope_append(void* q, void* k, const void* v,
                                const void* q_bias, const void* k_bias, const void* v_bias,
                                void* k_cache, void* v_cache,
                                int rows, int n_q_heads, int n_kv_heads, int head_dim,
                                int position_offset, int cache_offset, const int* d_position,
                                const float* inv_freq, int keep_k, int kv_format, const void* k_ref,
                                const int* page_table, void* k_meta, void* v_meta, void* stream) {
    if (kv_format < KV_RAW || kv_format > KV_TQ1_5 || !aligned16(k_ref)) return (int)cudaErrorNotSupported;
    const bool tq = kv_is_tq(kv_format);
    if (tq && (head_dim != 128 || k_meta == nullptr || v_meta == nullptr || n_kv_heads > 32 ||
               (reinterpret_cast<uintptr_t>(k_meta) & 1u) || (reinterpret_cast<uintptr_t>(v_meta) & 1u)))
        return (int)cudaErrorNotSupported;
    if (head_dim % 16 != 0 || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(q_bias) ||
        !aligned16(k_bias) || !aligned16(v_bias) || !aligned16(k_cache) || !aligned16(v_cache))
        return (int)cudaErrorNotSupported;
    RopeAppendArgs A;
    unsigned gx, gy;
    /* a flat grid: the V CTAs first, then the tiles over the Q and K heads */
    /* TurboQuant: the CTA's rotated K tile (its K columns x 2 halves x its rows) must fit the
     * 512-vector staging buffer, which bounds the rows a CTA takes */
    int max_passes = kRopeMaxRowsPerThread;
    if (tq) {
        const int kcols = n_kv_heads * (head_dim / 16);          /* <= 256: one column chunk holds them all */
        const int fit = 512 / (2 * kcols);
        if (fit < 1) return (int)cudaErrorNotSupported;
        if (max_passes > fit) max_passes = fit;
    }
    rope_plan(A.r, q, k, rows, n_q_heads, n_kv_heads, head_dim, position_offset, d_position, inv_freq,
              max_passes, &gx, &gy);
    const unsigned gx_v = (unsigned)((rows + kVRowsPerCta - 1) / kVRowsPerCta);
    A.v_ctas = (int)gx_v;
    A.row_tiles = (int)gx;
    const unsigned long long total = (unsigned long long)gx * gy + gx_v;
    if (total > 0x7fffffffull) return (int)cudaErrorInvalidValue;
    A.v = (const vec16*)v;
    A.k_cache = (vec16*)k_cache;
    A.v_cache = (vec16*)v_cache;
    A.q_bias = (const vec16*)q_bias;
    A.k_bias = (const vec16*)k_bias;
    A.v_bias = (const vec16*)v_bias;
    A.k_ref = (kv_format == KV_RAW) ? nullptr : (const vec16*)k_ref;
    A.k_meta = (__half*)k_meta;
    A.v_meta = (__half*)v_meta;
    A.page_table = page_table;
    A.cache_offset = cache_offset;
    A.keep_k = keep_k;
    const dim3 grid((unsigned)total), block(kRopeThreads);
    cudaStream_t s = (cudaStream_t)stream;
    /* the paged mapping is a template parameter so that the contiguous cache pays nothing for it */
#define VVB_APPEND_CASE(F)                                                                          \
    case F:                                                                                         \
        if (page_table == nullptr) launch_pdl(rope_append_kernel<F, false>, grid, block, 0, s, A);  \
        else launch_pdl(rope_append_kernel<F, true>, grid, block, 0, s, A);                         \
        break;
    switch (kv_format) {
        VVB_APPEND_CASE(KV_E4M3)
        VVB_APPEND_CASE(KV_E5M2)
        VVB_APPEND_CASE(KV_TQ4)
        VVB_APPEND_CASE(KV_TQ3)
        VVB_APPEND_CASE(KV_TQ2)
        VVB_APPEND_CASE(KV_TQ1_5)
        default:
            if (page_table == nullptr) launch_pdl(rope_append_kernel<KV_RAW, false>, grid, block, 0, s, A);
            else launch_pdl(rope_append_kernel<KV_RAW, true>, grid, block, 0, s, A);
    }
#undef VVB_APPEND_CASE
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}
