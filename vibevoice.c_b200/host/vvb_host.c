/*
 * vvb_host.c -- C11 host layer, part 2: token-row sharding and the
 * host-buffer pipeline.
 *
 * vvb_shard_rows is the whole multi-GPU story of this path: rows are
 * independent, so GPU g of n takes a contiguous block of rows and RoPE is told
 * the block's first position (the reference's position_offset parameter,
 * src/cuda/rope.cu:49). There is no exchange step and no collective.
 *
 * The pipeline serves callers whose tensors are in host memory (the
 * reference's engine keeps activations on the device, so it has no
 * counterpart there: the nearest thing is its chunked prefill, which also
 * walks the prompt in slices of at most 2048 rows,
 * src/inference/decoder.c:1147-1177). A slice's rows travel host -> device on
 * one stream, run the three kernels on a second, and travel back on a third;
 * three sets of device buffers rotate so that slice i+1 uploads and slice i-1
 * downloads while slice i computes. The math runs only on the GPU.
 *
 * vvb_host_multi_t puts one such pipeline on each of several GPUs: a call
 * splits the rows with vvb_shard_rows and drives every device from a host
 * thread of its own (the reference's multi-device code also walks its devices
 * from the host, src/inference/pipeline.c:389-513, src/cuda/cuda_utils.cu:301-325),
 * so a caller with host buffers gets all the GPUs of the box from one call.
 */
#include "vvb200.h"

#include <cuda_runtime_api.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* --------------------------------------------------------------- sharding */

vv_status_t vvb_shard_rows(int64_t total_rows, int parts, int part,
                           int64_t* first, int64_t* count) {
    if (!first || !count) return VV_ERR_NULL_PTR;
    if (total_rows < 0 || parts <= 0 || part < 0 || part >= parts) return VV_ERR_INVALID_ARG;
    const int64_t block = (total_rows + parts - 1) / parts;
    int64_t lo = block * part;
    if (lo > total_rows) lo = total_rows;
    int64_t hi = lo + block;
    if (hi > total_rows) hi = total_rows;
    *first = lo;
    *count = hi - lo;
    return VV_OK;
}

/* --------------------------------------------------------------- pipeline */

#define VVB_SLOTS 3
#define VVB_TAIL_MIN_ROWS 128      /* the tapering of the last slices stops here */

typedef struct vvb_slot {
    void *hidden, *delta, *normed, *q, *k, *gate, *up;
    cudaEvent_t uploaded, computed, downloaded;
} vvb_slot_t;

struct vvb_host_ctx {
    int device, max_rows;
    int hidden_size, n_q_heads, n_kv_heads, head_dim, inter;
    void* norm_w;
    cudaStream_t s_up, s_run, s_down;
    vvb_slot_t slot[VVB_SLOTS];
    cudaEvent_t t_begin, t_end;      /* timing events bracketing one call */
    uint64_t last_h2d, last_d2h;
    float last_ms;
};

static vv_status_t cuda_status(cudaError_t e) {
    if (e == cudaSuccess) return VV_OK;
    if (e == cudaErrorMemoryAllocation) return VV_ERR_CUDA_OOM;
    return VV_ERR_CUDA;
}

#define CK(call)                                   \
    do {                                           \
        cudaError_t e_ = (call);                   \
        if (e_ != cudaSuccess) { st = cuda_status(e_); goto fail; } \
    } while (0)

void vvb_host_ctx_destroy(vvb_host_ctx_t* c) {
    if (!c) return;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(c->device);
    if (c->s_down) cudaStreamSynchronize(c->s_down);
    for (int i = 0; i < VVB_SLOTS; i++) {
        vvb_slot_t* s = &c->slot[i];
        cudaFree(s->hidden); cudaFree(s->delta); cudaFree(s->normed);
        cudaFree(s->q); cudaFree(s->k); cudaFree(s->gate); cudaFree(s->up);
        if (s->uploaded) cudaEventDestroy(s->uploaded);
        if (s->computed) cudaEventDestroy(s->computed);
        if (s->downloaded) cudaEventDestroy(s->downloaded);
    }
    cudaFree(c->norm_w);
    if (c->t_begin) cudaEventDestroy(c->t_begin);
    if (c->t_end) cudaEventDestroy(c->t_end);
    if (c->s_up) cudaStreamDestroy(c->s_up);
    if (c->s_run) cudaStreamDestroy(c->s_run);
    if (c->s_down) cudaStreamDestroy(c->s_down);
    if (prev >= 0) cudaSetDevice(prev);
    free(c);
}

vv_status_t vvb_host_ctx_create(vvb_host_ctx_t** out, int device, int max_slice_rows,
                                int hidden_size, int n_q_heads, int n_kv_heads,
                                int head_dim, int inter) {
    if (!out) return VV_ERR_NULL_PTR;
    *out = NULL;
    if (device < 0 || max_slice_rows <= 0 || hidden_size <= 0 || n_q_heads < 0 ||
        n_kv_heads < 0 || head_dim < 0 || inter < 0)
        return VV_ERR_INVALID_ARG;
    vvb_host_ctx_t* c = (vvb_host_ctx_t*)calloc(1, sizeof *c);
    if (!c) return VV_ERR_OUT_OF_MEMORY;
    vv_status_t st = VV_OK;
    c->device = device;
    c->max_rows = max_slice_rows;
    c->hidden_size = hidden_size;
    c->n_q_heads = n_q_heads;
    c->n_kv_heads = n_kv_heads;
    c->head_dim = head_dim;
    c->inter = inter;
    int prev = -1;
    cudaGetDevice(&prev);
    CK(cudaSetDevice(device));
    const size_t rows = (size_t)max_slice_rows;
    const size_t hb = rows * (size_t)hidden_size * 2u;
    const size_t qb = rows * (size_t)n_q_heads * (size_t)head_dim * 2u;
    const size_t kb = rows * (size_t)n_kv_heads * (size_t)head_dim * 2u;
    const size_t ib = rows * (size_t)inter * 2u;
    CK(cudaStreamCreateWithFlags(&c->s_up, cudaStreamNonBlocking));
    CK(cudaStreamCreateWithFlags(&c->s_run, cudaStreamNonBlocking));
    CK(cudaStreamCreateWithFlags(&c->s_down, cudaStreamNonBlocking));
    CK(cudaMalloc(&c->norm_w, (size_t)hidden_size * 2u));
    CK(cudaEventCreate(&c->t_begin));
    CK(cudaEventCreate(&c->t_end));
    for (int i = 0; i < VVB_SLOTS; i++) {
        vvb_slot_t* s = &c->slot[i];
        CK(cudaMalloc(&s->hidden, hb));
        CK(cudaMalloc(&s->delta, hb));
        CK(cudaMalloc(&s->normed, hb));
        CK(cudaMalloc(&s->q, qb ? qb : 16));
        CK(cudaMalloc(&s->k, kb ? kb : 16));
        CK(cudaMalloc(&s->gate, ib ? ib : 16));
        CK(cudaMalloc(&s->up, ib ? ib : 16));
        CK(cudaEventCreateWithFlags(&s->uploaded, cudaEventDisableTiming));
        CK(cudaEventCreateWithFlags(&s->computed, cudaEventDisableTiming));
        CK(cudaEventCreateWithFlags(&s->downloaded, cudaEventDisableTiming));
    }
    if (prev >= 0) cudaSetDevice(prev);
    *out = c;
    return VV_OK;
fail:
    vvb_host_ctx_destroy(c);
    if (prev >= 0) cudaSetDevice(prev);
    return st;
}

vv_status_t vvb_layer_chain_host(vvb_host_ctx_t* c, const vvb_layer_chain_t* h) {
    if (!c || !h) return VV_ERR_NULL_PTR;
    if (h->rows == 0) {                 /* nothing to do, whatever the pointers are */
        c->last_h2d = c->last_d2h = 0;
        c->last_ms = 0.0f;
        return VV_OK;
    }
    if (!h->hidden || !h->delta || !h->norm_w || !h->normed) return VV_ERR_NULL_PTR;
    if ((h->n_q_heads > 0 && !h->q) || (h->n_kv_heads > 0 && !h->k)) return VV_ERR_NULL_PTR;
    if (h->inter > 0 && (!h->gate || !h->up)) return VV_ERR_NULL_PTR;
    if (h->rows < 0) return VV_ERR_INVALID_ARG;
    if (h->hidden_size != c->hidden_size || h->n_q_heads != c->n_q_heads ||
        h->n_kv_heads != c->n_kv_heads || h->head_dim != c->head_dim || h->inter != c->inter)
        return VV_ERR_INVALID_ARG;
    vv_status_t st = VV_OK;
    int prev = -1;
    cudaGetDevice(&prev);
    CK(cudaSetDevice(c->device));
    c->last_h2d = c->last_d2h = 0;

    const size_t hrow = (size_t)c->hidden_size * 2u;
    const size_t qrow = (size_t)c->n_q_heads * (size_t)c->head_dim * 2u;
    const size_t krow = (size_t)c->n_kv_heads * (size_t)c->head_dim * 2u;
    const size_t irow = (size_t)c->inter * 2u;

    CK(cudaEventRecord(c->t_begin, c->s_up));
    CK(cudaMemcpyAsync(c->norm_w, h->norm_w, hrow, cudaMemcpyHostToDevice, c->s_up));
    c->last_h2d += hrow;

    /* Slices are max_rows long until the last max_rows of the prompt, which go in halves
     * (1024 -> 512, 256, 128, 128): the upload stream is the busy one, and what follows its last
     * copy -- the last slice's kernels and download -- overlaps nothing, so that slice is
     * kept short. */
    int slice = 0;
    for (int r0 = 0, n = 0; r0 < h->rows; r0 += n, slice++) {
        const int left = h->rows - r0;
        n = left < c->max_rows ? left : c->max_rows;
        if (left <= c->max_rows && left > VVB_TAIL_MIN_ROWS) n = (left + 1) / 2;
        vvb_slot_t* s = &c->slot[slice % VVB_SLOTS];
        const size_t off = (size_t)r0;

        /* upload: the slot is free once its previous download has finished */
        if (slice >= VVB_SLOTS) CK(cudaStreamWaitEvent(c->s_up, s->downloaded, 0));
        CK(cudaMemcpyAsync(s->hidden, (const char*)h->hidden + off * hrow, n * hrow, cudaMemcpyHostToDevice, c->s_up));
        CK(cudaMemcpyAsync(s->delta, (const char*)h->delta + off * hrow, n * hrow, cudaMemcpyHostToDevice, c->s_up));
        if (qrow) CK(cudaMemcpyAsync(s->q, (const char*)h->q + off * qrow, n * qrow, cudaMemcpyHostToDevice, c->s_up));
        if (krow) CK(cudaMemcpyAsync(s->k, (const char*)h->k + off * krow, n * krow, cudaMemcpyHostToDevice, c->s_up));
        if (irow) {
            CK(cudaMemcpyAsync(s->gate, (const char*)h->gate + off * irow, n * irow, cudaMemcpyHostToDevice, c->s_up));
            CK(cudaMemcpyAsync(s->up, (const char*)h->up + off * irow, n * irow, cudaMemcpyHostToDevice, c->s_up));
        }
        CK(cudaEventRecord(s->uploaded, c->s_up));
        c->last_h2d += (uint64_t)n * (2 * hrow + qrow + krow + 2 * irow);

        /* compute */
        CK(cudaStreamWaitEvent(c->s_run, s->uploaded, 0));
        vvb_layer_chain_t d = *h;
        d.hidden = s->hidden; d.delta = s->delta; d.norm_w = c->norm_w; d.normed = s->normed;
        d.q = s->q; d.k = s->k; d.gate = s->gate; d.up = s->up;
        d.rows = n;
        d.position_offset = h->position_offset + r0;
        st = vvb_layer_chain_dev(&d, c->s_run);
        if (st != VV_OK) goto fail;
        CK(cudaEventRecord(s->computed, c->s_run));

        /* download */
        CK(cudaStreamWaitEvent(c->s_down, s->computed, 0));
        CK(cudaMemcpyAsync((char*)h->hidden + off * hrow, s->hidden, n * hrow, cudaMemcpyDeviceToHost, c->s_down));
        CK(cudaMemcpyAsync((char*)h->normed + off * hrow, s->normed, n * hrow, cudaMemcpyDeviceToHost, c->s_down));
        if (qrow) CK(cudaMemcpyAsync((char*)h->q + off * qrow, s->q, n * qrow, cudaMemcpyDeviceToHost, c->s_down));
        if (krow) CK(cudaMemcpyAsync((char*)h->k + off * krow, s->k, n * krow, cudaMemcpyDeviceToHost, c->s_down));
        if (irow) CK(cudaMemcpyAsync((char*)h->gate + off * irow, s->gate, n * irow, cudaMemcpyDeviceToHost, c->s_down));
        CK(cudaEventRecord(s->downloaded, c->s_down));
        c->last_d2h += (uint64_t)n * (2 * hrow + qrow + krow + irow);
    }
    /* the end marker waits for the last upload too */
    CK(cudaEventRecord(c->slot[0].uploaded, c->s_up));
    CK(cudaStreamWaitEvent(c->s_down, c->slot[0].uploaded, 0));
    CK(cudaEventRecord(c->t_end, c->s_down));
    CK(cudaStreamSynchronize(c->s_down));
    c->last_ms = 0.0f;
    cudaEventElapsedTime(&c->last_ms, c->t_begin, c->t_end);
    if (prev >= 0) cudaSetDevice(prev);
    return VV_OK;
fail:
    /* leave nothing in flight that still points into the caller's buffers */
    cudaStreamSynchronize(c->s_up);
    cudaStreamSynchronize(c->s_run);
    cudaStreamSynchronize(c->s_down);
    if (prev >= 0) cudaSetDevice(prev);
    return st;
}

float vvb_host_ctx_last_ms(const vvb_host_ctx_t* c) { return c ? c->last_ms : 0.0f; }

void vvb_host_ctx_last_traffic(const vvb_host_ctx_t* c, uint64_t* h2d_bytes, uint64_t* d2h_bytes) {
    if (h2d_bytes) *h2d_bytes = c ? c->last_h2d : 0;
    if (d2h_bytes) *d2h_bytes = c ? c->last_d2h : 0;
}

/* ----------------------------------------------------- several devices at once */

struct vvb_host_multi {
    int n;
    vvb_host_ctx_t** ctx;      /* one pipeline per device */
    float last_ms;
    uint64_t last_h2d, last_d2h;
};

typedef struct vvb_multi_job {
    vvb_host_ctx_t* ctx;
    vvb_layer_chain_t shard;
    vv_status_t status;
} vvb_multi_job_t;

static void* vvb_multi_worker(void* arg) {
    vvb_multi_job_t* j = (vvb_multi_job_t*)arg;
    j->status = vvb_layer_chain_host(j->ctx, &j->shard);   /* sets the device for this thread */
    return NULL;
}

void vvb_host_multi_destroy(vvb_host_multi_t* m) {
    if (!m) return;
    if (m->ctx) {
        for (int i = 0; i < m->n; i++) vvb_host_ctx_destroy(m->ctx[i]);
        free(m->ctx);
    }
    free(m);
}

vv_status_t vvb_host_multi_create(vvb_host_multi_t** out, const int* devices, int n_devices,
                                  int max_slice_rows, int hidden_size, int n_q_heads,
                                  int n_kv_heads, int head_dim, int inter) {
    if (!out) return VV_ERR_NULL_PTR;
    *out = NULL;
    if (n_devices <= 0 || n_devices > 64) return VV_ERR_INVALID_ARG;
    vvb_host_multi_t* m = (vvb_host_multi_t*)calloc(1, sizeof *m);
    if (!m) return VV_ERR_OUT_OF_MEMORY;
    m->ctx = (vvb_host_ctx_t**)calloc((size_t)n_devices, sizeof *m->ctx);
    if (!m->ctx) { free(m); return VV_ERR_OUT_OF_MEMORY; }
    m->n = n_devices;
    for (int i = 0; i < n_devices; i++) {
        const int dev = devices ? devices[i] : i;      /* NULL: devices 0 .. n-1 */
        const vv_status_t st = vvb_host_ctx_create(&m->ctx[i], dev, max_slice_rows, hidden_size,
                                                   n_q_heads, n_kv_heads, head_dim, inter);
        if (st != VV_OK) { vvb_host_multi_destroy(m); return st; }
    }
    *out = m;
    return VV_OK;
}

int vvb_host_multi_devices(const vvb_host_multi_t* m) { return m ? m->n : 0; }

vv_status_t vvb_layer_chain_host_multi(vvb_host_multi_t* m, const vvb_layer_chain_t* h) {
    if (!m || !h) return VV_ERR_NULL_PTR;
    if (h->rows < 0) return VV_ERR_INVALID_ARG;
    if (m->n > 64) return VV_ERR_INVALID_ARG;
    vvb_multi_job_t job[64];
    pthread_t thread[64];
    int started[64];
    const size_t hrow = (size_t)h->hidden_size * 2u;
    const size_t qrow = (size_t)h->n_q_heads * (size_t)h->head_dim * 2u;
    const size_t krow = (size_t)h->n_kv_heads * (size_t)h->head_dim * 2u;
    const size_t irow = (size_t)h->inter * 2u;
    for (int g = 0; g < m->n; g++) {
        int64_t first = 0, count = 0;
        vv_status_t st = vvb_shard_rows(h->rows, m->n, g, &first, &count);
        if (st != VV_OK) return st;
        vvb_layer_chain_t* s = &job[g].shard;
        *s = *h;
        const size_t off = (size_t)first;
        s->hidden = h->hidden ? (char*)h->hidden + off * hrow : NULL;
        s->delta = h->delta ? (const char*)h->delta + off * hrow : NULL;
        s->normed = h->normed ? (char*)h->normed + off * hrow : NULL;
        s->q = h->q ? (char*)h->q + off * qrow : NULL;
        s->k = h->k ? (char*)h->k + off * krow : NULL;
        s->gate = h->gate ? (char*)h->gate + off * irow : NULL;
        s->up = h->up ? (const char*)h->up + off * irow : NULL;
        s->rows = (int)count;
        s->position_offset = h->position_offset + (int)first;    /* the shard's first token position */
        job[g].ctx = m->ctx[g];
        job[g].status = VV_OK;
    }
    /* one host thread per device; the calling thread takes device 0's shard itself */
    for (int g = 1; g < m->n; g++) {
        started[g] = pthread_create(&thread[g], NULL, vvb_multi_worker, &job[g]) == 0;
        if (!started[g]) vvb_multi_worker(&job[g]);      /* no thread to be had: run it here, in turn */
    }
    vvb_multi_worker(&job[0]);
    for (int g = 1; g < m->n; g++)
        if (started[g]) pthread_join(thread[g], NULL);
    vv_status_t result = VV_OK;
    m->last_ms = 0.0f;
    m->last_h2d = m->last_d2h = 0;
    for (int g = 0; g < m->n; g++) {
        if (job[g].status != VV_OK && result == VV_OK) result = job[g].status;
        const float ms = vvb_host_ctx_last_ms(m->ctx[g]);
        if (ms > m->last_ms) m->last_ms = ms;
        uint64_t a = 0, b = 0;
        vvb_host_ctx_last_traffic(m->ctx[g], &a, &b);
        m->last_h2d += a;
        m->last_d2h += b;
    }
    return result;
}

float vvb_host_multi_last_ms(const vvb_host_multi_t* m) { return m ? m->last_ms : 0.0f; }

void vvb_host_multi_last_traffic(const vvb_host_multi_t* m, uint64_t* h2d_bytes, uint64_t* d2h_bytes) {
    if (h2d_bytes) *h2d_bytes = m ? m->last_h2d : 0;
    if (d2h_bytes) *d2h_bytes = m ? m->last_d2h : 0;
}
