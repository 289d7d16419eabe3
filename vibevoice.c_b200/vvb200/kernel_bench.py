"""Per-kernel timings at the BASELINE shapes (configs 1-4) and for the int8
activation quantizers: `python bench.py --workload kernels`.

Each case is launched `iters` times from one CUDA graph over rotating buffer
sets whose total size exceeds 2.5x the L2 (so every launch reads cold HBM even
when one set would fit in the cache), timed with CUDA events on the replaying
stream; the figure is the best of three replays divided by `iters`. A second
figure, `warm_us`, replays over a single buffer set (L2-resident for the small
shapes) and is the launch latency a decode step sees; it is never reported as
HBM bandwidth.
"""
from __future__ import annotations

import json

import torch

import vvb200 as vv

H, NQ, NKV, HD, INTER, VOCAB = 3584, 28, 4, 128, 18944, 151936
L2_BYTES = 126e6


def _time_graph(fn, nsets, iters):
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for i in range(min(nsets, 3)):
            fn(i % nsets, s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for i in range(iters):
                fn(i % nsets, s)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = float("inf")
        for _ in range(3):
            e0.record(s)
            g.replay()
            e1.record(s)
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) * 1e3 / iters)
    return best


def _nsets(bytes_per_set):
    return max(1, min(48, int(2.5 * L2_BYTES / bytes_per_set) + 1))


ONLY = None      # substring filter on case names (bench.py --case), for profiler runs
PLAIN = False    # direct launches, few of them, instead of graph replays (bench.py --plain-launches)


def _case(name, make_set, call, set_bytes, algo_bytes, peak, iters=40):
    if ONLY is not None and ONLY not in name:
        return None
    if PLAIN:
        # a handful of direct launches over two buffer sets: what a profiler capture wants
        sets = [make_set() for _ in range(2)]
        s = torch.cuda.current_stream()
        for i in range(4):
            call(sets[i % 2], s)
        torch.cuda.synchronize()
        return {"case": name, "plain_launches": 4}
    ns = _nsets(set_bytes)
    sets = [make_set() for _ in range(ns)]
    cold = _time_graph(lambda i, s: call(sets[i], s), ns, iters)
    warm = _time_graph(lambda i, s: call(sets[0], s), 1, iters)
    gbs = algo_bytes / cold / 1e3
    del sets
    torch.cuda.empty_cache()
    return {"case": name, "us": round(cold, 2), "GB/s": round(gbs, 1), "frac_of_peak": round(gbs / peak, 3),
            "algorithmic_bytes": algo_bytes, "buffer_sets": ns, "warm_us": round(warm, 2)}


def run(peak_gbs: float, peak_kind: str):
    dev = torch.device("cuda", torch.cuda.current_device())
    rn = lambda *s: torch.randn(*s, device=dev).half()
    w = (1 + 0.02 * torch.randn(H, device=dev)).half()
    out = []

    def ok(st):
        assert st == 0, st

    # config 1: add + RMSNorm [512, 3584]
    for rows in (512, 4096):
        out.append(_case(
            f"add_rmsnorm [{rows},3584]", lambda: (rn(rows, H), rn(rows, H), torch.empty(rows, H, device=dev, dtype=torch.float16)),
            lambda b, s: ok(vv.vvb_add_rmsnorm_dev(b[0], b[1], w, b[2], rows, H, 1e-6, s)),
            rows * H * 2 * 3, rows * H * 2 * 4 + 2 * H, peak_gbs))
    # config 2: RoPE prefill, Q [4096,28,128] + K [4096,4,128]
    rows = 4096
    out.append(_case(
        "rope_qk [4096,28+4,128]", lambda: (rn(rows, NQ, HD), rn(rows, NKV, HD)),
        lambda b, s: ok(vv.vvb_rope_qk_dev(b[0], b[1], rows, NQ, NKV, HD, 0, None, 1e6, s)),
        rows * (NQ + NKV) * HD * 2, 2 * rows * (NQ + NKV) * HD * 2, peak_gbs))
    # bias + RoPE + KV-cache append in one launch (Q in place; K, V read once and written into the cache)
    rows = 14449
    bq, bk, bv = rn(NQ * HD), rn(NKV * HD), rn(NKV * HD)
    out.append(_case(
        "rope_qk_append [14449,28+4+4,128] with biases",
        lambda: (rn(rows, NQ, HD), rn(rows, NKV, HD), rn(rows, NKV, HD),
                 torch.empty(rows, NKV * HD, device=dev, dtype=torch.float16),
                 torch.empty(rows, NKV * HD, device=dev, dtype=torch.float16)),
        lambda b, s: ok(vv.vvb_rope_qk_append_dev(b[0], b[1], b[2], bq, bk, bv, b[3], b[4], rows, NQ, NKV, HD, 0, 0,
                                                  None, 1e6, 0, s)),
        rows * (NQ + 4 * NKV) * HD * 2, rows * (2 * NQ + 4 * NKV) * HD * 2, peak_gbs))
    # the same launch for the FP8 (E4M3) KV cache: K and V leave as one byte per element, K minus a reference key
    kref = rn(NKV * HD)
    out.append(_case(
        "rope_qk_append_fp8 [14449,28+4+4,128] with biases, e4m3 cache, reference key",
        lambda: (rn(rows, NQ, HD), rn(rows, NKV, HD), rn(rows, NKV, HD),
                 torch.empty(rows, NKV * HD, device=dev, dtype=torch.uint8),
                 torch.empty(rows, NKV * HD, device=dev, dtype=torch.uint8)),
        lambda b, s: ok(vv.vvb_rope_qk_append_fp8_dev(b[0], b[1], b[2], bq, bk, bv, b[3], b[4], kref, rows, NQ, NKV, HD,
                                                      0, 0, None, 1e6, vv.VVB_KV_FP8_E4M3, 0, s)),
        rows * (NQ + 2 * NKV) * HD * 2 + rows * 2 * NKV * HD, rows * (2 * NQ + 2 * NKV) * HD * 2 + rows * 2 * NKV * HD,
        peak_gbs))
    # config 3: SwiGLU [4096,18944] and the decode shape [64,18944], in place on gate
    for rows in (4096, 64):
        out.append(_case(
            f"swiglu [{rows},18944]", lambda: (rn(rows, INTER), rn(rows, INTER)),
            lambda b, s: ok(vv.vvb_swiglu_dev(b[0], b[1], b[0], rows * INTER, s)),
            rows * INTER * 2 * 2, rows * INTER * 2 * 3, peak_gbs))
    # config 4: gather 16384 rows of [151936, 3584] + RMSNorm (fused), and the plain gather
    rows = 16384
    table = torch.empty(VOCAB, H, device=dev, dtype=torch.float16).normal_(0, 0.02)
    mk_ids = lambda: torch.randint(0, VOCAB, (rows,), device=dev, dtype=torch.int32)
    out.append(_case(
        "embedding_rmsnorm 16384 of [151936,3584]",
        lambda: (mk_ids(), torch.empty(rows, H, device=dev, dtype=torch.float16), torch.empty(rows, H, device=dev, dtype=torch.float16)),
        lambda b, s: ok(vv.vvb_embedding_rmsnorm_dev(table, b[0], b[1], w, b[2], rows, H, VOCAB, 1e-6, s)),
        rows * H * 2 * 3, rows * H * 2 * 3 + rows * 4 + 2 * H, peak_gbs, iters=20))
    out.append(_case(
        "embedding 16384 of [151936,3584]",
        lambda: (mk_ids(), torch.empty(rows, H, device=dev, dtype=torch.float16)),
        lambda b, s: ok(vv.vv_embedding_dev(table, b[0], b[1], rows, H, s)),
        rows * H * 2 * 2, rows * H * 2 * 2 + rows * 4, peak_gbs, iters=20))
    del table
    torch.cuda.empty_cache()
    # int8 activation quantizers at long-prompt prefill size (14449 rows), with run sums
    rows = 14449

    def qbufs(K):
        return (torch.empty(rows, K, device=dev, dtype=torch.int8), torch.empty(rows, device=dev, dtype=torch.float32),
                torch.empty(rows, K // 32, device=dev, dtype=torch.int32))

    qout = lambda K: rows * (K + 4 + K // 8)
    for layout, lname in ((0, "natural"), (3, "w4_mma")):
        out.append(_case(
            f"rmsnorm_q8 [14449,3584] {lname}", lambda: (rn(rows, H),) + qbufs(H),
            lambda b, s: ok(vv.vv_rmsnorm_q8_dev(b[0], w, rows, H, 1e-6, layout, b[1], b[2], b[3], s)),
            rows * H * 2 + qout(H), rows * H * 2 + 2 * H + qout(H), peak_gbs))
        out.append(_case(
            f"swiglu_q8 [14449,18944] {lname}", lambda: (rn(rows, INTER), rn(rows, INTER)) + qbufs(INTER),
            lambda b, s: ok(vv.vv_swiglu_q8_dev(b[0], b[1], rows, INTER, layout, b[2], b[3], b[4], s)),
            rows * INTER * 4 + qout(INTER), rows * INTER * 4 + qout(INTER), peak_gbs, iters=20))
    out.append(_case(
        "act_quant [14449,3584] natural", lambda: (rn(rows, H),) + qbufs(H),
        lambda b, s: ok(vv.vv_act_quant_dev(b[0], rows, H, 0, b[1], b[2], b[3], s)),
        rows * H * 2 + qout(H), rows * H * 2 + qout(H), peak_gbs))
    # the decode tail: final RMSNorm + LM head [152064, 3584] + argmax (two launches), and the plain GEMV
    V = 152064
    head = torch.empty(V, H, device=dev, dtype=torch.float16).normal_(0, 0.02)
    sbytes = vv.vvb_lm_head_scratch_bytes(V)
    mk = lambda: (rn(H), torch.empty(sbytes, device=dev, dtype=torch.uint8), torch.empty(1, device=dev, dtype=torch.int32),
                  torch.empty(V, device=dev, dtype=torch.float32))
    out.append(_case(
        "final_norm + lm_head + argmax [152064,3584]", mk,
        lambda b, s: ok(vv.vvb_lm_head_argmax_dev(b[0], w, 1e-6, head, V, H, None, b[1], sbytes, b[2], None, s)),
        V * H * 2, V * H * 2 + 2 * H * 2, peak_gbs, iters=10))
    out.append(_case(
        "lm_head_gemv [152064,3584] (logits)", mk,
        lambda b, s: ok(vv.vv_lm_head_gemv_dev(b[0], head, b[3], V, H, s)),
        V * H * 2, V * H * 2 + V * 4, peak_gbs, iters=10))
    # one decode token (M = 1) of the 28-layer model, this library's kernels only (the GEMMs and the
    # attention between them are the engine's): embedding, then per layer [norm (layer 0) or residual
    # add + norm] -> bias + RoPE + KV append -> residual add + norm -> SwiGLU, then final norm + LM
    # head + argmax; one CUDA graph, replayed. Launch-bound: reported as microseconds per token.
    L, max_len = 28, 64
    table = torch.empty(4096, H, device=dev, dtype=torch.float16).normal_(0, 0.02)
    tok = torch.zeros(1, device=dev, dtype=torch.int32)
    hid, dlt, nrm = rn(1, H), rn(1, H), rn(1, H)
    q1, k1, v1, g1, u1 = rn(1, NQ, HD), rn(1, NKV, HD), rn(1, NKV, HD), rn(1, INTER), rn(1, INTER)
    kc = [torch.zeros(max_len, NKV * HD, device=dev, dtype=torch.float16) for _ in range(L)]
    vc = [torch.zeros(max_len, NKV * HD, device=dev, dtype=torch.float16) for _ in range(L)]
    dpos = torch.tensor([7], device=dev, dtype=torch.int32)
    scr = torch.empty(sbytes, device=dev, dtype=torch.uint8)

    def decode_token(_i, s):
        ok(vv.vvb_embedding_rmsnorm_dev(table, tok, hid, w, nrm, 1, H, 4096, 1e-6, s))
        for layer in range(L):
            if layer:
                ok(vv.vvb_add_rmsnorm_dev(hid, dlt, w, nrm, 1, H, 1e-6, s))
            ok(vv.vvb_rope_qk_append_dev(q1, k1, v1, bq, bk, bv, kc[layer], vc[layer], 1, NQ, NKV, HD, 0, 0, dpos,
                                         1e6, 0, s))
            ok(vv.vvb_add_rmsnorm_dev(hid, dlt, w, nrm, 1, H, 1e-6, s))
            ok(vv.vvb_swiglu_dev(g1, u1, g1, INTER, s))
        ok(vv.vvb_residual_add_dev(hid, dlt, H, s))
        ok(vv.vvb_lm_head_argmax_dev(hid, w, 1e-6, head, V, H, None, scr, sbytes, tok, None, s))

    if not PLAIN and (ONLY is None or ONLY in "decode step"):
        launches0 = vv.launch_count()
        decode_token(0, torch.cuda.current_stream())
        torch.cuda.synchronize()
        n_launch = vv.launch_count() - launches0
        us_tok = _time_graph(decode_token, 1, 5)
        out.append({"case": "decode step, 28 layers, M=1 (row kernels + LM head only)", "us": round(us_tok, 1),
                    "launches": n_launch})
    del head
    torch.cuda.empty_cache()
    return {"workload": "kernels", "peak_GB/s": peak_gbs, "peak_kind": "of " + peak_kind,
            "method": "CUDA-graph replay over rotating buffer sets > 2.5x L2, CUDA events, best of 3",
            "cases": [c for c in out if c is not None]}


def main(peak_gbs, peak_kind, only=None, plain=False):
    global ONLY, PLAIN
    ONLY, PLAIN = only, plain
    print(json.dumps(run(peak_gbs, peak_kind)), flush=True)
