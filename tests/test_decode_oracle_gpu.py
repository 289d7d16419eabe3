"""One decode token (M = 1) of a small stack of layers, composed TWICE: from
CPU-oracle calls in the order the reference's engine issues its ops
(src/inference/decoder.c:810-988 per layer, src/inference/pipeline.c:1962-1986
for the tail), and as this library's launch sequence captured once in a CUDA
graph and replayed while the device-side position and the device-side token
advance (src/inference/decoder.c:1020-1093, pipeline.c:1653-1721). Every
kernel consumes what the one before it produced; the engine's GEMMs and
attention, which are not part of this library, are stood in for by copies of
slices (bit-exact on both sides, so the comparison sees only this library's
arithmetic).

Per replay the hidden state, the cache rows written at the position and the
greedy token are compared with the oracle's. RoPE's bar is 2 FP16 ulp at
operand scale and SwiGLU's 2 ulp, so a rounding-boundary accident in one of
them may move later values by an ulp; the bars below allow that and the test
prints how many elements differed (normally none).
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

H, NQ, NKV, HD, INTER = 3584, 28, 4, 128, 18944
EPS, THETA = 1e-6, 1e6


@pytest.fixture(scope="module")
def vv():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import vvb200
    torch.cuda.set_device(0)
    return vvb200


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bias_add_f16(x, b):
    """vv_bias_add_dev: float sum, one rounding to FP16 (src/cuda/conv_vae.cu:54-66)."""
    return (x.astype(np.float32) + b.astype(np.float32)).astype(np.float16)


def lm_tol(x, w, depth=128):
    return depth * 2.0 ** -24 * (np.abs(w.astype(np.float64)) @ np.abs(x.astype(np.float64)))


@pytest.mark.parametrize("L,V,p0", [(4, 4096, 37), (6, 2048, 900)])
def test_decode_token_sequence_against_oracle(vv, orc, L, V, p0):
    rng = np.random.default_rng(100 * L + p0)
    f16 = lambda *s, scale=1.0: (scale * rng.standard_normal(s)).astype(np.float16)
    max_len, steps = p0 + 8, 3
    table, head = f16(V, H, scale=0.5), f16(V, H, scale=0.02)
    w_in = [(1 + 0.05 * rng.standard_normal(H)).astype(np.float16) for _ in range(L)]
    w_post = [(1 + 0.05 * rng.standard_normal(H)).astype(np.float16) for _ in range(L)]
    w_final = (1 + 0.05 * rng.standard_normal(H)).astype(np.float16)
    bq, bk, bv = [f16(NQ * HD, scale=0.3) for _ in range(L)], [f16(NKV * HD, scale=0.3) for _ in range(L)], \
                 [f16(NKV * HD, scale=0.3) for _ in range(L)]
    up = [f16(1, INTER) for _ in range(L)]
    tok0 = 11

    # ------------------------------------------------------------ oracle, op by op
    def oracle_token(tok, p, kc, vc):
        h = table[tok:tok + 1].copy()                                   # vv_embedding_dev
        _, nrm = orc.add_rmsnorm_f16(h, None, w_in[0], EPS)             # vv_rmsnorm_dev (layer 0)
        for l in range(L):
            # stand-ins for the q/k/v projections: slices of the normed row
            q = nrm[:, :NQ * HD].reshape(1, NQ, HD)
            k = nrm[:, :NKV * HD].reshape(1, NKV, HD)
            v = nrm[:, NKV * HD:2 * NKV * HD].reshape(1, NKV, HD)
            qb = bias_add_f16(q.reshape(1, -1), bq[l]).reshape(q.shape)  # vv_bias_add_dev x3
            kb = bias_add_f16(k.reshape(1, -1), bk[l]).reshape(k.shape)
            vb = bias_add_f16(v.reshape(1, -1), bv[l]).reshape(v.shape)
            qr, kr = orc.rope_f16(qb, p, THETA), orc.rope_f16(kb, p, THETA)   # vv_rope_dev x2 at *d_position
            kc[l][p], vc[l][p] = kr.reshape(-1), vb.reshape(-1)          # vv_kv_cache_append, row *d_position
            # stand-in for attention + o_proj: the rotated queries; residual add + post-attention norm
            h, nrm = orc.add_rmsnorm_f16(h, qr.reshape(1, -1), w_post[l], EPS)
            gate = np.ascontiguousarray(np.tile(nrm, (1, INTER // H + 1))[:, :INTER])   # stand-in for gate_proj
            act = orc.swiglu_f16(gate, up[l])                            # vv_swiglu_dev, in place
            delta = np.ascontiguousarray(act[:, :H])                     # stand-in for down_proj
            if l + 1 < L:
                h, nrm = orc.add_rmsnorm_f16(h, delta, w_in[l + 1], EPS)  # residual add, next layer's input norm
            else:
                h = orc.residual_add_f16(h, delta)                       # the last residual add
        _, xn = orc.add_rmsnorm_f16(h, None, w_final, EPS)               # final norm (FP16 row) ...
        logits, t, _ = orc.restated().lm_head(xn.reshape(-1).astype(np.float32), head)   # ... LM head + argmax
        srt = np.sort(logits)
        return h, t, srt[-1] - srt[-2], lm_tol(xn.reshape(-1), head).max()

    # ------------------------------------------------------------ the GPU sequence, captured once
    d_table, d_head, d_wfin = dev(table), dev(head), dev(w_final)
    d_win, d_wpost = [dev(x) for x in w_in], [dev(x) for x in w_post]
    d_bq, d_bk, d_bv, d_up = ([dev(x) for x in y] for y in (bq, bk, bv, up))
    e16 = lambda *s: torch.empty(*s, device="cuda", dtype=torch.float16)
    hid, nrm, dlt = e16(1, H), e16(1, H), e16(1, H)
    q, k, v, gate = e16(1, NQ, HD), e16(1, NKV, HD), e16(1, NKV, HD), e16(1, INTER)
    d_kc = [torch.zeros(max_len, NKV * HD, device="cuda", dtype=torch.float16) for _ in range(L)]
    d_vc = [torch.zeros(max_len, NKV * HD, device="cuda", dtype=torch.float16) for _ in range(L)]
    dpos = torch.tensor([p0], device="cuda", dtype=torch.int32)
    tok = torch.tensor([tok0], device="cuda", dtype=torch.int32)
    nb = vv.vvb_lm_head_scratch_bytes(V)
    scratch = torch.empty(nb, device="cuda", dtype=torch.uint8)
    hid_out = e16(1, H)
    reps = INTER // H + 1

    def ok(st):
        assert st == 0, st

    def token(s):
        ok(vv.vvb_embedding_rmsnorm_dev(d_table, tok, hid, d_win[0], nrm, 1, H, V, EPS, s))
        for l in range(L):
            q.copy_(nrm[:, :NQ * HD].reshape(1, NQ, HD))
            k.copy_(nrm[:, :NKV * HD].reshape(1, NKV, HD))
            v.copy_(nrm[:, NKV * HD:2 * NKV * HD].reshape(1, NKV, HD))
            ok(vv.vvb_rope_qk_append_dev(q, k, v, d_bq[l], d_bk[l], d_bv[l], d_kc[l], d_vc[l], 1, NQ, NKV, HD, 0, 0,
                                         dpos, THETA, 0, s))
            ok(vv.vvb_add_rmsnorm_dev(hid, q.reshape(1, NQ * HD), d_wpost[l], nrm, 1, H, EPS, s))
            for r in range(reps):
                n = min(H, INTER - r * H)
                gate[:, r * H:r * H + n].copy_(nrm[:, :n])
            ok(vv.vvb_swiglu_dev(gate, d_up[l], gate, INTER, s))
            dlt.copy_(gate[:, :H])
            if l + 1 < L:
                ok(vv.vvb_add_rmsnorm_dev(hid, dlt, d_win[l + 1], nrm, 1, H, EPS, s))
            else:
                ok(vv.vvb_residual_add_dev(hid, dlt, H, s))
        hid_out.copy_(hid)
        ok(vv.vvb_lm_head_argmax_dev(hid, d_wfin, EPS, d_head, V, H, None, scratch, nb, tok, None, s))
        dpos.add_(1)                                   # the engine's vv_pos_add_dev, on the stream

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        token(stream.cuda_stream)                      # warm the library before capture
        torch.cuda.synchronize()
        dpos.fill_(p0)
        tok.fill_(tok0)
        for c in d_kc + d_vc:
            c.zero_()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            token(stream.cuda_stream)

    kc = [np.zeros((max_len, NKV * HD), np.float16) for _ in range(L)]
    vc = [np.zeros((max_len, NKV * HD), np.float16) for _ in range(L)]
    cur, differing = tok0, 0
    for step in range(steps):
        p = p0 + step
        for t_ in (hid, nrm, gate, q, k):
            t_.fill_(3.0)                              # stale data a wrong dependency would pick up
        graph.replay()
        torch.cuda.synchronize()
        assert int(dpos.item()) == p + 1
        want_h, want_tok, margin, tol = oracle_token(cur, p, kc, vc)
        got_h = hid_out.cpu().numpy()
        dh = orc.ulp_distance(got_h, want_h)
        differing += int((dh > 0).sum())
        assert dh.max() <= 4 and (dh > 0).mean() < 1e-2, (step, int(dh.max()))
        for l in range(L):
            got_k, got_v = d_kc[l].cpu().numpy(), d_vc[l].cpu().numpy()
            dk = orc.ulp_distance(got_k[p], kc[l][p])
            dv = orc.ulp_distance(got_v[p], vc[l][p])
            differing += int((dk > 0).sum() + (dv > 0).sum())
            # K row: RoPE's bar (absolute, at operand scale, 2 ulp) -- plus an upstream ulp
            err = np.abs(got_k[p].astype(np.float32) - kc[l][p].astype(np.float32))
            scale = orc.f16_ulp_of(np.maximum(np.abs(kc[l][p].astype(np.float32)), 1.0))
            assert (err <= 4 * scale).all(), (step, l)
            assert dv.max() <= 2, (step, l)            # V: bias sum of a normed slice, a bit copy after that
            # rows of earlier positions keep the oracle's bytes, later rows stay empty
            assert not got_k[p + 1:].any() and not got_v[p + 1:].any()
        got_tok = int(tok.item())
        if margin > 2 * tol:
            assert got_tok == want_tok, (step, got_tok, want_tok)
        cur = got_tok                                  # follow the GPU's token: the next replay embeds it
    print(f"decode sequence L={L}: {differing} element(s) differed from the oracle over {steps} tokens")
