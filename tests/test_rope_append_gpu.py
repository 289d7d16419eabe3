"""vvb_rope_qk_append_dev: bias add + RoPE + KV-cache append in one launch,
against (a) the oracle composed the way the reference's engine composes its
ops and (b) this library's own separate ops followed by a device copy."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROPE_ULP = 2.0


@pytest.fixture(scope="module")
def vv():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import vvb200
    torch.cuda.set_device(0)
    return vvb200


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(t):
    torch.cuda.synchronize()
    return t.cpu().numpy().view(np.uint16)


def bias_add_f16(x, b):
    """vv_bias_add_dev's arithmetic: float sum, one rounding to FP16
    (src/cuda/conv_vae.cu:54-66)."""
    return (x.astype(np.float32) + b.astype(np.float32)).astype(np.float16)


@pytest.mark.parametrize("rows,nq,nkv,hd,pos,cache_off,with_bias,keep_k", [
    (1, 28, 4, 128, 913, 913, True, 0),         # a decode step
    (300, 28, 4, 128, 0, 0, True, 1),           # prefill from an empty cache, K kept
    (2048, 28, 4, 128, 4096, 4096, False, 0),   # third 2048-row chunk of a long prompt, no biases
    (48, 2, 1, 128, 5, 5, True, 0),             # the reference's tiny test model
    (17, 12, 2, 128, 100, 40, True, 0),         # BitNet-1.5B heads; cache row != position
    (9, 3, 3, 64, 7, 0, True, 1),
    (70, 40, 8, 128, 33, 33, True, 1),          # 384 columns: two column chunks, K in the second
    (37, 16, 2, 256, 3, 9, True, 0),            # head_dim 256: 288 columns, K split over both chunks' ends
])
def test_rope_append_matches_oracle_and_separate_ops(vv, orc, rows, nq, nkv, hd, pos, cache_off, with_bias, keep_k):
    rng = np.random.default_rng(rows * 31 + nq)
    f16 = lambda *s: rng.standard_normal(s).astype(np.float16)
    q, k, v = f16(rows, nq, hd), f16(rows, nkv, hd), f16(rows, nkv, hd)
    bq, bk, bv = (f16(nq * hd), f16(nkv * hd), f16(nkv * hd)) if with_bias else (None, None, None)
    max_len = cache_off + rows + 3
    kc0, vc0 = f16(max_len, nkv * hd), f16(max_len, nkv * hd)       # pre-existing cache contents

    # ---- oracle, in the engine's order: bias adds, RoPE, append
    qb = bias_add_f16(q.reshape(rows, -1), bq).reshape(q.shape) if with_bias else q
    kb = bias_add_f16(k.reshape(rows, -1), bk).reshape(k.shape) if with_bias else k
    vb = bias_add_f16(v.reshape(rows, -1), bv).reshape(v.shape) if with_bias else v
    want_q, want_k = orc.rope_f16(qb, pos, 1e6), orc.rope_f16(kb, pos, 1e6)
    want_kc, want_vc = kc0.copy(), vc0.copy()
    want_kc[cache_off:cache_off + rows] = want_k.reshape(rows, -1)
    want_vc[cache_off:cache_off + rows] = vb.reshape(rows, -1)

    dq, dk, dv_, dkc, dvc = dev(q), dev(k), dev(v), dev(kc0), dev(vc0)
    n0 = vv.launch_count()
    st = vv.vvb_rope_qk_append_dev(dq, dk, dv_, dev(bq) if with_bias else None, dev(bk) if with_bias else None,
                                   dev(bv) if with_bias else None, dkc, dvc, rows, nq, nkv, hd, pos, cache_off, None,
                                   1e6, keep_k)
    assert st == 0 and vv.launch_count() - n0 == 1
    got_q = dq.cpu().numpy()
    assert orc.rope_error_in_ulps(got_q, want_q, qb).max() <= ROPE_ULP
    got_kc = dkc.cpu().numpy()
    err_k = orc.rope_error_in_ulps(got_kc[cache_off:cache_off + rows].reshape(k.shape), want_k, kb)
    assert err_k.max() <= ROPE_ULP
    # V is a bit copy (after the exact bias sum); untouched cache rows keep their bytes
    assert np.array_equal(bits(dvc), want_vc.view(np.uint16))
    keep = np.ones(max_len, bool)
    keep[cache_off:cache_off + rows] = False
    assert np.array_equal(got_kc.view(np.uint16)[keep], kc0.view(np.uint16)[keep])
    assert np.array_equal(bits(dv_), v.view(np.uint16))                       # V source untouched
    if keep_k:
        assert np.array_equal(bits(dk).reshape(rows, -1), got_kc.view(np.uint16)[cache_off:cache_off + rows])
    else:
        assert np.array_equal(bits(dk), k.view(np.uint16))                    # K source untouched

    # ---- this library's separate ops + device copies give the same bytes
    sq, sk, sv = dev(q), dev(k), dev(v)
    if with_bias:
        assert vv.vv_bias_add_dev(sq, dev(bq), rows, nq * hd) == 0
        assert vv.vv_bias_add_dev(sk, dev(bk), rows, nkv * hd) == 0
        assert vv.vv_bias_add_dev(sv, dev(bv), rows, nkv * hd) == 0
    assert vv.vv_rope_dev(sq, rows, nq, hd, pos, None, 1e6) == 0
    assert vv.vv_rope_dev(sk, rows, nkv, hd, pos, None, 1e6) == 0
    assert np.array_equal(bits(sq), got_q.view(np.uint16))
    assert np.array_equal(bits(sk).reshape(rows, -1), got_kc.view(np.uint16)[cache_off:cache_off + rows])


def test_rope_append_device_position_and_graph_replay(vv, orc):
    """Decode: the device int gives both the RoPE position and the cache row,
    and a captured launch follows it on replay."""
    nq, nkv, hd, max_len = 28, 4, 128, 64
    rng = np.random.default_rng(2)
    q, k, v = (rng.standard_normal((1, n, hd)).astype(np.float16) for n in (nq, nkv, nkv))
    dq, dk, dv_ = dev(q), dev(k), dev(v)
    src_q = dq.clone()
    kc = torch.zeros(max_len, nkv * hd, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    dpos = torch.tensor([3], dtype=torch.int32, device="cuda")
    s = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            dq.copy_(src_q)
            assert vv.vvb_rope_qk_append_dev(dq, dk, dv_, None, None, None, kc, vc, 1, nq, nkv, hd, 0, 0, dpos,
                                             1e6, 0, stream=s) == 0
    for p in (3, 41):
        dpos.fill_(p)
        g.replay()
        torch.cuda.synchronize()
        assert orc.rope_error_in_ulps(dq.cpu().numpy(), orc.rope_f16(q, p, 1e6), q).max() <= ROPE_ULP
        want_k = orc.rope_f16(k, p, 1e6).reshape(-1)
        assert orc.rope_error_in_ulps(kc[p].cpu().numpy().reshape(1, nkv, hd), want_k.reshape(1, nkv, hd), k).max() <= ROPE_ULP
        assert np.array_equal(bits(vc[p]), v.reshape(-1).view(np.uint16))
    written = (kc.abs().sum(dim=1) > 0).nonzero().flatten().tolist()
    assert written == [3, 41]


def test_rope_append_argument_checks(vv):
    x = torch.zeros(4, 2, 128, dtype=torch.float16, device="cuda")
    c = torch.zeros(8, 256, dtype=torch.float16, device="cuda")
    assert vv.vvb_rope_qk_append_dev(None, x, x, None, None, None, c, c, 4, 2, 2, 128, 0, 0, None, 1e6) == vv.VV_ERR_NULL_PTR
    assert vv.vvb_rope_qk_append_dev(x, x, x, None, None, None, None, c, 4, 2, 2, 128, 0, 0, None, 1e6) == vv.VV_ERR_NULL_PTR
    assert vv.vvb_rope_qk_append_dev(x, x, x, None, None, None, c, c, -1, 2, 2, 128, 0, 0, None, 1e6) == vv.VV_ERR_INVALID_ARG
    assert vv.vvb_rope_qk_append_dev(x, x, x, None, None, None, c, c, 4, 2, 2, 128, 0, -2, None, 1e6) == vv.VV_ERR_INVALID_ARG
    assert vv.vvb_rope_qk_append_dev(x, x, x, None, None, None, c, c, 4, 2, 2, 24, 0, 0, None, 1e6) == vv.VV_ERR_UNSUPPORTED
    assert vv.vvb_rope_qk_append_dev(x, x, x, None, None, None, c, c, 0, 2, 2, 128, 0, 0, None, 1e6) == vv.VV_OK
