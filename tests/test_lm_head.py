"""LM head: logits = W @ x, greedy argmax, and the fused final-norm + head +
argmax. Floating-point dot products, so the bar is a tolerance: an FP32
accumulation over K terms must sit within TOL(K) of the double-precision
oracle, and the token must equal the oracle's whenever the winner's margin over
the runner-up exceeds twice that tolerance."""
import numpy as np
import pytest


def tol(x, w, depth=128):
    """Per-row bound on |fp32 dot - exact dot|: depth * 2^-24 * sum|x_k w_k|,
    the worst case of a summation whose longest chain is `depth` additions
    (the kernel: 112 sequential FMAs per lane + a 5-level shuffle tree for
    K = 3584; the reference's AVX2 loop: 448 + 3, so it is checked at 512)."""
    return depth * 2.0 ** -24 * (np.abs(w.astype(np.float64)) @ np.abs(x.astype(np.float64)))


def make_case(rng, V, K, planted=None):
    x = rng.standard_normal(K).astype(np.float16)
    w = (0.02 * rng.standard_normal((V, K))).astype(np.float16)
    if planted is not None:                         # a clear winner: a row aligned with x
        w[planted] = (0.05 * np.sign(x.astype(np.float32))).astype(np.float16)
    return x, w


# ------------------------------------------------------------------ CPU: pin the oracle
def test_oracle_lm_head_against_numpy_and_reference(orc):
    rng = np.random.default_rng(0)
    for V, K, planted in ((1000, 3584, 77), (333, 256, None), (5, 8, 4)):
        x, w = make_case(rng, V, K, planted)
        logits, tok, val = orc.restated().lm_head(x.astype(np.float32), w)
        want = w.astype(np.float64) @ x.astype(np.float64)
        assert np.allclose(logits, want, rtol=1e-12, atol=1e-12)
        assert tok == int(np.argmax(want)) and val == logits[tok]
        if planted is not None:
            assert tok == planted
        if orc.have_reference():
            rtok, rval = orc.reference().lm_head_argmax(x.astype(np.float32), w)   # the reference's FP32 path
            margin = np.sort(want)[-1] - np.sort(want)[-2]
            t = tol(x, w, 512)
            if margin > 2 * t.max():
                assert rtok == tok
            assert abs(rval - want[rtok]) <= t[rtok]


# ------------------------------------------------------------------ GPU
torch = pytest.importorskip("torch")
gpu = pytest.mark.gpu


@pytest.fixture(scope="module")
def vv():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import vvb200
    torch.cuda.set_device(0)
    return vvb200


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@gpu
@pytest.mark.parametrize("V,K,planted", [(152064, 3584, 151000), (4097, 3584, None), (1000, 1536, 3), (37, 256, 36),
                                         (64, 8, None), (50, 250, 7), (9, 12000, 2)])
def test_lm_head_gemv_and_argmax(vv, orc, V, K, planted):
    rng = np.random.default_rng(V + K)
    x, w = make_case(rng, V, K, planted)
    want, wtok, _ = orc.restated().lm_head(x.astype(np.float32), w)
    t = tol(x, w, max(128, K // 32 + 16))          # the scalar path chains K/32 additions per lane
    logits = torch.full((V + 64,), 7.0, dtype=torch.float32, device="cuda")        # canary tail
    dx, dw = dev(x), dev(w)
    assert vv.vv_lm_head_gemv_dev(dx, dw, logits, V, K) == 0
    torch.cuda.synchronize()
    got = logits.cpu().numpy()
    assert (got[V:] == 7.0).all()
    assert (np.abs(got[:V] - want) <= t).all()
    # stand-alone two-stage argmax over those logits (caller scratch of 256 + 256)
    sv = torch.empty(256, dtype=torch.float32, device="cuda")
    si = torch.empty(256, dtype=torch.int32, device="cuda")
    tok = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    val = torch.zeros(1, dtype=torch.float32, device="cuda")
    assert vv.vv_argmax_dev(logits, V, sv, si, tok, val) == 0
    torch.cuda.synchronize()
    assert int(tok.item()) == int(np.argmax(got[:V])) and float(val.item()) == got[:V].max()
    srt = np.sort(want)
    clear = V == 1 or (srt[-1] - srt[-2]) > 2 * t.max()
    if clear:
        assert int(tok.item()) == wtok
    assert vv.vv_argmax_dev(logits, V, sv, si, tok, None) == 0                      # out_value may be NULL


@gpu
@pytest.mark.parametrize("V,K,planted,with_logits", [(152064, 3584, 99999, True), (152064, 3584, 5, False),
                                                     (1000, 1536, 999, True), (33, 256, 0, True)])
def test_fused_final_norm_lm_head_argmax(vv, orc, V, K, planted, with_logits):
    """One GEMV launch (final RMSNorm inside) + one reduce == rmsnorm, gemv,
    argmax of the separate ops, and the oracle's token."""
    rng = np.random.default_rng(V * 3 + K)
    h = (rng.standard_normal(K) * 3).astype(np.float16)
    gamma = (1 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    _, normed = orc.add_rmsnorm_f16(h[None, :], None, gamma, 1e-6)
    x = normed[0]
    w = (0.02 * rng.standard_normal((V, K))).astype(np.float16)
    w[planted] = (0.05 * np.sign(x.astype(np.float32))).astype(np.float16)
    want, wtok, _ = orc.restated().lm_head(x.astype(np.float32), w)
    assert wtok == planted
    nbytes = vv.vvb_lm_head_scratch_bytes(V)
    assert nbytes == 8 * ((V + 31) // 32)
    scratch = torch.full((nbytes + 64,), 0x5A, dtype=torch.uint8, device="cuda")     # garbage in, canary tail
    logits = torch.zeros(V, dtype=torch.float32, device="cuda") if with_logits else None
    tok = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    val = torch.zeros(1, dtype=torch.float32, device="cuda")
    dw = dev(w)
    n0 = vv.launch_count()
    assert vv.vvb_lm_head_argmax_dev(dev(h), dev(gamma), 1e-6, dw, V, K, logits, scratch, nbytes, tok, val) == 0
    assert vv.launch_count() - n0 == 2
    torch.cuda.synchronize()
    assert int(tok.item()) == planted
    assert abs(float(val.item()) - want[planted]) <= tol(x, w)[planted]
    assert (scratch[nbytes:].cpu().numpy() == 0x5A).all()
    if with_logits:
        # the separate ops give the same bits (same device code for the norm, same dot order)
        nx = torch.empty(K, dtype=torch.float16, device="cuda")
        lg = torch.empty(V, dtype=torch.float32, device="cuda")
        assert vv.vv_rmsnorm_dev(dev(h), dev(gamma), nx, 1, K, 1e-6) == 0
        assert vv.vv_lm_head_gemv_dev(nx, dw, lg, V, K) == 0
        torch.cuda.synchronize()
        assert np.array_equal(nx.cpu().numpy().view(np.uint16), x.view(np.uint16))
        assert torch.equal(lg, logits)
    # already-normalised input (final_norm_w == NULL) agrees too
    tok2 = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    assert vv.vvb_lm_head_argmax_dev(dev(x), None, 0.0, dw, V, K, None, scratch, nbytes, tok2, None) == 0
    torch.cuda.synchronize()
    assert int(tok2.item()) == planted


@gpu
def test_argmax_ties_and_edges(vv):
    sv = torch.empty(256, dtype=torch.float32, device="cuda")
    si = torch.empty(256, dtype=torch.int32, device="cuda")
    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    lg = torch.zeros(100000, dtype=torch.float32, device="cuda")
    lg[[70000, 512, 99999]] = 5.0                                  # a three-way tie: the smallest index wins
    assert vv.vv_argmax_dev(lg, 100000, sv, si, tok, None) == 0
    torch.cuda.synchronize()
    assert int(tok.item()) == 512
    one = torch.tensor([-3.0], device="cuda")
    assert vv.vv_argmax_dev(one, 1, sv, si, tok, None) == 0
    torch.cuda.synchronize()
    assert int(tok.item()) == 0
    assert vv.vv_argmax_dev(None, 1, sv, si, tok, None) == vv.VV_ERR_NULL_PTR
    assert vv.vv_argmax_dev(lg, 10, None, si, tok, None) == vv.VV_ERR_NULL_PTR
    assert vv.vv_lm_head_gemv_dev(None, lg, lg, 4, 8) == vv.VV_ERR_NULL_PTR
    x = torch.zeros(8, dtype=torch.float16, device="cuda")
    assert vv.vvb_lm_head_argmax_dev(x, None, 0.0, x, 1, 8, None, sv, 4, tok, None) == vv.VV_ERR_INVALID_ARG  # scratch too small
    assert vv.vvb_lm_head_argmax_dev(x, None, 0.0, x, 1, 12, None, sv, 1024, tok, None) == vv.VV_ERR_UNSUPPORTED
