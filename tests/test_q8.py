"""Per-token int8 activation quantizers: the oracle against the reference's
golden vectors (CPU), and the CUDA kernels against the oracle (GPU, bit-exact:
the outputs are integers and a correctly rounded scale)."""
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LAYOUTS = [0, 1, 2, 3]


@pytest.fixture(scope="module")
def q8gold():
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "q8_golden.npz")))


# ------------------------------------------------------------------ CPU: pin the oracle
@pytest.mark.parametrize("K", [1536, 3584])
@pytest.mark.parametrize("layout", LAYOUTS)
def test_oracle_quantizer_matches_reference_golden(orc, q8gold, K, layout):
    x = q8gold[f"x_{K}"].astype(np.float32)
    xq, sx, xsum = orc.restated().quant_act_q8(x, layout)
    assert np.array_equal(xq, q8gold[f"xq_{K}_{layout}"])
    assert np.array_equal(sx.view(np.uint32), q8gold[f"sx_{K}_{layout}"].view(np.uint32))
    assert np.array_equal(xsum, q8gold[f"xsum_{K}_{layout}"])


def test_oracle_q8_layouts_are_permutations_with_equal_sums(orc):
    """include/vibevoice/q8.h:1-11: every layout is a permutation of each run
    of 32 columns and the per-run sums are layout-independent."""
    pos = [[orc.restated().lib.orc_q8_pos(l, j) for j in range(32)] for l in LAYOUTS]
    for p in pos:
        assert sorted(p) == list(range(32))
    assert pos[1][:4] == [0, 16, 1, 17]                      # evens first, then odds
    rng = np.random.default_rng(3)
    x = rng.standard_normal((3, 256)).astype(np.float16).astype(np.float32)
    base = orc.restated().quant_act_q8(x, 0)
    for l in LAYOUTS[1:]:
        xq, sx, xsum = orc.restated().quant_act_q8(x, l)
        assert np.array_equal(xsum, base[2]) and np.array_equal(sx, base[1])
        runs, nat = xq.reshape(3, -1, 32), base[0].reshape(3, -1, 32)
        assert np.array_equal(runs[:, :, pos[l]], nat)
    assert np.abs(base[0]).max() == 127


def test_oracle_quantizer_live_against_reference(orc):
    if not orc.have_reference_int8():
        pytest.skip("compiled reference quantizer not present")
    rng = np.random.default_rng(4)
    for M, K in ((1, 1536), (7, 3584), (285, 8960), (3, 18944)):
        x = (rng.standard_normal((M, K)) * 3).astype(np.float16).astype(np.float32)
        for l in LAYOUTS:
            a, b = orc.restated().quant_act_q8(x, l), orc.reference_int8().quant_act_q8(x, l)
            assert all(np.array_equal(p, q) for p, q in zip(a, b))


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


def alloc_q(M, K):
    """Outputs with canary bands: int8 rows, scales, run sums."""
    pad = 256
    xq = torch.full((M * K + 2 * pad,), 0x5A, dtype=torch.int8, device="cuda")
    sx = torch.full((M + 2 * pad,), 7.5, dtype=torch.float32, device="cuda")
    xs = torch.full((M * (K // 32) + 2 * pad,), 123456, dtype=torch.int32, device="cuda")
    return pad, xq, sx, xs


def fetch_q(pad, xq, sx, xs, M, K):
    torch.cuda.synchronize()
    a, b, c = xq.cpu().numpy(), sx.cpu().numpy(), xs.cpu().numpy()
    for arr, fill in ((a, 0x5A), (b, 7.5), (c, 123456)):
        assert (arr[:pad] == fill).all() and (arr[-pad:] == fill).all(), "canary overwritten"
    return a[pad:-pad].reshape(M, K), b[pad:-pad], c[pad:-pad].reshape(M, K // 32)


def run_q(fn, M, K, with_xsum=True):
    pad, xq, sx, xs = alloc_q(M, K)
    st = fn(xq.data_ptr() + pad, sx.data_ptr() + 4 * pad, (xs.data_ptr() + 4 * pad) if with_xsum else None)
    assert st == 0, st
    return fetch_q(pad, xq, sx, xs, M, K)


def same(a, b):
    return (np.array_equal(a[0], b[0]) and np.array_equal(a[1].view(np.uint32), b[1].view(np.uint32))
            and (a[2] is None or b[2] is None or np.array_equal(a[2], b[2])))


@gpu
@pytest.mark.parametrize("K", [1536, 3584])
@pytest.mark.parametrize("layout", LAYOUTS)
def test_act_quant_golden(vv, q8gold, K, layout):
    x = q8gold[f"x_{K}"]
    got = run_q(lambda q, s, u: vv.vv_act_quant_dev(dev(x), x.shape[0], K, layout, q, s, u), x.shape[0], K)
    assert same(got, (q8gold[f"xq_{K}_{layout}"], q8gold[f"sx_{K}_{layout}"], q8gold[f"xsum_{K}_{layout}"]))


@gpu
@pytest.mark.parametrize("M,K", [(m, k) for m in (1, 7, 285) for k in (1536, 3584, 8960, 18944)] +
                         # deep grids (more rows than one wave): the two-warps-per-row instances for every
                         # width they serve, and widths either side of them that take the general shape
                         [(700, k) for k in (1024, 1536, 2048, 2560, 3072, 3584, 4096, 4608, 3616, 18944)])
def test_q8_kernels_equal_oracle_and_unfused(vv, orc, M, K):
    """The shapes of tests/test_int8_linear.c:295-354. Each fused quantizer is
    bit-identical (a) to the CPU quantizer applied to the FP16 values the
    unfused op writes and (b) to the unfused op followed by vv_act_quant_dev."""
    rng = np.random.default_rng(M * 100 + K)
    x = (rng.standard_normal((M, K)) * 2).astype(np.float16)
    d = rng.standard_normal((M, K)).astype(np.float16)
    w = (1 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    up = rng.standard_normal((M, K)).astype(np.float16)
    R = orc.restated()
    for layout in LAYOUTS:
        # plain
        got = run_q(lambda q, s, u: vv.vv_act_quant_dev(dev(x), M, K, layout, q, s, u), M, K)
        assert same(got, R.quant_act_q8(x.astype(np.float32), layout))
        # RMSNorm + quantize: against the oracle's norm (bit-exact on the GPU) and the unfused pair
        got = run_q(lambda q, s, u: vv.vv_rmsnorm_q8_dev(dev(x), dev(w), M, K, 1e-6, layout, q, s, u), M, K)
        _, normed = orc.add_rmsnorm_f16(x, None, w, 1e-6)
        assert same(got, R.quant_act_q8(normed.astype(np.float32), layout))
        y = torch.empty(M, K, dtype=torch.float16, device="cuda")
        assert vv.vv_rmsnorm_dev(dev(x), dev(w), y, M, K, 1e-6) == 0
        assert same(got, run_q(lambda q, s, u: vv.vv_act_quant_dev(y, M, K, layout, q, s, u), M, K))
        # SwiGLU + quantize: the unfused op's own FP16 values, then the CPU quantizer
        got = run_q(lambda q, s, u: vv.vv_swiglu_q8_dev(dev(x), dev(up), M, K, layout, q, s, u), M, K)
        o = torch.empty(M, K, dtype=torch.float16, device="cuda")
        assert vv.vv_swiglu_dev(dev(x), dev(up), o, M * K) == 0
        torch.cuda.synchronize()
        assert same(got, R.quant_act_q8(o.cpu().numpy().astype(np.float32), layout))
        assert same(got, run_q(lambda q, s, u: vv.vv_act_quant_dev(o, M, K, layout, q, s, u), M, K))
    # residual add + norm + quantize, and without the run sums
    h = dev(x)
    got = run_q(lambda q, s, u: vv.vvb_add_rmsnorm_q8_dev(h, dev(d), dev(w), M, K, 1e-6, 0, q, s, u), M, K, False)
    hn, normed = orc.add_rmsnorm_f16(x, d, w, 1e-6)
    torch.cuda.synchronize()
    assert np.array_equal(h.cpu().numpy().view(np.uint16), hn.view(np.uint16))
    want = R.quant_act_q8(normed.astype(np.float32), 0)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
    assert (got[2] == 123456).all()                      # xsum == NULL: never written


@gpu
@pytest.mark.parametrize("M,K", [(1, 3584), (285, 3584), (1000, 18944), (37, 1536), (5, 250), (70, 7)])
def test_col_absmax(vv, M, K):
    """acc[k] = max(acc[k], max_m |x[m,k]|) (tests/test_int8_linear.c:370-395
    checks it against a host loop): exact, and it accumulates over calls."""
    rng = np.random.default_rng(M + K)
    x1 = (rng.standard_normal((M, K)) * 3).astype(np.float16)
    x2 = (rng.standard_normal((M, K)) * 3).astype(np.float16)
    acc = torch.zeros(K + 64, dtype=torch.float32, device="cuda")
    acc[K:] = -5.0                                               # canary: never touched
    assert vv.vv_col_absmax_dev(dev(x1), M, K, acc) == 0
    torch.cuda.synchronize()
    want1 = np.abs(x1.astype(np.float32)).max(axis=0)
    assert np.array_equal(acc[:K].cpu().numpy(), want1)
    assert vv.vv_col_absmax_dev(dev(x2), M, K, acc) == 0
    torch.cuda.synchronize()
    assert np.array_equal(acc[:K].cpu().numpy(), np.maximum(want1, np.abs(x2.astype(np.float32)).max(axis=0)))
    assert (acc[K:].cpu().numpy() == -5.0).all()
    assert vv.vv_col_absmax_dev(None, M, K, acc) == vv.VV_ERR_NULL_PTR
    assert vv.vv_col_absmax_dev(dev(x1), 0, K, acc) == vv.VV_ERR_INVALID_ARG


@gpu
def test_q8_argument_checks(vv):
    """src/cuda/act_quant.cu:222-233: NULL -> NULL_PTR, M or K <= 0 ->
    INVALID_ARG, K % 32 != 0 or K > 22528 -> UNSUPPORTED, bad layout ->
    INVALID_ARG, RMSNorm rows narrower than 256 -> UNSUPPORTED."""
    x = torch.zeros(4, 512, dtype=torch.float16, device="cuda")
    q = torch.zeros(4, 512, dtype=torch.int8, device="cuda")
    s = torch.zeros(4, dtype=torch.float32, device="cuda")
    assert vv.vv_act_quant_dev(None, 4, 512, 0, q, s, None) == vv.VV_ERR_NULL_PTR
    assert vv.vv_act_quant_dev(x, 4, 512, 0, None, s, None) == vv.VV_ERR_NULL_PTR
    assert vv.vv_act_quant_dev(x, 0, 512, 0, q, s, None) == vv.VV_ERR_INVALID_ARG
    assert vv.vv_act_quant_dev(x, 4, 500, 0, q, s, None) == vv.VV_ERR_UNSUPPORTED
    assert vv.vv_act_quant_dev(x, 4, 22560, 0, q, s, None) == vv.VV_ERR_UNSUPPORTED
    assert vv.vv_act_quant_dev(x, 4, 512, 4, q, s, None) == vv.VV_ERR_INVALID_ARG
    assert vv.vv_rmsnorm_q8_dev(x, None, 4, 512, 1e-6, 0, q, s, None) == vv.VV_ERR_NULL_PTR
    assert vv.vv_rmsnorm_q8_dev(x, x, 4, 128, 1e-6, 0, q, s, None) == vv.VV_ERR_UNSUPPORTED
    assert vv.vv_swiglu_q8_dev(x, None, 4, 512, 0, q, s, None) == vv.VV_ERR_NULL_PTR
    assert vv.vv_act_quant_dev(x, 4, 512, 0, q, s, None) == vv.VV_OK
