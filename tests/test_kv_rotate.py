"""vvb_kv_rotate_dev / vvb_kv_unrotate_dev: the randomized Hadamard rotation the
reference applies to Q before, and undoes on the attention output after,
attention over a TurboQuant cache (src/inference/decoder.c:878-901,
src/cuda/kv_quant.cu:173-200,473-494). CPU: the oracle's restatement against
the definition (the signed Sylvester-Hadamard matrix in float64) and against
golden bytes of the reference's kernel. GPU: this library's kernels against the
oracle and against the live reference kernel, byte for byte."""
import ctypes as C
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden", "kv_rotate_golden.npz")
REF_CUDA = os.path.join(ROOT, "oracle", "_ref", "libvvref_cuda.so")


def signed_hadamard(orc):
    """M with rotate(x) = M x: H_128 / sqrt(128) times diag(sign)."""
    R = orc.restated()
    R.lib.orc_kv_sign.restype = C.c_float
    R.lib.orc_kv_sign.argtypes = [C.c_int]
    s = np.array([R.lib.orc_kv_sign(d) for d in range(128)], np.float64)
    i = np.arange(128)
    H = (-1.0) ** np.array([[bin(a & b).count("1") for b in i] for a in i])
    return H / np.sqrt(128.0) * s[None, :], s


# ------------------------------------------------------------------ CPU
def test_oracle_rotation_is_the_signed_hadamard_matrix(orc):
    R = orc.restated()
    M, _ = signed_hadamard(orc)
    assert np.allclose(M @ M.T, np.eye(128), atol=1e-12)              # orthonormal
    rng = np.random.default_rng(2)
    x = rng.standard_normal((64, 128)).astype(np.float16)
    want = x.astype(np.float64) @ M.T
    got = R.kv_rotate_f16(x).astype(np.float64)
    # float accumulation over seven butterfly stages, then one FP16 rounding
    assert np.abs(got - want).max() <= 2.0 ** -11 * np.abs(want).max() + 1e-6
    back = R.kv_rotate_f16(x, inverse=True).astype(np.float64)
    assert np.abs(back - x.astype(np.float64) @ M).max() <= 2.0 ** -11 * np.abs(want).max() + 1e-6


def test_oracle_unrotate_undoes_rotate_within_fp16_rounding(orc):
    R = orc.restated()
    rng = np.random.default_rng(3)
    x = (rng.standard_normal((200, 128)) * 2.0).astype(np.float16)
    y = R.kv_rotate_f16(x)
    z = R.kv_rotate_f16(y, inverse=True).astype(np.float32)
    assert np.abs(z - x.astype(np.float32)).max() <= 6e-3             # two FP16 roundings at scale ~8
    n0, n1 = np.linalg.norm(x.astype(np.float64), axis=1), np.linalg.norm(y.astype(np.float64), axis=1)
    assert np.allclose(n0, n1, rtol=2e-3)
    # one spike becomes a flat vector of magnitude spike / sqrt(128)
    e = np.zeros((1, 128), np.float16)
    e[0, 40] = 32.0
    assert np.allclose(np.abs(R.kv_rotate_f16(e).astype(np.float32)), 32.0 / np.sqrt(128.0), rtol=1e-3)


def test_oracle_rotation_matches_golden_bytes_of_the_reference_kernel(orc):
    if not os.path.exists(GOLD):
        pytest.skip("tests/golden/kv_rotate_golden.npz not generated yet (tests/golden/make_golden_rotate.py, needs a GPU)")
    g = dict(np.load(GOLD))
    R = orc.restated()
    x = g["x"].view(np.float16)
    for key, inverse in (("rotated", False), ("unrotated", True)):
        got = R.kv_rotate_f16(x, inverse=inverse).view(np.uint16)
        want = g[key]
        nan = np.isnan(want.view(np.float16))
        assert np.array_equal(np.isnan(got.view(np.float16)), nan), key
        assert np.array_equal(got[~nan], want[~nan]), key


# ------------------------------------------------------------------ GPU
try:
    import torch
except ImportError:                      # pragma: no cover
    torch = None
gpu = pytest.mark.gpu


@pytest.fixture(scope="module")
def vv():
    if torch is None or not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import vvb200
    torch.cuda.set_device(0)
    return vvb200


@pytest.fixture(scope="module")
def refk():
    if not os.path.exists(REF_CUDA):
        pytest.skip("the reference's CUDA kernels were not compiled")
    ref = C.CDLL(REF_CUDA)
    for name in ("vv_kv_rotate_dev", "vv_kv_unrotate_dev"):
        getattr(ref, name).argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        getattr(ref, name).restype = C.c_int
    return ref


def stress_input(rows, heads, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((rows, heads, 128)).astype(np.float16)
    if rows > 8:
        x[1, :, 17] = 40.0
        x[2] *= np.float16(1e-3)
        x[3, 0] = 0
        x[4, -1] = 65504.0
        x[5, 0] = 6e-8
        x[6, 0, 9] = np.inf
        x[7, -1, 100] = np.nan
    return x


def same_bits(a, b):
    """Equal FP16 bit patterns; a NaN may differ in payload."""
    na, nb = np.isnan(a), np.isnan(b)
    return np.array_equal(na, nb) and np.array_equal(a.view(np.uint16)[~na], b.view(np.uint16)[~nb])


@gpu
@pytest.mark.parametrize("rows,heads", [(1, 28), (300, 28), (2048, 4), (7, 3), (33, 1), (611, 1), (171, 3), (4099, 28)])
@pytest.mark.parametrize("inverse", [False, True])
def test_rotate_equals_oracle_and_the_live_reference_kernel(vv, refk, orc, rows, heads, inverse):
    x = stress_input(rows, heads, rows * 3 + heads)
    ours = torch.from_numpy(x.copy()).cuda()
    theirs = torch.from_numpy(x.copy()).cuda()
    n0 = vv.launch_count()
    fn = vv.vvb_kv_unrotate_dev if inverse else vv.vvb_kv_rotate_dev
    assert fn(ours, heads, 128, rows) == 0
    assert vv.launch_count() - n0 == 1
    rfn = refk.vv_kv_unrotate_dev if inverse else refk.vv_kv_rotate_dev
    assert rfn(theirs.data_ptr(), heads, 128, rows, None) == 0
    torch.cuda.synchronize()
    got, ref_out = ours.cpu().numpy(), theirs.cpu().numpy()
    assert same_bits(got, ref_out), "against the reference's kernel"
    if rows <= 2048:
        assert same_bits(got, orc.restated().kv_rotate_f16(x, inverse=inverse)), "against the oracle"


@gpu
def test_rotate_on_a_pointer_that_is_only_two_byte_aligned(vv, orc):
    rows, heads = 19, 5
    x = stress_input(rows, heads, 77)
    buf = torch.zeros(rows * heads * 128 + 8, dtype=torch.float16, device="cuda")
    buf[0], buf[-7:] = 123.0, 321.0                       # guard values around the view
    view = buf[1:1 + rows * heads * 128]
    view.copy_(torch.from_numpy(x.reshape(-1)))
    assert view.data_ptr() % 8 == 2
    assert vv.vvb_kv_rotate_dev(view, heads, 128, rows) == 0
    torch.cuda.synchronize()
    assert same_bits(view.cpu().numpy().reshape(x.shape), orc.restated().kv_rotate_f16(x))
    assert float(buf[0]) == 123.0 and bool((buf[-7:] == 321.0).all())


@gpu
def test_rotate_then_unrotate_under_graph_replay(vv, orc):
    """Both directions captured in one graph (as the reference's decode step holds them around its
    attention call) and replayed over fresh data."""
    rows, heads = 1, 28
    d = torch.zeros(rows, heads, 128, dtype=torch.float16, device="cuda")
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        assert vv.vvb_kv_rotate_dev(d, heads, 128, rows, s) == 0
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            assert vv.vvb_kv_rotate_dev(d, heads, 128, rows, s) == 0
            assert vv.vvb_kv_unrotate_dev(d, heads, 128, rows, s) == 0
        for seed in (1, 2, 3):
            x = stress_input(rows, heads, seed)
            d.copy_(torch.from_numpy(x))
            g.replay()
            torch.cuda.synchronize()
            R = orc.restated()
            want = R.kv_rotate_f16(R.kv_rotate_f16(x), inverse=True)
            assert same_bits(d.cpu().numpy(), want)


@gpu
def test_rotate_argument_checks(vv):
    x = torch.zeros(4, 2, 128, dtype=torch.float16, device="cuda")
    x64 = torch.zeros(4, 2, 64, dtype=torch.float16, device="cuda")
    for fn in (vv.vvb_kv_rotate_dev, vv.vvb_kv_unrotate_dev):
        assert fn(None, 2, 128, 4) == vv.VV_ERR_NULL_PTR
        assert fn(x64, 2, 64, 4) == vv.VV_ERR_UNSUPPORTED          # as the reference: head_dim 128 only
        assert fn(x, 2, 128, -1) == vv.VV_ERR_INVALID_ARG
        assert fn(x, -2, 128, 4) == vv.VV_ERR_INVALID_ARG
        n0 = vv.launch_count()
        assert fn(x, 2, 128, 0) == 0 and fn(x, 0, 128, 4) == 0     # empty work: VV_OK, nothing launched
        assert vv.launch_count() == n0
    assert not x.any()
