"""TurboQuant KV-cache formats (4, 3, 2 and 1.5 bits per value): the oracle's
restatement of the reference's store kernel (src/cuda/kv_quant.cu:40-121,
src/cuda/kv_codec.cuh), checked on the CPU by the properties the format
promises, pinned to bytes the reference's own kernel produced on a B200
(tests/golden/tq_kv_golden.npz, written by tests/golden/make_golden_tq.py),
and, on a GPU, the fused bias + RoPE + TurboQuant append against the live
reference kernel and the oracle.

The reference has no CPU code for these formats and its CUDA build is
fast-math (approximate square root and reciprocal), so oracle and device agree
except when a scaled value lands within a few float ulps of a decision
threshold or sigma within as much of a FP16 rounding boundary: comparisons
with the oracle allow a stated handful of such elements; comparisons with the
live reference kernel are exact.
"""
import ctypes as C
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden", "tq_kv_golden.npz")
REF_CUDA = os.path.join(ROOT, "oracle", "_ref", "libvvref_cuda.so")
FMTS = [(3, "tq4", 64), (4, "tq3", 48), (5, "tq2", 32), (6, "tq1_5", 24)]
# signal-to-quantization-noise of a unit Gaussian per format, as the reference's header states it
# (src/cuda/kv_codec.cuh:44): 20.2, 14.6, 9.3, 7.0 dB
SQNR_DB = {3: 20.2, 4: 14.6, 5: 9.3, 6: 7.0}
NQ, NKV, HD = 28, 4, 128


# ------------------------------------------------------------------ CPU: the oracle's properties
def test_rotation_is_orthonormal_and_spreads_an_outlier(orc):
    R = orc.restated()
    rng = np.random.default_rng(1)
    x = rng.standard_normal((50, 128)).astype(np.float32)
    y = R.tq_rotate(x)
    assert np.allclose(np.linalg.norm(y, axis=1), np.linalg.norm(x, axis=1), rtol=1e-5)
    assert np.allclose(y @ y.T, x @ x.T, atol=2e-4)                 # dot products survive: dot(Hq, Hk) == dot(q, k)
    spike = np.zeros((1, 128), np.float32)
    spike[0, 77] = 16.0
    assert np.allclose(np.abs(R.tq_rotate(spike)), 16.0 / np.sqrt(128), rtol=1e-6)   # an outlier channel becomes flat


@pytest.mark.parametrize("fmt,name,bpv", FMTS)
def test_oracle_store_round_trip_reaches_the_formats_sqnr(orc, fmt, name, bpv):
    R = orc.restated()
    assert R.tq_bytes_per_vec(fmt) == bpv
    rng = np.random.default_rng(fmt)
    x = (rng.standard_normal((64, 4, 128)) * 1.7).astype(np.float16)
    store, meta = R.kv_store_tq(x, None, fmt)
    assert store.shape == (64, 4 * bpv) and meta.shape == (64, 4)
    rot = R.tq_rotate(x.astype(np.float32))
    sig = np.sqrt((rot.astype(np.float64) ** 2).mean(axis=-1))
    assert np.allclose(meta.astype(np.float64), sig, rtol=2e-3)      # sigma is the vector's RMS, kept as FP16
    noise = signal = 0.0
    for p in range(64):
        for h in range(4):
            back = R.kv_load_tq(store[p, h * bpv:(h + 1) * bpv], meta[p, h], fmt)
            noise += float(((back - rot[p, h]) ** 2).sum())
            signal += float((rot[p, h] ** 2).sum())
    sqnr = 10 * np.log10(signal / noise)
    assert abs(sqnr - SQNR_DB[fmt]) < 0.6, sqnr


@pytest.mark.parametrize("fmt,name,bpv", FMTS)
def test_oracle_bit_layout_and_reference_key(orc, fmt, name, bpv):
    """Lane L of 32 owns values 4L..4L+3 and bits [nb*L, nb*(L+1)) of the vector; a
    reference key is subtracted in float before the rotation; rows land at first_row."""
    R = orc.restated()
    nb = bpv * 8 // 32
    rng = np.random.default_rng(10 + fmt)
    x = rng.standard_normal((3, 2, 128)).astype(np.float16)
    ref = rng.standard_normal((2, 128)).astype(np.float16)
    store, meta = R.kv_store_tq(x, ref, fmt, first_row=5)
    assert not store[:5].any() and not meta[:5].view(np.uint16).any()
    diff = (x.astype(np.float32) - ref.astype(np.float32)[None]).astype(np.float32)
    # the same vectors fed as plain inputs: only valid where the difference is a half again
    exact = diff.astype(np.float16).astype(np.float32) == diff
    if exact.all():
        s2, m2 = R.kv_store_tq(diff.astype(np.float16), None, fmt)
        assert np.array_equal(s2, store[5:]) and np.array_equal(m2.view(np.uint16), meta[5:].view(np.uint16))
    # decode by hand from the bit layout and compare with the oracle's loader
    vec = store[6, bpv:2 * bpv]
    bits = np.unpackbits(vec, bitorder="little")
    back = R.kv_load_tq(vec, meta[6, 1], fmt)
    sigma = float(meta[6, 1])
    lev = {3: [-2.725112, -2.065280, -1.613787, -1.251845, -0.938657, -0.654379, -0.386970, -0.127960,
               0.127960, 0.386970, 0.654379, 0.938657, 1.251845, 1.613787, 2.065280, 2.725112],
           4: [-2.150300, -1.343258, -0.755588, -0.244756, 0.244756, 0.755588, 1.343258, 2.150300],
           5: [-1.511418, -0.452456, 0.452456, 1.511418]}
    for lane in (0, 7, 31):
        mine = bits[nb * lane: nb * (lane + 1)]
        if fmt != 6:
            w = nb // 4
            for i in range(4):
                code = int(sum(int(b) << k for k, b in enumerate(mine[w * i: w * (i + 1)])))
                assert np.isclose(back[4 * lane + i], sigma * lev[fmt][code], rtol=1e-6)
        else:
            assert len(mine) == 6


def test_oracle_degenerate_vectors(orc):
    """A zero vector has sigma clamped at 1e-6 and codes on the middle levels; a constant vector is fine."""
    R = orc.restated()
    z = np.zeros((1, 1, 128), np.float16)
    for fmt, _, bpv in FMTS:
        store, meta = R.kv_store_tq(z, None, fmt)
        assert float(meta[0, 0]) == pytest.approx(1e-6, rel=0.06)      # 1e-6 on the FP16 subnormal grid
        back = R.kv_load_tq(store[0], meta[0, 0], fmt)
        assert np.abs(back).max() < 3e-6


# ------------------------------------------------------------------ CPU: pin the oracle to the reference kernel's bytes
@pytest.fixture(scope="module")
def gold():
    if not os.path.exists(GOLD):
        pytest.skip("tests/golden/tq_kv_golden.npz not generated yet (tests/golden/make_golden_tq.py, needs a GPU)")
    return dict(np.load(GOLD))


def compare_with_allowance(got_store, got_meta, want_store, want_meta, bpv, what):
    """Codes and sigmas against the device's. The device's square root and reciprocal are
    approximations (within 2 float ulps), so a code may differ where value / sigma sits on a
    threshold and a sigma where it sits on a FP16 rounding boundary: at most a few in a
    thousand vectors, and never by more than one level / one FP16 ulp."""
    gm, wm = got_meta.view(np.uint16).astype(np.int32), want_meta.view(np.uint16).astype(np.int32)
    assert np.abs(gm - wm).max() <= 1, what
    assert (gm != wm).mean() < 5e-3, what
    n_vec = got_store.size // bpv
    vec_diff = (got_store.reshape(n_vec, bpv) != want_store.reshape(n_vec, bpv)).any(axis=1)
    assert vec_diff.mean() < 2e-2, (what, float(vec_diff.mean()))
    byte_diff = (got_store != want_store).mean()
    assert byte_diff < 1e-3, (what, float(byte_diff))
    return int(vec_diff.sum()), int((gm != wm).sum())


@pytest.mark.parametrize("fmt,name,bpv", FMTS)
def test_oracle_matches_reference_kernel_golden(orc, gold, fmt, name, bpv):
    R = orc.restated()
    k, v, kref = (gold[n].view(np.float16) for n in ("k", "v", "k_ref"))
    ks, km = R.kv_store_tq(k, kref, fmt)
    vs, vm = R.kv_store_tq(v, None, fmt)
    dk = compare_with_allowance(ks, km, gold[f"k_store_{name}"], gold[f"k_meta_{name}"], bpv, "K")
    dv = compare_with_allowance(vs, vm, gold[f"v_store_{name}"], gold[f"v_meta_{name}"], bpv, "V")
    print(f"{name}: oracle vs reference kernel: vectors / sigmas differing: K {dk}, V {dv} of {k.shape[0] * k.shape[1]}")


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


@pytest.fixture(scope="module")
def refk():
    """The reference's own store kernel, live (oracle/_ref/libvvref_cuda.so)."""
    if not os.path.exists(REF_CUDA):
        pytest.skip("the reference's CUDA kernels were not compiled")
    ref = C.CDLL(REF_CUDA)
    vp, i = C.c_void_p, C.c_int
    ref.vv_kv_store_dev.argtypes = [vp, vp, vp, vp, vp, vp, vp, C.c_bool, i, i, i, vp, i, i, vp, vp]
    ref.vv_kv_store_dev.restype = i
    ref.vv_rope_dev.argtypes = [vp, i, i, i, i, vp, C.c_float, vp]
    ref.vv_bias_add_dev.argtypes = [vp, vp, i, i, vp]
    return ref


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def p(t):
    return t.data_ptr() if t is not None else None


@gpu
@pytest.mark.parametrize("fmt,name,bpv", FMTS)
@pytest.mark.parametrize("rows,pos0,row0,with_bias,with_ref,paged", [
    (1, 913, 913, True, True, False),            # a decode step
    (300, 0, 0, True, True, False),              # prefill from an empty cache
    (2048, 4096, 4096, False, False, False),     # a later chunk: no biases, no reference key
    (130, 64, 64, True, True, True),             # the server's paged cache
])
def test_fused_append_writes_the_reference_kernels_bytes(vv, refk, orc, fmt, name, bpv, rows, pos0, row0, with_bias,
                                                         with_ref, paged):
    """bias adds + RoPE + TurboQuant store in ONE launch against the reference's store kernel fed
    the FP16 tensors this library's own separate ops produce (bias adds, RoPE): the stored codes
    and sigmas must be the reference kernel's, byte for byte; and against the oracle with the
    approximation allowance."""
    rng = np.random.default_rng(rows * 7 + fmt)
    f16 = lambda *s, sc=1.0: (rng.standard_normal(s) * sc).astype(np.float16)
    q, k, v = f16(rows, NQ, HD), f16(rows, NKV, HD, sc=1.5), f16(rows, NKV, HD, sc=0.4)
    if rows > 10:
        k[3, :, 40] = 30.0
        v[5] = 0
    qb, kb, vb = (f16(NQ * HD, sc=0.3), f16(NKV * HD, sc=0.3), f16(NKV * HD, sc=0.3)) if with_bias else (None,) * 3
    kref = f16(NKV, HD, sc=0.5) if with_ref else None
    n_pages = (row0 + rows + 63) // 64 + 2
    max_len = n_pages * 64
    table = None
    if paged:
        perm = rng.permutation(n_pages).astype(np.int32)
        table = dev(perm)
    fill = lambda w, dt=torch.uint8: torch.full((max_len, w), 0xA5 if dt == torch.uint8 else 7.0, dtype=dt, device="cuda")

    # ---- ours: one launch
    dq, dk, dv = dev(q), dev(k), dev(v)
    ks, vs = fill(NKV * bpv), fill(NKV * bpv)
    km, vm = fill(NKV, torch.float16), fill(NKV, torch.float16)
    n0 = vv.launch_count()
    st = vv.vvb_kv_append_dev(dq, dk, dv, ks, vs, rows, NQ, NKV, HD, q_bias=dev(qb) if with_bias else None,
                              k_bias=dev(kb) if with_bias else None, v_bias=dev(vb) if with_bias else None,
                              k_ref=dev(kref) if with_ref else None, page_table=table, position_offset=pos0,
                              cache_offset=row0, theta=1e6, kv_format=fmt, keep_k=1, k_meta=km, v_meta=vm)
    assert st == 0 and vv.launch_count() - n0 == 1
    torch.cuda.synchronize()

    # ---- the reference's kernel on this library's own FP16 intermediates (bias adds, RoPE: both
    #      bit-identical to what the fused launch forms inside; keep_k = 1 left the rotated K in dk)
    v16 = dev(v)
    if with_bias:
        assert vv.vv_bias_add_dev(v16, dev(vb), rows, NKV * HD) == 0
    rks, rvs = fill(NKV * bpv), fill(NKV * bpv)
    rkm, rvm = fill(NKV, torch.float16), fill(NKV, torch.float16)
    rref = dev(kref) if with_ref else None
    st = refk.vv_kv_store_dev(p(dk), p(v16), p(rks), p(rvs), p(rkm), p(rvm), p(rref), False, NKV, HD, row0, None,
                              rows, fmt, p(table), None)
    assert st == 0
    torch.cuda.synchronize()
    for got, want, what in ((ks, rks, "K codes"), (vs, rvs, "V codes"), (km.view(torch.int16), rkm.view(torch.int16), "K sigma"),
                            (vm.view(torch.int16), rvm.view(torch.int16), "V sigma")):
        assert torch.equal(got, want), what            # untouched rows keep their fill on both sides, too

    # ---- Q rotated in place as ever, K kept
    add = lambda x, b: (x.astype(np.float32) + b.astype(np.float32)).astype(np.float16) if b is not None else x
    want_q = orc.rope_f16(add(q.reshape(rows, -1), qb).reshape(q.shape), pos0, 1e6)
    assert orc.rope_error_in_ulps(dq.cpu().numpy(), want_q, add(q.reshape(rows, -1), qb).reshape(q.shape)).max() <= 2.0

    # ---- the oracle on the same FP16 K and V, with the approximation allowance (contiguous cases)
    if not paged and rows >= 100:
        R = orc.restated()
        ok_s, ok_m = R.kv_store_tq(dk.cpu().numpy(), kref, fmt)
        ov_s, ov_m = R.kv_store_tq(v16.cpu().numpy(), None, fmt)
        sl = slice(row0, row0 + rows)
        compare_with_allowance(ok_s, ok_m, ks.cpu().numpy()[sl], km.cpu().numpy()[sl], bpv, "K vs oracle")
        compare_with_allowance(ov_s, ov_m, vs.cpu().numpy()[sl], vm.cpu().numpy()[sl], bpv, "V vs oracle")


@gpu
@pytest.mark.parametrize("fmt,name,bpv", FMTS)
def test_extreme_and_nonfinite_vectors_match_the_reference_kernel(vv, refk, fmt, name, bpv):
    """Vectors the code search must not trip over: infinities and NaNs (every scaled value is
    then NaN and exceeds no threshold), values far outside the outermost threshold, the largest
    halves, subnormals, exact zeros, and values on a grid of quarters. V goes through the fused
    launch untouched (no bias), so both kernels see the same bits; codes and sigmas must be the
    reference kernel's."""
    rng = np.random.default_rng(40 + fmt)
    rows = 96
    v = (rng.standard_normal((rows, NKV, HD)) * 0.7).astype(np.float16)
    v[1, 0, 17] = np.inf
    v[2, 1, 5] = -np.inf
    v[2, 1, 90] = np.inf
    v[3, 2, :] = np.nan
    v[4, 3, 64] = np.nan
    v[5, 0, :] = 65504.0
    v[6, 1, ::2] = 65504.0
    v[6, 1, 1::2] = -65504.0
    v[7, 2, :] = 6e-8                      # subnormal halves
    v[8, 3, :] = 0
    v[9, 0, :] = 0
    v[9, 0, 3] = 1.0                       # one spike: every transformed value has the same size
    v[10, 1, :] = (rng.integers(-16, 17, HD) * 0.25).astype(np.float16)
    v[11, 2, :] = 1.0
    v[12, 3, 7] = 1000.0                   # one value many sigmas out
    q = rng.standard_normal((rows, NQ, HD)).astype(np.float16)
    k = rng.standard_normal((rows, NKV, HD)).astype(np.float16)
    dq, dk, dv = dev(q), dev(k), dev(v)
    fill = lambda w, dt=torch.uint8: torch.full((rows, w), 0xA5 if dt == torch.uint8 else 7.0, dtype=dt, device="cuda")
    ks, vs, km, vm = fill(NKV * bpv), fill(NKV * bpv), fill(NKV, torch.float16), fill(NKV, torch.float16)
    assert vv.vvb_kv_append_dev(dq, dk, dv, ks, vs, rows, NQ, NKV, HD, kv_format=fmt, keep_k=1, k_meta=km,
                                v_meta=vm) == 0
    rks, rvs, rkm, rvm = fill(NKV * bpv), fill(NKV * bpv), fill(NKV, torch.float16), fill(NKV, torch.float16)
    assert refk.vv_kv_store_dev(p(dk), p(dv), p(rks), p(rvs), p(rkm), p(rvm), None, False, NKV, HD, 0, None, rows, fmt,
                                None, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(vs, rvs), "V codes"
    assert torch.equal(ks, rks), "K codes"
    # sigmas as bit patterns; a NaN sigma may differ in payload only
    for got, want, what in ((vm, rvm, "V sigma"), (km, rkm, "K sigma")):
        g, w = got.view(torch.int16).cpu().numpy(), want.view(torch.int16).cpu().numpy()
        nan_g, nan_w = np.isnan(got.cpu().numpy()), np.isnan(want.cpu().numpy())
        assert np.array_equal(nan_g, nan_w), what
        assert np.array_equal(g[~nan_g], w[~nan_w]), what


@gpu
def test_fuzz_tq_append_against_the_reference_kernel(vv, refk):
    """Random head counts (K columns that straddle the kernel's column chunks, KV head counts that do
    not divide its warp count), row counts, formats, paged or not, with and without biases and
    reference key: the fused launch's codes and sigmas against the reference's store kernel fed the
    FP16 K this library leaves in place (keep_k) and the biased V."""
    rng = np.random.default_rng(2024)
    bpv_of = {3: 64, 4: 48, 5: 32, 6: 24}
    for case in range(24):
        nq, nkv = int(rng.integers(1, 41)), int(rng.integers(1, 9))
        rows = int(rng.choice([1, 2, 5, 64, 65, 200]))
        fmt = int(rng.integers(3, 7))
        bpv = bpv_of[fmt]
        paged = bool(rng.integers(2))
        first = int(rng.choice([0, 3, 64, 100]))
        pos0 = int(rng.choice([0, 7, 5000]))
        f16 = lambda *s, sc=1.0: (rng.standard_normal(s) * sc).astype(np.float16)
        q, k, v = f16(rows, nq, HD), f16(rows, nkv, HD, sc=1.5), f16(rows, nkv, HD, sc=0.4)
        qb = f16(nq * HD, sc=0.3) if rng.integers(2) else None
        kb = f16(nkv * HD, sc=0.3) if rng.integers(2) else None
        vb = f16(nkv * HD, sc=0.3) if rng.integers(2) else None
        kref = f16(nkv, HD, sc=0.5) if rng.integers(2) else None
        n_pages = (first + rows + 63) // 64
        pool = n_pages + 3
        table = dev(rng.permutation(pool)[:n_pages].astype(np.int32)) if paged else None
        cache_rows = pool * 64 if paged else first + rows + 2
        fill = lambda w, dt=torch.uint8: torch.full((cache_rows, w), 0xA5 if dt == torch.uint8 else 7.0, dtype=dt, device="cuda")
        opt = lambda a: dev(a) if a is not None else None
        dq, dk, dv = dev(q), dev(k), dev(v)
        ks, vs, km, vm = fill(nkv * bpv), fill(nkv * bpv), fill(nkv, torch.float16), fill(nkv, torch.float16)
        tag = (case, nq, nkv, rows, fmt, paged, first)
        st = vv.vvb_kv_append_dev(dq, dk, dv, ks, vs, rows, nq, nkv, HD, q_bias=opt(qb), k_bias=opt(kb), v_bias=opt(vb),
                                  k_ref=opt(kref), page_table=table, position_offset=pos0, cache_offset=first,
                                  kv_format=fmt, keep_k=1, k_meta=km, v_meta=vm)
        assert st == 0, tag + (st,)
        v16 = dev(v)
        if vb is not None:
            assert vv.vv_bias_add_dev(v16, dev(vb), rows, nkv * HD) == 0
        rks, rvs, rkm, rvm = fill(nkv * bpv), fill(nkv * bpv), fill(nkv, torch.float16), fill(nkv, torch.float16)
        st = refk.vv_kv_store_dev(p(dk), p(v16), p(rks), p(rvs), p(rkm), p(rvm), p(opt(kref)), False, nkv, HD, first,
                                  None, rows, fmt, p(table), None)
        assert st == 0, tag
        torch.cuda.synchronize()
        for got, want, what in ((ks, rks, "K codes"), (vs, rvs, "V codes"),
                                (km.view(torch.int16), rkm.view(torch.int16), "K sigma"),
                                (vm.view(torch.int16), rvm.view(torch.int16), "V sigma")):
            assert torch.equal(got, want), tag + (what,)


@gpu
def test_tq_argument_checks(vv):
    x = torch.zeros(4, 4, 128, dtype=torch.float16, device="cuda")
    q = torch.zeros(4, 28, 128, dtype=torch.float16, device="cuda")
    store = torch.zeros(8, 4 * 64, dtype=torch.uint8, device="cuda")
    meta = torch.zeros(8, 4, dtype=torch.float16, device="cuda")
    # sigma arrays are required; head_dim must be 128
    assert vv.vvb_kv_append_dev(q, x, x, store, store, 4, 28, 4, 128, kv_format=3) == vv.VV_ERR_NULL_PTR
    q64 = torch.zeros(4, 28, 64, dtype=torch.float16, device="cuda")
    x64 = torch.zeros(4, 4, 64, dtype=torch.float16, device="cuda")
    assert vv.vvb_kv_append_dev(q64, x64, x64, store, store, 4, 28, 4, 64, kv_format=3, k_meta=meta,
                                v_meta=meta) == vv.VV_ERR_UNSUPPORTED
    assert vv.vvb_kv_append_dev(q, x, x, store, store, 4, 28, 4, 128, kv_format=7, k_meta=meta,
                                v_meta=meta) == vv.VV_ERR_UNSUPPORTED
    assert vv.vvb_kv_append_dev(q, x, x, store, store, 0, 28, 4, 128, kv_format=3, k_meta=meta, v_meta=meta) == vv.VV_OK
