"""FP8 KV cache: the oracle against the reference's own store kernel (golden
bytes, and live on a GPU), and the fused bias + RoPE + FP8 append against the
oracle. Bytes are integers, so every comparison is exact."""
import ctypes as C
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden", "fp8_kv_golden.npz")
REF_CUDA = os.path.join(ROOT, "oracle", "_ref", "libvvref_cuda.so")
FMTS = [(1, "e4m3"), (2, "e5m2")]
NQ, NKV, HD = 28, 4, 128


@pytest.fixture(scope="module")
def gold():
    return dict(np.load(GOLD))


# ------------------------------------------------------------------ CPU: pin the oracle
@pytest.mark.parametrize("fmt,name", FMTS)
def test_oracle_encodes_every_half_as_the_reference_kernel(orc, gold, fmt, name):
    """All 65 536 FP16 bit patterns (zeros, subnormals, infinities and NaNs included)."""
    every = np.arange(65536, dtype=np.uint16).view(np.float16).reshape(128, 512)
    got = orc.restated().kv_store_fp8(every, None, fmt).reshape(-1)
    assert np.array_equal(got, gold[f"all_halves_{name}"])
    # the scalar encoder agrees wherever the input is not a NaN (a NaN reaches the device
    # encoder in canonical form, sign clear, and is stored as 0x00)
    flat = every.reshape(-1).astype(np.float32)
    ok = ~np.isnan(flat)
    assert np.array_equal(orc.restated().fp8_encode(flat[ok], fmt), gold[f"all_halves_{name}"][ok])


@pytest.mark.parametrize("fmt,name", FMTS)
def test_oracle_store_with_reference_key_matches_golden(orc, gold, fmt, name):
    R = orc.restated()
    k, v, kref = (gold[n].view(np.float16) for n in ("k", "v", "k_ref"))
    assert np.array_equal(R.kv_store_fp8(k, kref, fmt), gold[f"k_minus_ref_{name}"])
    assert np.array_equal(R.kv_store_fp8(v, None, fmt), gold[f"v_{name}"])


@pytest.mark.parametrize("fmt", [1, 2])
def test_oracle_fp8_properties(orc, fmt):
    """Known answers of the format: the largest finite value and where it
    saturates, the smallest normal, the half-up subnormal rounding, NaN -> 0,
    and decode(encode(x)) == x for every representable value."""
    R = orc.restated()
    enc = lambda *x: R.fp8_encode(np.array(x, np.float32), fmt).tolist()
    if fmt == 1:
        assert enc(448.0, 463.9, 464.0, 1e9, np.inf) == [0x7E] * 5
        assert enc(-448.0, 2.0 ** -6, 2.0 ** -9, 2.0 ** -10, 0.99 * 2.0 ** -10) == [0xFE, 0x08, 0x01, 0x01, 0x00]
        assert enc(7.5 * 2.0 ** -9, 1.0, 1.0625, 1.1875) == [0x08, 0x38, 0x38, 0x3A]      # ties to even in the normal range
    else:
        assert enc(57344.0, 61439.0, 61440.0, np.inf) == [0x7B] * 4
        assert enc(2.0 ** -14, 2.0 ** -16, 2.0 ** -17, 1.0, 1.125, 1.375) == [0x04, 0x01, 0x01, 0x3C, 0x3C, 0x3E]
    assert enc(np.nan, 0.0, -0.0) == [0x00, 0x00, 0x80]
    top = 0x7E if fmt == 1 else 0x7B
    codes = np.array([c for c in range(256) if (c & 0x7F) <= top], np.uint8)
    back = R.fp8_encode(R.fp8_decode(codes, fmt), fmt)
    assert np.array_equal(back, codes)


@pytest.mark.parametrize("fmt", [1, 2])
def test_oracle_fp8_is_monotone_and_nearest_on_floats(orc, fmt):
    """Arbitrary floats (the reference-key path feeds differences of halves, not
    halves): the code is monotone in the magnitude, symmetric in the sign, and
    decodes to a value within half a grid step of the input inside the finite
    range (the subnormal range rounds half up, the rest to nearest even)."""
    R = orc.restated()
    rng = np.random.default_rng(50 + fmt)
    top, tiny = (448.0, 2.0 ** -9) if fmt == 1 else (57344.0, 2.0 ** -16)
    mags = np.sort(np.concatenate([
        np.exp(rng.uniform(np.log(tiny / 8), np.log(top * 2), 4000)),
        np.array([tiny / 2, tiny, 2.0 ** (-6 if fmt == 1 else -14), top, top * 1.03], np.float64)])).astype(np.float32)
    codes = R.fp8_encode(mags, fmt).astype(np.int32)
    assert (np.diff(codes) >= 0).all()                                    # monotone
    assert np.array_equal(R.fp8_encode(-mags, fmt).astype(np.int32), codes | 0x80)
    back = R.fp8_decode(codes.astype(np.uint8), fmt).astype(np.float64)
    inside = mags <= top
    M = 3 if fmt == 1 else 2
    emin = -6 if fmt == 1 else -14
    expo = np.maximum(np.floor(np.log2(np.maximum(mags[inside].astype(np.float64), 1e-30))), emin)
    step = np.ldexp(1.0, (expo - M).astype(np.int64))
    assert (np.abs(back[inside] - mags[inside]) <= 0.5 * step * (1 + 1e-6)).all()
    assert (codes[~inside] == (0x7E if fmt == 1 else 0x7B)).all()         # saturation above the largest finite value


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


def expected(orc, q, k, v, qb, kb, vb, kref, pos0, row0, max_len, fmt, theta=1e6, NKV=NKV, HD=HD):
    """The reference's sequence on the CPU: bias adds rounded to FP16, RoPE, FP16
    result, then the FP8 store (K minus the reference key, V as is)."""
    add = lambda x, b: (x.astype(np.float32) + b.astype(np.float32)).astype(np.float16) if b is not None else x
    qq, kk, vv_ = add(q, qb), add(k, kb), add(v, vb)
    q_out = orc.rope_f16(qq, pos0, theta)
    k_rot = orc.rope_f16(kk, pos0, theta)
    R = orc.restated()
    ks = R.kv_store_fp8(k_rot, kref, fmt, row0, np.full((max_len, NKV * HD), 0xA5, np.uint8))
    vs = R.kv_store_fp8(vv_, None, fmt, row0, np.full((max_len, NKV * HD), 0xA5, np.uint8))
    return q_out, k_rot, ks, vs


@gpu
@pytest.mark.parametrize("fmt,name", FMTS)
@pytest.mark.parametrize("rows,with_bias,with_ref,keep_k", [(1, True, True, 0), (37, True, False, 1), (300, False, True, 0)])
def test_fused_fp8_append_equals_oracle(vv, orc, fmt, name, rows, with_bias, with_ref, keep_k):
    rng = np.random.default_rng(rows + fmt)
    q = rng.standard_normal((rows, NQ, HD)).astype(np.float16)
    k = (rng.standard_normal((rows, NKV, HD)) * 1.5).astype(np.float16)
    v = (rng.standard_normal((rows, NKV, HD)) * 0.05).astype(np.float16)
    qb = (rng.standard_normal((NQ, HD)) * 0.3).astype(np.float16) if with_bias else None
    kb = (rng.standard_normal((NKV, HD)) * 0.3).astype(np.float16) if with_bias else None
    vb = (rng.standard_normal((NKV, HD)) * 0.01).astype(np.float16) if with_bias else None
    kref = (rng.standard_normal((NKV, HD)) * 0.5).astype(np.float16) if with_ref else None
    pos0, row0, max_len = 1000, 5, rows + 9
    want_q, want_k, want_ks, want_vs = expected(orc, q, k, v, qb, kb, vb, kref, pos0, row0, max_len, fmt)

    dq, dk, dv = dev(q), dev(k), dev(v)
    ks = torch.full((max_len, NKV * HD), 0xA5, dtype=torch.uint8, device="cuda")
    vs = torch.full((max_len, NKV * HD), 0xA5, dtype=torch.uint8, device="cuda")
    opt = lambda a: dev(a) if a is not None else None
    st = vv.vvb_rope_qk_append_fp8_dev(dq, dk, dv, opt(qb), opt(kb), opt(vb), ks, vs, opt(kref), rows, NQ, NKV, HD,
                                       pos0, row0, None, 1e6, fmt, keep_k)
    assert st == 0, st
    torch.cuda.synchronize()
    assert np.array_equal(ks.cpu().numpy(), want_ks)          # rows outside [row0, row0+rows) keep their fill
    assert np.array_equal(vs.cpu().numpy(), want_vs)
    err = orc.rope_error_in_ulps(dq.cpu().numpy(), want_q, (q.astype(np.float32) + (qb if with_bias else 0)).astype(np.float16))
    assert float(err.max()) <= 2.0
    got_k = dk.cpu().numpy()
    if keep_k:
        assert np.array_equal(got_k.view(np.uint16), want_k.view(np.uint16))
    else:
        assert np.array_equal(got_k.view(np.uint16), k.view(np.uint16))       # K itself untouched
    # V is never modified
    assert np.array_equal(dv.cpu().numpy().view(np.uint16), v.view(np.uint16))


@gpu
@pytest.mark.parametrize("fmt", [1, 2])
@pytest.mark.parametrize("rows,nq,nkv,hd", [(9, 8, 40, 128),      # many KV heads: K tile too large to stage
                                            (75, 4, 2, 64),       # narrow heads: 10 rows per pass, staged
                                            (33, 2, 1, 256)])     # wide head
def test_fused_fp8_append_other_shapes(vv, orc, fmt, rows, nq, nkv, hd):
    rng = np.random.default_rng(rows * 7 + fmt)
    q = rng.standard_normal((rows, nq, hd)).astype(np.float16)
    k = (rng.standard_normal((rows, nkv, hd)) * 1.5).astype(np.float16)
    v = (rng.standard_normal((rows, nkv, hd)) * 0.05).astype(np.float16)
    kb = (rng.standard_normal((nkv, hd)) * 0.3).astype(np.float16)
    kref = (rng.standard_normal((nkv, hd)) * 0.5).astype(np.float16)
    pos0, row0, max_len = 77, 3, rows + 5
    want_q, want_k, want_ks, want_vs = expected(orc, q, k, v, None, kb, None, kref, pos0, row0, max_len, fmt, NKV=nkv, HD=hd)
    dq, dk, dv = dev(q), dev(k), dev(v)
    ks = torch.full((max_len, nkv * hd), 0xA5, dtype=torch.uint8, device="cuda")
    vs = torch.full((max_len, nkv * hd), 0xA5, dtype=torch.uint8, device="cuda")
    st = vv.vvb_rope_qk_append_fp8_dev(dq, dk, dv, None, dev(kb), None, ks, vs, dev(kref), rows, nq, nkv, hd,
                                       pos0, row0, None, 1e6, fmt, 1)
    assert st == 0, st
    torch.cuda.synchronize()
    # the cache holds the bytes of the K this launch rotated (kept in place), and that K meets the RoPE bar
    kk = (k.astype(np.float32) + kb.astype(np.float32)).astype(np.float16)
    k_rot = dk.cpu().numpy()
    assert float(orc.rope_error_in_ulps(k_rot, want_k, kk).max()) <= 2.0
    R = orc.restated()
    assert np.array_equal(ks.cpu().numpy(), R.kv_store_fp8(k_rot, kref, fmt, row0, np.full((max_len, nkv * hd), 0xA5, np.uint8)))
    assert np.array_equal(vs.cpu().numpy(), want_vs)
    assert float(orc.rope_error_in_ulps(dq.cpu().numpy(), want_q, q).max()) <= 2.0


@gpu
def test_fused_fp8_append_every_half_through_v(vv, orc, gold):
    """V goes through the encoder unrotated: feed all 65 536 halves and demand the
    reference kernel's golden bytes."""
    every = np.arange(65536, dtype=np.uint16).view(np.float16).reshape(128, NKV, HD)
    q = np.zeros((128, NQ, HD), np.float16)
    for fmt, name in FMTS:
        ks = torch.zeros(128, NKV * HD, dtype=torch.uint8, device="cuda")
        vs = torch.zeros_like(ks)
        st = vv.vvb_rope_qk_append_fp8_dev(dev(q), dev(every.copy()), dev(every), None, None, None, ks, vs, None,
                                           128, NQ, NKV, HD, 0, 0, None, 1e6, fmt, 0)
        assert st == 0, st
        torch.cuda.synchronize()
        assert np.array_equal(vs.cpu().numpy().reshape(-1), gold[f"all_halves_{name}"])


@gpu
@pytest.mark.parametrize("fmt,name", FMTS)
def test_decode_by_device_position_under_graph_replay(vv, orc, fmt, name):
    """One token per replay; the device int gives the RoPE position and the cache row."""
    rng = np.random.default_rng(3)
    max_len = 16
    q = rng.standard_normal((1, NQ, HD)).astype(np.float16)
    k = rng.standard_normal((1, NKV, HD)).astype(np.float16)
    v = rng.standard_normal((1, NKV, HD)).astype(np.float16)
    dq0, dk, dv = dev(q), dev(k), dev(v)
    dq = torch.empty_like(dq0)
    ks = torch.zeros(max_len, NKV * HD, dtype=torch.uint8, device="cuda")
    vs = torch.zeros_like(ks)
    dpos = torch.zeros(1, dtype=torch.int32, device="cuda")
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        dq.copy_(dq0)
        assert vv.vvb_rope_qk_append_fp8_dev(dq, dk, dv, None, None, None, ks, vs, None, 1, NQ, NKV, HD, 0, 0, dpos,
                                             1e6, fmt, 0, s.cuda_stream) == 0
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            dq.copy_(dq0)
            assert vv.vvb_rope_qk_append_fp8_dev(dq, dk, dv, None, None, None, ks, vs, None, 1, NQ, NKV, HD, 0, 0,
                                                 dpos, 1e6, fmt, 0, s.cuda_stream) == 0
    ks.zero_(); vs.zero_()
    want_ks = np.zeros((max_len, NKV * HD), np.uint8)
    want_vs = np.zeros_like(want_ks)
    R = orc.restated()
    for pos in (3, 4, 9):
        dpos.fill_(pos)
        g.replay()
        torch.cuda.synchronize()
        R.kv_store_fp8(orc.rope_f16(k, pos, 1e6), None, fmt, pos, want_ks)
        R.kv_store_fp8(v, None, fmt, pos, want_vs)
        assert np.array_equal(ks.cpu().numpy(), want_ks) and np.array_equal(vs.cpu().numpy(), want_vs)
        assert float(orc.rope_error_in_ulps(dq.cpu().numpy(), orc.rope_f16(q, pos, 1e6), q).max()) <= 2.0


@gpu
@pytest.mark.parametrize("fmt", [0, 1, 2])
def test_paged_cache_append(vv, orc, fmt):
    """The server's paged cache (64-position pages of one pool): logical position t
    lands in row page_table[t // 64] * 64 + t % 64 (src/cuda/kv_codec.cuh:29-36).
    FP16 and both FP8 formats, against the oracle's contiguous result scattered by
    the table, and against the reference's own vv_kv_store_dev where it is present."""
    rng = np.random.default_rng(40 + fmt)
    rows, first, pool_pages = 150, 70, 8
    table = np.array([5, 2, 7, 0], np.int32)                 # pages of logical positions 0..255
    q = rng.standard_normal((rows, NQ, HD)).astype(np.float16)
    k = (rng.standard_normal((rows, NKV, HD)) * 1.5).astype(np.float16)
    v = (rng.standard_normal((rows, NKV, HD)) * 0.05).astype(np.float16)
    kb = (rng.standard_normal((NKV, HD)) * 0.3).astype(np.float16)
    kref = (rng.standard_normal((NKV, HD)) * 0.5).astype(np.float16) if fmt else None
    width = NKV * HD
    kk = (k.astype(np.float32) + kb.astype(np.float32)).astype(np.float16)
    dt, fill = (torch.uint8, 0xA5) if fmt else (torch.int16, 0x1234)
    ks = torch.full((pool_pages * 64, width), fill, dtype=dt, device="cuda")
    vs = torch.full((pool_pages * 64, width), fill, dtype=dt, device="cuda")
    dk, dv, dtab = dev(k), dev(v), dev(table)
    st = vv.vvb_kv_append_dev(dev(q), dk, dv, ks, vs, rows, NQ, NKV, HD, k_bias=dev(kb), k_ref=dev(kref) if fmt else None,
                              page_table=dtab, position_offset=9, cache_offset=first, kv_format=fmt, keep_k=1)
    assert st == 0, st
    torch.cuda.synchronize()
    # keep_k left the rotated FP16 K in place: it meets the RoPE bar against the oracle, and the
    # cache must hold exactly that K (FP16) or exactly its FP8 bytes
    k_rot = dk.cpu().numpy()
    assert float(orc.rope_error_in_ulps(k_rot, orc.rope_f16(kk, 9, 1e6), kk).max()) <= 2.0
    if fmt:
        R = orc.restated()
        want_k_rows, want_v_rows = R.kv_store_fp8(k_rot, kref, fmt), R.kv_store_fp8(v, None, fmt)
    else:
        want_k_rows, want_v_rows = k_rot.reshape(rows, width).view(np.uint16), v.reshape(rows, width).view(np.uint16)
    np_dt = np.uint8 if fmt else np.uint16
    want_k = np.full((pool_pages * 64, width), fill, np_dt)
    want_v = np.full((pool_pages * 64, width), fill, np_dt)
    for r in range(rows):
        t = first + r
        phys = int(table[t // 64]) * 64 + t % 64
        want_k[phys], want_v[phys] = want_k_rows[r], want_v_rows[r]
    got_k = ks.cpu().numpy().view(np_dt)
    got_v = vs.cpu().numpy().view(np_dt)
    bad_v = np.nonzero((got_v != want_v).any(axis=1))[0]
    assert bad_v.size == 0, f"V rows differ: {bad_v[:8]}"
    bad_k = np.nonzero((got_k != want_k).any(axis=1))[0]
    assert bad_k.size == 0, f"K rows differ: {bad_k[:8]} ({int((got_k != want_k).sum())} elements)"

    if os.path.exists(REF_CUDA):
        ref = C.CDLL(REF_CUDA)
        vp, i = C.c_void_p, C.c_int
        ref.vv_kv_store_dev.argtypes = [vp, vp, vp, vp, vp, vp, vp, C.c_bool, i, i, i, vp, i, i, vp, vp]
        ks2 = torch.full((pool_pages * 64, width), fill, dtype=dt, device="cuda")
        vs2 = torch.full((pool_pages * 64, width), fill, dtype=dt, device="cuda")
        dkref = dev(kref) if fmt else None
        # dk holds the rotated FP16 K (keep_k): hand it to the reference's store
        assert ref.vv_kv_store_dev(dk.data_ptr(), dv.data_ptr(), ks2.data_ptr(), vs2.data_ptr(), None, None,
                                   dkref.data_ptr() if fmt else None, False, NKV, HD, first, None, rows, fmt,
                                   dtab.data_ptr(), None) == 0
        torch.cuda.synchronize()
        assert torch.equal(ks, ks2) and torch.equal(vs, vs2)

    # a decode step on the same paged cache: the device int gives the RoPE position AND the
    # logical cache position, which the page table maps (position 220 -> page 3 -> pool page 0)
    pos = first + rows
    dpos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    k1 = (rng.standard_normal((1, NKV, HD)) * 1.5).astype(np.float16)
    v1 = (rng.standard_normal((1, NKV, HD)) * 0.05).astype(np.float16)
    dk1 = dev(k1)
    before_k, before_v = ks.clone(), vs.clone()
    assert vv.vvb_kv_append_dev(dev(q[:1]), dk1, dev(v1), ks, vs, 1, NQ, NKV, HD, k_ref=dev(kref) if fmt else None,
                                page_table=dtab, d_position=dpos, kv_format=fmt, keep_k=1) == 0
    torch.cuda.synchronize()
    phys = int(table[pos // 64]) * 64 + pos % 64
    k1_rot = dk1.cpu().numpy()
    assert float(orc.rope_error_in_ulps(k1_rot, orc.rope_f16(k1, pos, 1e6), k1).max()) <= 2.0
    if fmt:
        wk, wv = R.kv_store_fp8(k1_rot, kref, fmt)[0], R.kv_store_fp8(v1, None, fmt)[0]
    else:
        wk, wv = k1_rot.reshape(width).view(np.uint16), v1.reshape(width).view(np.uint16)
    assert np.array_equal(ks[phys].cpu().numpy().view(np_dt), wk) and np.array_equal(vs[phys].cpu().numpy().view(np_dt), wv)
    before_k[phys], before_v[phys] = ks[phys], vs[phys]
    assert torch.equal(before_k, ks) and torch.equal(before_v, vs)        # no other row moved


@gpu
def test_fp8_append_argument_checks(vv):
    z = torch.zeros(1, NKV, HD, dtype=torch.float16, device="cuda")
    zq = torch.zeros(1, NQ, HD, dtype=torch.float16, device="cuda")
    st8 = torch.zeros(4, NKV * HD, dtype=torch.uint8, device="cuda")
    call = lambda fmt, k=z, ks=st8, rows=1: vv.vvb_rope_qk_append_fp8_dev(zq, k, z, None, None, None, ks, st8, None, rows,
                                                                          NQ, NKV, HD, 0, 0, None, 1e6, fmt, 0)
    assert call(0) == vv.VV_ERR_UNSUPPORTED and call(3) == vv.VV_ERR_UNSUPPORTED     # raw and TurboQuant formats
    assert call(1, k=None) == vv.VV_ERR_NULL_PTR and call(1, ks=None) == vv.VV_ERR_NULL_PTR
    assert call(1, rows=-1) == vv.VV_ERR_INVALID_ARG
    assert call(1, rows=0) == vv.VV_OK


@gpu
@pytest.mark.parametrize("fmt,name", FMTS)
def test_oracle_and_kernel_against_the_live_reference_kernel(vv, orc, fmt, name):
    """Where the reference's CUDA store kernel is present: the unfused reference
    sequence (its rope kernel is fast-math, so K is rotated by this library and
    handed to ITS store) against the fused launch, byte for byte."""
    if not os.path.exists(REF_CUDA):
        pytest.skip("reference CUDA kernels not compiled")
    ref = C.CDLL(REF_CUDA)
    vp, i = C.c_void_p, C.c_int
    ref.vv_kv_quant_store_dev.argtypes = [vp, vp, vp, vp, vp, vp, vp, C.c_bool, i, i, i, vp, i, i, vp]
    rng = np.random.default_rng(9 + fmt)
    rows, row0, max_len = 129, 7, 160
    q = rng.standard_normal((rows, NQ, HD)).astype(np.float16)
    k = (rng.standard_normal((rows, NKV, HD)) * 2).astype(np.float16)
    v = (rng.standard_normal((rows, NKV, HD)) * 0.03).astype(np.float16)
    kref = (rng.standard_normal((NKV, HD)) * 0.4).astype(np.float16)
    # fused
    ks, vs = (torch.zeros(max_len, NKV * HD, dtype=torch.uint8, device="cuda") for _ in range(2))
    dk = dev(k)
    assert vv.vvb_rope_qk_append_fp8_dev(dev(q), dk, dev(v), None, None, None, ks, vs, dev(kref), rows, NQ, NKV, HD,
                                         50, row0, None, 1e6, fmt, 1) == 0
    torch.cuda.synchronize()
    # the reference's store on the rotated FP16 K (kept in place by keep_k) and V
    ks2, vs2 = (torch.zeros(max_len, NKV * HD, dtype=torch.uint8, device="cuda") for _ in range(2))
    dkref, dv = dev(kref), dev(v)
    assert ref.vv_kv_quant_store_dev(dk.data_ptr(), dv.data_ptr(), ks2.data_ptr(), vs2.data_ptr(), None, None,
                                     dkref.data_ptr(), False, NKV, HD, row0, None, rows, fmt, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(ks, ks2) and torch.equal(vs, vs2)
