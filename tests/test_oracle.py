"""Pins the CPU restatement (oracle/vvb_oracle.c).

Three anchors:
 1. the committed golden vectors, which the reference's own compiled CPU
    kernels produced (tests/golden/make_golden.py);
 2. the reference's known-answer checks restated at their shapes and
    tolerances (tests/test_cpu_kernels.c:150-183);
 3. where the compiled reference is present, a live bit-for-bit comparison on
    fresh seeded inputs.
"""
import numpy as np
import pytest


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32 if a.dtype == np.float32 else np.uint16)


# ---------------------------------------------------------------- converters
def test_half_to_float_all_65536_patterns(orc):
    L = orc.restated().lib
    h = np.arange(65536, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32)
    out = np.empty(65536, np.float32)
    L.orc_widen_f16(h.ctypes.data_as(orc._u16p), out.ctypes.data_as(orc._f32p), h.size)
    assert np.array_equal(bits(out), bits(want))


def test_float_to_half_rne_matches_ieee(orc):
    L = orc.restated().lib
    rng = np.random.default_rng(1)
    u = rng.integers(0, 2 ** 32, size=400_000, dtype=np.uint64).astype(np.uint32)
    # ties and boundaries: every half value +- half an ulp, the documented
    # cases of include/vibevoice/types.h:171-180 (1+2^-11 -> 0x3C00, 1+3*2^-11 -> 0x3C02)
    halves = np.arange(0x7C00, dtype=np.uint16).view(np.float16).astype(np.float64)
    step = np.diff(halves, append=65536.0)
    ties = (halves + step / 2).astype(np.float32)
    special = np.array([1 + 2.0 ** -11, 1 + 3 * 2.0 ** -11, 65504.0, 65519.99, 65520.0, 2.0 ** -25,
                        np.nextafter(np.float32(2.0 ** -25), np.float32(1)), 0.0, -0.0, np.inf, -np.inf],
                       np.float32)
    x = np.concatenate([u.view(np.float32), ties, -ties, special])
    x = x[~np.isnan(x)]
    out = np.empty(x.size, np.uint16)
    L.orc_round_f16(np.ascontiguousarray(x).ctypes.data_as(orc._f32p), out.ctypes.data_as(orc._u16p), x.size)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(out, want)
    assert L.orc_float_to_half_rne(np.float32(1 + 2.0 ** -11)) == 0x3C00
    assert L.orc_float_to_half_rne(np.float32(1 + 3 * 2.0 ** -11)) == 0x3C02
    assert L.orc_float_to_half_rne(np.float32(np.nan)) & 0x7C00 == 0x7C00


# ---------------------------------------------------------------- golden vectors
@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_rmsnorm_golden(orc, golden, tag):
    x, w, y = (golden[f"rmsnorm_{tag}_{k}"] for k in "xwy")
    got = orc.restated().rmsnorm(x, w, x.shape[0], x.shape[1], np.float32(1e-6))
    assert np.array_equal(bits(got), bits(y))


def test_add_rmsnorm_f16_golden(orc, golden):
    h, d, w = golden["addnorm_h"], golden["addnorm_d"], golden["addnorm_w"]
    hn, y = orc.add_rmsnorm_f16(h, d, w, 1e-6)
    assert np.array_equal(bits(hn), bits(golden["addnorm_h_out"]))
    assert np.array_equal(bits(y), bits(golden["addnorm_y"]))
    # the single-call C composite agrees with the python composition
    h2, y2 = h.copy(), np.empty_like(h)
    st = orc.restated().lib.orc_add_rmsnorm_f16(
        h2.view(np.uint16).ctypes.data_as(orc._u16p), d.view(np.uint16).ctypes.data_as(orc._u16p),
        w.view(np.uint16).ctypes.data_as(orc._u16p), y2.view(np.uint16).ctypes.data_as(orc._u16p),
        h.shape[0], h.shape[1], np.float32(1e-6))
    assert st == 0
    assert np.array_equal(bits(h2), bits(hn)) and np.array_equal(bits(y2), bits(y))


@pytest.mark.parametrize("tag", ["a", "b", "c", "d"])
def test_rope_golden(orc, golden, tag):
    x = golden[f"rope_{tag}_x"]
    off, theta = golden[f"rope_{tag}_meta"]
    rows, heads, hd = x.shape
    got32 = orc.restated().rope(x.astype(np.float32), rows, heads, hd, int(off), np.float32(theta))
    assert np.array_equal(bits(got32), bits(golden[f"rope_{tag}_y32"]))
    got16 = orc.rope_f16(x, int(off), theta)
    assert np.array_equal(bits(got16), bits(golden[f"rope_{tag}_y16"]))
    x2 = x.copy()
    st = orc.restated().lib.orc_rope_f16(x2.view(np.uint16).ctypes.data_as(orc._u16p),
                                         rows, heads, hd, int(off), np.float32(theta))
    assert st == 0 and np.array_equal(bits(x2), bits(got16))


def test_swiglu_golden(orc, golden):
    got = orc.restated().swiglu(golden["swiglu_a_g"], golden["swiglu_a_u"])
    assert np.array_equal(bits(got), bits(golden["swiglu_a_y"]))
    got16 = orc.swiglu_f16(golden["swiglu_b_g"], golden["swiglu_b_u"])
    assert np.array_equal(bits(got16), bits(golden["swiglu_b_y"]))
    g, u = golden["swiglu_b_g"], golden["swiglu_b_u"]
    out = np.empty_like(g)
    st = orc.restated().lib.orc_swiglu_f16(g.view(np.uint16).ctypes.data_as(orc._u16p),
                                           u.view(np.uint16).ctypes.data_as(orc._u16p),
                                           out.view(np.uint16).ctypes.data_as(orc._u16p), g.size)
    assert st == 0 and np.array_equal(bits(out), bits(got16))


def test_residual_add_golden(orc, golden):
    got = orc.restated().residual_add(golden["resadd_x"], golden["resadd_y"])
    assert np.array_equal(bits(got), bits(golden["resadd_out"]))


def test_embedding_golden(orc, golden):
    t, ids = golden["embed_table"], golden["embed_ids"]
    got = orc.restated().embedding(t, ids, ids.size, t.shape[1])
    assert np.array_equal(bits(got), bits(golden["embed_out"]))
    # the gather is a bit copy: rounding the widened rows back returns the table's bits
    assert np.array_equal(bits(orc.embedding_f16(t, ids)), bits(t[ids]))


# ---------------------------------------------------------------- known-answer restatements
def test_rmsnorm_known_answer(orc):
    """tests/test_cpu_kernels.c:150-168: rows 4 x n 128, inputs in [-3, 3],
    weight 1 +- 0.2, relative tolerance 1e-5 against a float64 evaluation."""
    rng = np.random.default_rng(7)
    x = rng.uniform(-3, 3, (4, 128)).astype(np.float32)
    w = (1.0 + rng.uniform(-0.2, 0.2, 128)).astype(np.float16)
    got = orc.restated().rmsnorm(x, w, 4, 128, np.float32(1e-6))
    xd = x.astype(np.float64)
    want = xd / np.sqrt((xd * xd).mean(1, keepdims=True) + 1e-6) * w.astype(np.float64)
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-3)) <= 1e-5


def test_swiglu_known_answer(orc):
    """tests/test_cpu_kernels.c:171-183: n 1024, gate in [-4, 4], up in
    [-1, 1], relative tolerance 1e-6."""
    rng = np.random.default_rng(8)
    g = rng.uniform(-4, 4, 1024).astype(np.float32)
    u = rng.uniform(-1, 1, 1024).astype(np.float32)
    got = orc.restated().swiglu(g, u)
    gd, ud = g.astype(np.float64), u.astype(np.float64)
    want = gd / (1 + np.exp(-gd)) * ud
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-3)) <= 1e-6


def test_rope_rotation_properties(orc):
    """Position 0 is the identity; the rotation preserves each pair's norm;
    rows at offset p equal one-row calls at p (row independence, the property
    token sharding rests on)."""
    rng = np.random.default_rng(9)
    x = rng.standard_normal((7, 3, 128)).astype(np.float32)
    R = orc.restated()
    y0 = R.rope(x[:1], 1, 3, 128, 0, np.float32(1e6))
    assert np.array_equal(bits(y0), bits(x[:1]))
    y = R.rope(x, 7, 3, 128, 1000, np.float32(1e6))
    n_in = x[..., :64] ** 2 + x[..., 64:] ** 2
    n_out = y[..., :64] ** 2 + y[..., 64:] ** 2
    assert np.allclose(n_in, n_out, rtol=1e-5, atol=1e-6)
    for r in range(7):
        one = R.rope(x[r:r + 1], 1, 3, 128, 1000 + r, np.float32(1e6))
        assert np.array_equal(bits(one), bits(y[r:r + 1]))


def test_null_and_empty(orc):
    L = orc.restated().lib
    assert L.orc_rmsnorm(None, None, None, 1, 8, np.float32(1e-6)) == -2
    assert L.orc_rope(None, 1, 1, 8, 0, np.float32(1e4)) == -2
    assert L.orc_swiglu(None, None, None, 0) == -2
    e = np.zeros((0, 8), np.float32)
    w = np.ones(8, np.float16)
    assert orc.restated().rmsnorm(e, w, 0, 8, np.float32(1e-6)).shape == (0, 8)


# ---------------------------------------------------------------- live reference
needs_ref = pytest.mark.skipif(
    not __import__("oracle").have_reference(), reason="compiled reference CPU kernels not present")


@needs_ref
def test_restated_equals_reference_live(orc):
    R, F = orc.restated(), orc.reference()
    rng = np.random.default_rng(123)
    for rows, n in ((9, 3584), (3, 1536), (5, 250), (2, 8)):
        x = rng.standard_normal((rows, n)).astype(np.float32) * 2
        w = (1 + 0.02 * rng.standard_normal(n)).astype(np.float16)
        for eps in (1e-6, 1e-5):
            assert np.array_equal(bits(R.rmsnorm(x, w, rows, n, np.float32(eps))),
                                  bits(F.rmsnorm(x, w, rows, n, np.float32(eps))))
    for rows, heads, hd, off, theta in ((17, 28, 128, 0, 1e6), (5, 4, 128, 14444, 1e6),
                                        (3, 2, 64, 77, 1e4), (2, 12, 128, 131071, 1e6), (2, 1, 6, 3, 50.0)):
        x = rng.standard_normal((rows, heads, hd)).astype(np.float32)
        assert np.array_equal(bits(R.rope(x, rows, heads, hd, off, np.float32(theta))),
                              bits(F.rope(x, rows, heads, hd, off, np.float32(theta))))
    g = (rng.standard_normal(200_001) * 5).astype(np.float32)
    u = rng.standard_normal(200_001).astype(np.float32)
    assert np.array_equal(bits(R.swiglu(g, u)), bits(F.swiglu(g, u)))
    assert np.array_equal(bits(R.residual_add(g, u)), bits(F.residual_add(g, u)))
    t = (0.02 * rng.standard_normal((500, 1536))).astype(np.float16)
    ids = rng.integers(0, 500, 64).astype(np.int32)
    assert np.array_equal(bits(R.embedding(t, ids, 64, 1536)), bits(F.embedding(t, ids, 64, 1536)))


@needs_ref
def test_f16_composites_equal_reference_live(orc):
    F = orc.reference()
    rng = np.random.default_rng(5)
    h = rng.standard_normal((33, 3584)).astype(np.float16)
    d = rng.standard_normal((33, 3584)).astype(np.float16)
    w = (1 + 0.02 * rng.standard_normal(3584)).astype(np.float16)
    a = orc.add_rmsnorm_f16(h, d, w, 1e-6)
    b = orc.add_rmsnorm_f16(h, d, w, 1e-6, impl=F)
    assert np.array_equal(bits(a[0]), bits(b[0])) and np.array_equal(bits(a[1]), bits(b[1]))
    q = rng.standard_normal((40, 28, 128)).astype(np.float16)
    assert np.array_equal(bits(orc.rope_f16(q, 4000, 1e6)), bits(orc.rope_f16(q, 4000, 1e6, impl=F)))
    g = rng.standard_normal((8, 18944)).astype(np.float16)
    u = rng.standard_normal((8, 18944)).astype(np.float16)
    assert np.array_equal(bits(orc.swiglu_f16(g, u)), bits(orc.swiglu_f16(g, u, impl=F)))
