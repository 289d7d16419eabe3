"""Seeded random shapes through every kernel family, against the CPU oracle.

The fixed-shape tests pin the model's sizes and the edges that were thought of;
this file walks launch-shape boundaries that were not: row counts either side
of the one-wave threshold, widths either side of the vector / CTA limits, odd
head counts and head sizes, offsets, optional arguments present or absent.
Every case guards its outputs with canary bands. Bars are the parity bars of
test_parity_gpu.py (bit-exact where the output is an integer, a copy or the
residual sum; 2 FP16 ulp for the norm and SwiGLU; 2 ulp at operand scale for
RoPE)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from test_parity_gpu import Guarded, bits, dev  # noqa: E402  (tests/ is on sys.path: conftest.py)


@pytest.fixture(scope="module")
def vv():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import vvb200
    torch.cuda.set_device(0)
    return vvb200


def r16(rng, *shape, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(np.float16)


def test_fuzz_add_rmsnorm(vv, orc):
    rng = np.random.default_rng(1001)
    widths = [8, 24, 256, 1536, 3584, 4096, 4104, 8192, 12288, 250, 3585]
    for case in range(40):
        rows = int(rng.choice([1, 2, 31, 148, 591, 592, 593, 700, 1200]))
        hidden = int(rng.choice(widths))
        if rows * hidden > 3_000_000:
            rows = max(1, 3_000_000 // hidden)
        with_delta = bool(rng.integers(2))
        h, d = r16(rng, rows, hidden), r16(rng, rows, hidden)
        w = (1 + 0.05 * rng.standard_normal(hidden)).astype(np.float16)
        eps = float(rng.choice([1e-6, 1e-5]))
        want_h, want_y = orc.add_rmsnorm_f16(h, d if with_delta else None, w, eps)
        gh, gy = Guarded(h), Guarded(np.zeros_like(h))
        if with_delta:
            st = vv.vvb_add_rmsnorm_dev(gh.ptr, dev(d), dev(w), gy.ptr, rows, hidden, eps)
        else:
            st = vv.vv_rmsnorm_dev(gh.ptr, dev(w), gy.ptr, rows, hidden, eps)
        assert st == 0, (case, rows, hidden, st)
        assert np.array_equal(bits(gh.get()), bits(want_h if with_delta else h)), (case, rows, hidden)
        assert orc.ulp_distance(gy.get(), want_y).max() <= 2, (case, rows, hidden)


def test_fuzz_rope(vv, orc):
    rng = np.random.default_rng(1002)
    for case in range(40):
        rows = int(rng.choice([1, 2, 3, 4, 5, 63, 64, 65, 257, 900]))
        nq, nkv = int(rng.integers(1, 33)), int(rng.integers(0, 9))
        hd = int(rng.choice([16, 32, 48, 64, 96, 128, 256, 30, 6]))       # 30 and 6: scalar path
        off = int(rng.choice([0, 1, 1000, 30000]))
        theta = float(rng.choice([1e4, 1e6]))
        q, k = r16(rng, rows, nq, hd), r16(rng, rows, max(nkv, 1), hd)
        gq, gk = Guarded(q), Guarded(k)
        by_device = bool(rng.integers(2))
        dpos = torch.tensor([off], dtype=torch.int32, device="cuda") if by_device else None
        st = vv.vvb_rope_qk_dev(gq.ptr, gk.ptr if nkv else None, rows, nq, nkv, hd, 0 if by_device else off, dpos, theta)
        assert st == 0, (case, rows, nq, nkv, hd, st)
        assert orc.rope_error_in_ulps(gq.get(), orc.rope_f16(q, off, theta), q).max() <= 2.0, (case, rows, nq, nkv, hd)
        if nkv:
            assert orc.rope_error_in_ulps(gk.get(), orc.rope_f16(k[:, :nkv], off, theta), k[:, :nkv]).max() <= 2.0
        else:
            assert np.array_equal(bits(gk.get()), bits(k))


def test_fuzz_swiglu_and_elementwise(vv, orc):
    rng = np.random.default_rng(1003)
    for case in range(30):
        n = int(rng.choice([1, 7, 8, 9, 2047, 2048, 2049, 18944, 18944 * 3 + 5, 300_001]))
        g, u = r16(rng, n, scale=2.0), r16(rng, n)
        out = Guarded(np.zeros(n, np.float16))
        in_place = bool(rng.integers(2))
        if in_place:
            gg = Guarded(g)
            assert vv.vv_swiglu_dev(gg.ptr, dev(u), gg.ptr, n) == 0
            got = gg.get()
        else:
            assert vv.vv_swiglu_dev(dev(g), dev(u), out.ptr, n) == 0
            got = out.get()
        assert orc.ulp_distance(got, orc.swiglu_f16(g, u)).max() <= 2, (case, n)
        # residual add: bit-exact
        x = Guarded(g)
        assert vv.vv_residual_add_dev(x.ptr, dev(u), n) == 0
        assert np.array_equal(bits(x.get()), bits(orc.residual_add_f16(g, u))), (case, n)
    for case in range(10):
        M, N = int(rng.integers(1, 200)), int(rng.choice([8, 64, 512, 3584, 100, 7]))
        y, b = r16(rng, M, N), r16(rng, N)
        gy = Guarded(y)
        assert vv.vv_bias_add_dev(gy.ptr, dev(b), M, N) == 0
        want = (y.astype(np.float32) + b.astype(np.float32)).astype(np.float16)
        assert np.array_equal(bits(gy.get()), bits(want)), (case, M, N)


def test_fuzz_int8_quantizers(vv, orc):
    from test_q8 import run_q, same
    rng = np.random.default_rng(1004)
    R = orc.restated()
    for case in range(24):
        M = int(rng.choice([1, 3, 64, 300, 591, 593]))
        K = int(rng.choice([256, 1536, 3584, 4096, 8192, 8224, 18944, 22528]))
        if M * K > 4_000_000:
            M = max(1, 4_000_000 // K)
        layout = int(rng.integers(4))
        x = r16(rng, M, K, scale=float(rng.choice([0.01, 1.0, 30.0])))
        if rng.integers(4) == 0:
            x[rng.integers(M)] = 0                                           # an all-zero row: scale 0, zeros out
        got = run_q(lambda q, s, u: vv.vv_act_quant_dev(dev(x), M, K, layout, q, s, u), M, K)
        assert same(got, R.quant_act_q8(x.astype(np.float32), layout)), (case, M, K, layout)
        if K <= 8192:                                                        # the norm kernel's register path and beyond
            w = (1 + 0.1 * rng.standard_normal(K)).astype(np.float16)
            got = run_q(lambda q, s, u: vv.vv_rmsnorm_q8_dev(dev(x), dev(w), M, K, 1e-6, layout, q, s, u), M, K)
            _, normed = orc.add_rmsnorm_f16(x, None, w, 1e-6)
            assert same(got, R.quant_act_q8(normed.astype(np.float32), layout)), (case, M, K, layout, "norm")
        up = r16(rng, M, K)
        got = run_q(lambda q, s, u: vv.vv_swiglu_q8_dev(dev(x), dev(up), M, K, layout, q, s, u), M, K)
        o = torch.empty(M, K, dtype=torch.float16, device="cuda")
        assert vv.vv_swiglu_dev(dev(x), dev(up), o, M * K) == 0
        torch.cuda.synchronize()
        assert same(got, R.quant_act_q8(o.cpu().numpy().astype(np.float32), layout)), (case, M, K, layout, "swiglu")


def test_fuzz_kv_append(vv, orc):
    rng = np.random.default_rng(1005)
    R = orc.restated()
    for case in range(30):
        nq, nkv = int(rng.integers(1, 33)), int(rng.integers(1, 9))
        hd = int(rng.choice([16, 32, 64, 128, 256]))
        rows = int(rng.choice([1, 2, 5, 64, 65, 200]))
        fmt = int(rng.integers(3))
        paged = bool(rng.integers(2))
        first = int(rng.choice([0, 3, 64, 100]))
        pos0 = int(rng.choice([0, 7, 5000]))
        width = nkv * hd
        q, k, v = r16(rng, rows, nq, hd), r16(rng, rows, nkv, hd, scale=1.5), r16(rng, rows, nkv, hd, scale=0.05)
        qb = r16(rng, nq, hd, scale=0.3) if rng.integers(2) else None
        kb = r16(rng, nkv, hd, scale=0.3) if rng.integers(2) else None
        vb = r16(rng, nkv, hd, scale=0.01) if rng.integers(2) else None
        kref = r16(rng, nkv, hd, scale=0.5) if (fmt and rng.integers(2)) else None
        n_pages = (first + rows + 63) // 64
        pool = n_pages + 3
        table = rng.permutation(pool)[:n_pages].astype(np.int32) if paged else None
        cache_rows = pool * 64 if paged else first + rows + 2
        dt, fill, np_dt = (torch.uint8, 0xA5, np.uint8) if fmt else (torch.int16, 0x1234, np.uint16)
        ks = torch.full((cache_rows, width), fill, dtype=dt, device="cuda")
        vs = torch.full((cache_rows, width), fill, dtype=dt, device="cuda")
        opt = lambda a: dev(a) if a is not None else None
        dq, dk, dv = dev(q), dev(k), dev(v)
        st = vv.vvb_kv_append_dev(dq, dk, dv, ks, vs, rows, nq, nkv, hd, q_bias=opt(qb), k_bias=opt(kb), v_bias=opt(vb),
                                  k_ref=opt(kref), page_table=opt(table), position_offset=pos0, cache_offset=first,
                                  kv_format=fmt, keep_k=1)
        tag = (case, nq, nkv, hd, rows, fmt, paged)
        assert st == 0, tag + (st,)
        torch.cuda.synchronize()
        add = lambda x, b: (x.astype(np.float32) + b.astype(np.float32)).astype(np.float16) if b is not None else x
        qq, kk, vvv = add(q, qb), add(k, kb), add(v, vb)
        assert orc.rope_error_in_ulps(dq.cpu().numpy(), orc.rope_f16(qq, pos0, 1e6), qq).max() <= 2.0, tag
        k_rot = dk.cpu().numpy()                                               # keep_k: the rotated K, in place
        assert orc.rope_error_in_ulps(k_rot, orc.rope_f16(kk, pos0, 1e6), kk).max() <= 2.0, tag
        if fmt:
            wk, wv = R.kv_store_fp8(k_rot, kref, fmt), R.kv_store_fp8(vvv, None, fmt)
        else:
            wk, wv = k_rot.reshape(rows, width).view(np.uint16), vvv.reshape(rows, width).view(np.uint16)
        want_k = np.full((cache_rows, width), fill, np_dt)
        want_v = np.full((cache_rows, width), fill, np_dt)
        for r in range(rows):
            t = first + r
            phys = int(table[t // 64]) * 64 + t % 64 if paged else t
            want_k[phys], want_v[phys] = wk[r], wv[r]
        assert np.array_equal(ks.cpu().numpy().view(np_dt), want_k), tag
        assert np.array_equal(vs.cpu().numpy().view(np_dt), want_v), tag
