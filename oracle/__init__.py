"""CPU checkers for the per-token layer kernels. TEST INFRASTRUCTURE ONLY.

Two libraries sit behind this module:

* ``liboracle.so``  -- our restatement of the reference's CPU arithmetic
  (``oracle/vvb_oracle.c``); always available once ``make -C oracle`` ran.
* ``_ref/libvvref_cpu.so`` -- the reference's own ``src/cpu/cpu_kernels.c``
  compiled unmodified; present where the reference was mounted at build time.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline
and ``--impl reference`` legs may import this package. The shipped library and
its Python binding never do.

All array arguments are numpy arrays. FP16 data is carried as ``np.float16``
(or ``np.uint16`` bit patterns); the reference CPU path works on FP32
activations, so the ``*_f16`` helpers widen exactly, run the FP32 op, and round
the result to FP16 with round-to-nearest-even -- the value an FP16 device
buffer would hold.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "liboracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libvvref_cpu.so")
REF_INT8_SO = os.path.join(_HERE, "_ref", "libvvref_int8.so")

_f32p = C.POINTER(C.c_float)
_u16p = C.POINTER(C.c_uint16)
_i32p = C.POINTER(C.c_int32)


def build(quiet: bool = True) -> None:
    """Compile liboracle.so (and _ref/ when the reference is mounted)."""
    subprocess.run(["make", "-C", _HERE], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def _ptr(a: np.ndarray, typ):
    assert a.flags["C_CONTIGUOUS"], "oracle arrays must be C-contiguous"
    return a.ctypes.data_as(typ)


def _as_u16(a: np.ndarray) -> np.ndarray:
    if a.dtype == np.float16:
        return a.view(np.uint16)
    assert a.dtype == np.uint16
    return a


class _Restated:
    """ctypes face of liboracle.so."""

    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build()
        self.lib = L = C.CDLL(ORACLE_SO)
        L.orc_half_to_float.restype = C.c_float
        L.orc_half_to_float.argtypes = [C.c_uint16]
        L.orc_float_to_half_rne.restype = C.c_uint16
        L.orc_float_to_half_rne.argtypes = [C.c_float]
        L.orc_rmsnorm.argtypes = [_f32p, _u16p, _f32p, C.c_int, C.c_int, C.c_float]
        L.orc_rope.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]
        L.orc_rope_inv_freq.argtypes = [_f32p, C.c_int, C.c_float]
        L.orc_swiglu.argtypes = [_f32p, _f32p, _f32p, C.c_size_t]
        L.orc_residual_add.argtypes = [_f32p, _f32p, C.c_size_t]
        L.orc_embedding.argtypes = [_u16p, _i32p, _f32p, C.c_int, C.c_int]
        L.orc_add_rmsnorm_f16.argtypes = [_u16p, _u16p, _u16p, _u16p, C.c_int, C.c_int, C.c_float]
        L.orc_rope_f16.argtypes = [_u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]
        L.orc_swiglu_f16.argtypes = [_u16p, _u16p, _u16p, C.c_size_t]
        L.orc_widen_f16.argtypes = [_u16p, _f32p, C.c_size_t]
        L.orc_round_f16.argtypes = [_f32p, _u16p, C.c_size_t]
        L.orc_threads.restype = C.c_int

    # --- FP32 ops (same signatures as the reference's vv_*_cpu) -------------
    def rmsnorm(self, x, w_f16, rows, n, eps):
        out = np.empty_like(x)
        st = self.lib.orc_rmsnorm(_ptr(x, _f32p), _ptr(_as_u16(w_f16), _u16p),
                                  _ptr(out, _f32p), rows, n, eps)
        assert st == 0, st
        return out

    def rope(self, x, rows, n_heads, head_dim, position_offset, theta):
        x = np.ascontiguousarray(x).copy()
        st = self.lib.orc_rope(_ptr(x, _f32p), rows, n_heads, head_dim,
                               position_offset, theta)
        assert st == 0, st
        return x

    def rope_inv_freq(self, head_dim, theta):
        out = np.empty(head_dim // 2, np.float32)
        self.lib.orc_rope_inv_freq(_ptr(out, _f32p), head_dim, theta)
        return out

    def swiglu(self, gate, up):
        out = np.empty_like(gate)
        st = self.lib.orc_swiglu(_ptr(gate, _f32p), _ptr(up, _f32p),
                                 _ptr(out, _f32p), gate.size)
        assert st == 0, st
        return out

    def residual_add(self, x, y):
        x = np.ascontiguousarray(x).copy()
        st = self.lib.orc_residual_add(_ptr(x, _f32p), _ptr(y, _f32p), x.size)
        assert st == 0, st
        return x

    def embedding(self, table_f16, ids, rows, hidden):
        out = np.empty((rows, hidden), np.float32)
        st = self.lib.orc_embedding(_ptr(_as_u16(table_f16), _u16p),
                                    _ptr(ids, _i32p), _ptr(out, _f32p), rows, hidden)
        assert st == 0, st
        return out

    def threads(self):
        return int(self.lib.orc_threads())

    def lm_head(self, x_f32, w_f16):
        """(logits float64 [V], token, value) for W[V,K] @ x[K], double accumulation."""
        L = self.lib
        L.orc_lm_head.argtypes = [_f32p, _u16p, C.c_int, C.c_int, C.POINTER(C.c_double), _i32p,
                                  C.POINTER(C.c_double)]
        V, K = w_f16.shape
        logits = np.empty(V, np.float64)
        tok, val = C.c_int32(), C.c_double()
        st = L.orc_lm_head(_ptr(np.ascontiguousarray(x_f32, dtype=np.float32), _f32p), _ptr(_as_u16(w_f16), _u16p),
                           V, K, logits.ctypes.data_as(C.POINTER(C.c_double)), C.byref(tok), C.byref(val))
        assert st == 0, st
        return logits, int(tok.value), float(val.value)

    def fp8_encode(self, x_f32, fmt):
        """The reference's software FP8 byte of each float (fmt 1 = E4M3, 2 = E5M2)."""
        L = self.lib
        L.orc_fp8_encode.restype = C.c_uint8
        L.orc_fp8_encode.argtypes = [C.c_float, C.c_int]
        flat = np.ascontiguousarray(x_f32, dtype=np.float32).reshape(-1)
        return np.array([L.orc_fp8_encode(float(v), int(fmt)) for v in flat], np.uint8).reshape(np.shape(x_f32))

    def fp8_decode(self, codes, fmt):
        L = self.lib
        L.orc_fp8_decode.restype = C.c_float
        L.orc_fp8_decode.argtypes = [C.c_uint8, C.c_int]
        flat = np.ascontiguousarray(codes, dtype=np.uint8).reshape(-1)
        return np.array([L.orc_fp8_decode(int(v), int(fmt)) for v in flat], np.float32).reshape(np.shape(codes))

    def kv_store_fp8(self, x_f16, ref_f16, fmt, first_row=0, out=None):
        """FP16 [n_pos, width] (minus ref [width], in float) -> FP8 bytes written to rows
        first_row.. of `out` (uint8 [max_len, width]; allocated [first_row + n_pos, width] if None)."""
        L = self.lib
        L.orc_kv_store_fp8.argtypes = [_u16p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        x = _as_u16(x_f16)
        n_pos, width = x.shape[0], int(np.prod(x.shape[1:]))
        if out is None:
            out = np.zeros((first_row + n_pos, width), np.uint8)
        r = _as_u16(ref_f16) if ref_f16 is not None else None
        st = L.orc_kv_store_fp8(_ptr(x, _u16p), r.ctypes.data if r is not None else None, n_pos, width,
                                int(first_row), int(fmt), out.ctypes.data)
        assert st == 0, st
        return out

    # --- TurboQuant KV formats (fmt 3..6 = 4, 3, 2, 1.5 bits per value) --------
    def tq_bytes_per_vec(self, fmt):
        self.lib.orc_tq_bytes_per_vec.argtypes = [C.c_int]
        return int(self.lib.orc_tq_bytes_per_vec(int(fmt)))

    def tq_rotate(self, x_f32):
        """Sign flips + 128-point Walsh-Hadamard transform + 1/sqrt(128), on the last axis (128)."""
        self.lib.orc_tq_rotate128.argtypes = [_f32p]
        out = np.ascontiguousarray(x_f32, dtype=np.float32).copy()
        flat = out.reshape(-1, 128)
        for r in flat:
            self.lib.orc_tq_rotate128(r.ctypes.data_as(_f32p))
        return out

    def kv_rotate_f16(self, x_f16, inverse=False):
        """vv_kv_rotate_dev (inverse: vv_kv_unrotate_dev) on FP16 [..., 128]; returns a new array."""
        self.lib.orc_kv_rotate_f16.argtypes = [_u16p, C.c_size_t, C.c_int]
        out = np.ascontiguousarray(x_f16, dtype=np.float16).copy()
        assert out.shape[-1] == 128
        u = _as_u16(out)
        assert self.lib.orc_kv_rotate_f16(u.ctypes.data_as(_u16p), out.size // 128, int(bool(inverse))) == 0
        return out

    def kv_store_tq(self, x_f16, ref_f16, fmt, first_row=0, store=None, meta=None):
        """FP16 [n_pos, n_heads, 128] (minus ref [n_heads, 128], in float) -> (codes uint8
        [first_row + n_pos, n_heads * bytes_per_vec], sigma float16 [first_row + n_pos, n_heads]);
        rows first_row.. are written into `store` / `meta` when given."""
        L = self.lib
        L.orc_kv_store_tq.argtypes = [_u16p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        x = _as_u16(np.ascontiguousarray(x_f16))
        n_pos, n_heads, hd = x.shape
        assert hd == 128
        bpv = self.tq_bytes_per_vec(fmt)
        if store is None:
            store = np.zeros((first_row + n_pos, n_heads * bpv), np.uint8)
        if meta is None:
            meta = np.zeros((first_row + n_pos, n_heads), np.float16)
        r = _as_u16(np.ascontiguousarray(ref_f16)) if ref_f16 is not None else None
        st = L.orc_kv_store_tq(_ptr(x, _u16p), r.ctypes.data if r is not None else None, n_pos, n_heads,
                               int(first_row), int(fmt), store.ctypes.data, meta.ctypes.data)
        assert st == 0, st
        return store, meta

    def kv_load_tq(self, vec_bytes, sigma_f16, fmt):
        """One stored vector back to its 128 ROTATED-domain values (sigma * level[code])."""
        L = self.lib
        L.orc_kv_load_tq.argtypes = [C.c_void_p, C.c_uint16, C.c_int, _f32p]
        vec = np.ascontiguousarray(vec_bytes, dtype=np.uint8)
        out = np.empty(128, np.float32)
        sig = int(np.array([sigma_f16], np.float16).view(np.uint16)[0])
        st = L.orc_kv_load_tq(vec.ctypes.data, sig, int(fmt), _ptr(out, _f32p))
        assert st == 0, st
        return out

    def quant_act_q8(self, x_f32, layout, want_xsum=True):
        """Per-token int8 quantizer on FP32 rows [M, K]: (xq int8 [M,K],
        sx float32 [M], xsum int32 [M, K/32] or None)."""
        L = self.lib
        L.orc_quant_act_q8.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_void_p, _f32p, C.c_void_p]
        M, K = x_f32.shape
        xq = np.empty((M, K), np.int8)
        sx = np.empty(M, np.float32)
        xsum = np.empty((M, K // 32), np.int32) if want_xsum else None
        st = L.orc_quant_act_q8(_ptr(np.ascontiguousarray(x_f32), _f32p), M, K, int(layout), xq.ctypes.data,
                                _ptr(sx, _f32p), xsum.ctypes.data if want_xsum else None)
        assert st == 0, st
        return xq, sx, xsum


class _ReferenceInt8:
    """The reference's own quantizer, vv_quant_act_q8_cpu
    (src/cpu/cpu_int8.c:181-194), compiled unmodified."""

    def __init__(self):
        self.lib = C.CDLL(REF_INT8_SO)
        self.lib.vv_quant_act_q8_cpu.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_void_p, _f32p, C.c_void_p]

    def quant_act_q8(self, x_f32, layout, want_xsum=True):
        M, K = x_f32.shape
        xq = np.empty((M, K), np.int8)
        sx = np.empty(M, np.float32)
        xsum = np.empty((M, K // 32), np.int32) if want_xsum else None
        st = self.lib.vv_quant_act_q8_cpu(_ptr(np.ascontiguousarray(x_f32), _f32p), M, K, int(layout),
                                          xq.ctypes.data, _ptr(sx, _f32p), xsum.ctypes.data if want_xsum else None)
        assert st == 0, st
        return xq, sx, xsum


class _Reference:
    """ctypes face of the reference's compiled CPU kernels
    (include/vibevoice/cpu_kernels.h:27-37,160-171)."""

    def __init__(self):
        self.lib = L = C.CDLL(REF_SO)
        L.vv_rmsnorm_cpu.argtypes = [_f32p, C.c_void_p, _f32p, C.c_int, C.c_int, C.c_float]
        L.vv_rope_cpu.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]
        L.vv_swiglu_cpu.argtypes = [_f32p, _f32p, _f32p, C.c_int]
        L.vv_residual_add_cpu.argtypes = [_f32p, _f32p, C.c_int]
        L.vv_embedding_cpu.argtypes = [C.c_void_p, _i32p, _f32p, C.c_int, C.c_int]
        L.vv_cpu_threads.restype = C.c_int
        L.vv_cpu_physical_cores.restype = C.c_int
        L.vv_cpu_simd_name.restype = C.c_char_p

    def rmsnorm(self, x, w_f16, rows, n, eps):
        out = np.empty_like(x)
        w = _as_u16(w_f16)
        st = self.lib.vv_rmsnorm_cpu(_ptr(x, _f32p), w.ctypes.data, _ptr(out, _f32p),
                                     rows, n, eps)
        assert st == 0, st
        return out

    def rope(self, x, rows, n_heads, head_dim, position_offset, theta):
        x = np.ascontiguousarray(x).copy()
        st = self.lib.vv_rope_cpu(_ptr(x, _f32p), rows, n_heads, head_dim,
                                  position_offset, theta)
        assert st == 0, st
        return x

    def swiglu(self, gate, up):
        out = np.empty_like(gate)
        st = self.lib.vv_swiglu_cpu(_ptr(gate, _f32p), _ptr(up, _f32p),
                                    _ptr(out, _f32p), gate.size)
        assert st == 0, st
        return out

    def residual_add(self, x, y):
        x = np.ascontiguousarray(x).copy()
        st = self.lib.vv_residual_add_cpu(_ptr(x, _f32p), _ptr(y, _f32p), x.size)
        assert st == 0, st
        return x

    def embedding(self, table_f16, ids, rows, hidden):
        out = np.empty((rows, hidden), np.float32)
        t = _as_u16(table_f16)
        st = self.lib.vv_embedding_cpu(t.ctypes.data, _ptr(ids, _i32p),
                                       _ptr(out, _f32p), rows, hidden)
        assert st == 0, st
        return out

    def lm_head_argmax(self, x_f32, w_f16):
        """vv_lm_head_argmax_cpu (src/cpu/cpu_kernels.c:1570): (token, value)."""
        L = self.lib
        L.vv_lm_head_argmax_cpu.argtypes = [_f32p, C.c_void_p, C.c_int, C.c_int, _i32p, _f32p]
        V, K = w_f16.shape
        tok, val = C.c_int32(), C.c_float()
        st = L.vv_lm_head_argmax_cpu(_ptr(np.ascontiguousarray(x_f32, dtype=np.float32), _f32p),
                                     _as_u16(w_f16).ctypes.data, V, K, C.byref(tok), C.byref(val))
        assert st == 0, st
        return int(tok.value), float(val.value)

    def threads(self):
        """Sets the OpenMP team to the physical cores and pins it
        (src/cpu/cpu_kernels.c:303-327). Pins the calling thread too."""
        return int(self.lib.vv_cpu_threads())

    def physical_cores(self):
        return int(self.lib.vv_cpu_physical_cores())

    def simd_name(self):
        return self.lib.vv_cpu_simd_name().decode()


_restated = None
_reference = None


def restated() -> _Restated:
    global _restated
    if _restated is None:
        _restated = _Restated()
    return _restated


def have_reference() -> bool:
    return os.path.exists(REF_SO)


def have_reference_int8() -> bool:
    return os.path.exists(REF_INT8_SO)


def reference_int8() -> _ReferenceInt8:
    return _ReferenceInt8()


def reference() -> _Reference:
    global _reference
    if _reference is None:
        _reference = _Reference()
    return _reference


# --- FP16-boundary composites (what an FP16 device buffer would hold) --------

def widen(a_f16: np.ndarray) -> np.ndarray:
    return a_f16.astype(np.float32)


def round_f16(a_f32: np.ndarray) -> np.ndarray:
    """float32 -> float16, round to nearest even (numpy's cast does RNE)."""
    with np.errstate(over="ignore"):
        return a_f32.astype(np.float16)


def add_rmsnorm_f16(hidden, delta, gamma, eps, impl=None):
    """Residual add then RMSNorm as the engine's FP16 buffers see it
    (src/inference/decoder.c:950-958): returns (hidden', normed), with
    hidden' = f16(hidden + delta) and normed = f16(rmsnorm(hidden')).
    ``delta`` None = plain RMSNorm (hidden' is hidden)."""
    impl = impl or restated()
    rows, n = hidden.shape
    h = widen(hidden)
    if delta is not None:
        h = impl.residual_add(h, widen(delta))
        hidden_new = round_f16(h)
        h = widen(hidden_new)
    else:
        hidden_new = hidden.copy()
    y = impl.rmsnorm(h, gamma, rows, n, np.float32(eps))
    return hidden_new, round_f16(y)


def rope_f16(x, position_offset, theta, impl=None):
    impl = impl or restated()
    rows, n_heads, head_dim = x.shape
    return round_f16(impl.rope(widen(x), rows, n_heads, head_dim,
                               int(position_offset), np.float32(theta)))


def swiglu_f16(gate, up, impl=None):
    impl = impl or restated()
    g = widen(np.ascontiguousarray(gate)).reshape(-1)
    u = widen(np.ascontiguousarray(up)).reshape(-1)
    return round_f16(impl.swiglu(g, u)).reshape(gate.shape)


def embedding_f16(table, ids, impl=None):
    """Gathered rows as FP16: the widening is exact, so rounding back returns
    the table's own bits -- the gather is compared bit for bit."""
    impl = impl or restated()
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    return round_f16(impl.embedding(table, ids, ids.size, table.shape[1]))


def residual_add_f16(x, y, impl=None):
    impl = impl or restated()
    return round_f16(impl.residual_add(widen(x).reshape(-1), widen(y).reshape(-1))).reshape(x.shape)


# --- comparison helpers -------------------------------------------------------

def f16_ordinal(a: np.ndarray) -> np.ndarray:
    """Map FP16 bit patterns onto a monotone integer line (-0 and +0 coincide),
    so |ordinal(a) - ordinal(b)| counts representable values between a and b."""
    u = _as_u16(np.ascontiguousarray(a)).astype(np.int32)
    mag = u & 0x7FFF
    return np.where(u & 0x8000, -mag, mag)


def ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Pure FP16 ulp distance, elementwise. NaN pairs count as 0 when both are
    NaN and as a large number when only one is."""
    af = a.astype(np.float32)
    bf = b.astype(np.float32)
    d = np.abs(f16_ordinal(a) - f16_ordinal(b))
    an, bn = np.isnan(af), np.isnan(bf)
    d = np.where(an & bn, 0, d)
    d = np.where(an ^ bn, 1 << 20, d)
    return d


def f16_ulp_of(mag: np.ndarray) -> np.ndarray:
    """Size of one FP16 ulp at magnitude ``mag`` (float32 array): 2^(e-10) for
    normals, 2^-24 in the subnormal range."""
    mag = np.abs(mag.astype(np.float32))
    e = np.floor(np.log2(np.maximum(mag, np.float32(2.0 ** -14))))
    return np.exp2(e - 10).astype(np.float32)


def rope_error_in_ulps(got, want, x_in):
    """|got - want| in units of the FP16 ulp at operand scale
    max(|x0|, |x1|, |want|): the rotation a*c - b*s cancels, so the distance
    between bit patterns of a near-zero result says nothing about accuracy."""
    rows, n_heads, head_dim = x_in.shape
    half = head_dim // 2
    xin = np.abs(x_in.astype(np.float32))
    pair = np.maximum(xin[..., :half], xin[..., half:])
    scale = np.concatenate([pair, pair], axis=-1)
    scale = np.maximum(scale, np.abs(want.astype(np.float32)))
    err = np.abs(got.astype(np.float32) - want.astype(np.float32))
    return err / f16_ulp_of(scale)
