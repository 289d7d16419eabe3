"""vvb200 -- Python face of libvvb200 (ctypes over the C-ABI in include/vvb200.h).

The functions carry the reference's op names and argument order
(include/vibevoice/device.h:486-514): ``vv_rmsnorm_dev(input, weight, output,
seq_len, hidden_size, eps, stream)`` and so on, and return the same status
codes. A tensor argument may be a ``torch.Tensor`` on a CUDA device (its
``data_ptr()`` is passed) or a raw integer device address; ``stream`` may be a
``torch.cuda.Stream``, a raw ``cudaStream_t`` integer, or None for torch's
current stream. torch is used for device memory and streams only -- every
computation happens in the library's own kernels, and importing this package
fails loudly if the library is missing: there is no fallback.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libvvb200.so")

VV_OK = 0
VV_ERR_INVALID_ARG = -1
VV_ERR_NULL_PTR = -2
VV_ERR_OUT_OF_MEMORY = -3
VV_ERR_UNSUPPORTED = -7
VV_ERR_OVERFLOW = -8
VV_ERR_CUDA = -100
VV_ERR_CUDA_OOM = -101
VV_ERR_CUDA_LAUNCH = -102


class VvbError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(f"{what}: status {status} ({status_string(status)})")


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `make -C {os.path.dirname(_HERE)}` "
            "(there is no fallback implementation)")
    return C.CDLL(LIB_PATH)


_lib = _load()

_vp, _i, _f, _sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t


class LayerChain(C.Structure):
    """vvb_layer_chain_t (include/vvb200.h)."""
    _fields_ = [
        ("hidden", _vp), ("delta", _vp), ("norm_w", _vp), ("normed", _vp),
        ("q", _vp), ("k", _vp), ("gate", _vp), ("up", _vp),
        ("rows", _i), ("hidden_size", _i), ("n_q_heads", _i), ("n_kv_heads", _i),
        ("head_dim", _i), ("inter", _i), ("position_offset", _i),
        ("eps", _f), ("theta", _f),
    ]


class KvAppend(C.Structure):
    """vvb_kv_append_t (include/vvb200.h)."""
    _fields_ = [
        ("q", _vp), ("k", _vp), ("v", _vp), ("q_bias", _vp), ("k_bias", _vp), ("v_bias", _vp),
        ("k_store", _vp), ("v_store", _vp), ("k_ref", _vp), ("page_table", _vp), ("d_position", _vp),
        ("rows", _i), ("n_q_heads", _i), ("n_kv_heads", _i), ("head_dim", _i),
        ("position_offset", _i), ("cache_offset", _i), ("theta", _f), ("kv_format", _i), ("keep_k", _i),
        ("k_meta", _vp), ("v_meta", _vp),
    ]


# name -> (restype, argtypes): every symbol include/vvb200.h declares
SIGNATURES = {
    "vvb_kv_append_dev": (_i, [C.POINTER(KvAppend), _vp]),
    "vvb_kv_rotate_dev": (_i, [_vp, _i, _i, _i, _vp]),
    "vvb_kv_unrotate_dev": (_i, [_vp, _i, _i, _i, _vp]),
    "vv_embedding_dev": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "vv_rmsnorm_dev": (_i, [_vp, _vp, _vp, _i, _i, _f, _vp]),
    "vv_rope_dev": (_i, [_vp, _i, _i, _i, _i, _vp, _f, _vp]),
    "vv_swiglu_dev": (_i, [_vp, _vp, _vp, _i, _vp]),
    "vv_swiglu_fused_dev": (_i, [_vp, _vp, _i, _i, _vp]),
    "vv_residual_add_dev": (_i, [_vp, _vp, _i, _vp]),
    "vv_bias_add_dev": (_i, [_vp, _vp, _i, _i, _vp]),
    "vv_fp32_to_fp16_dev": (_i, [_vp, _vp, _i, _vp]),
    "vv_fp16_to_fp32_dev": (_i, [_vp, _vp, _i, _vp]),
    "vv_act_quant_dev": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "vv_rmsnorm_q8_dev": (_i, [_vp, _vp, _i, _i, _f, _i, _vp, _vp, _vp, _vp]),
    "vv_swiglu_q8_dev": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "vvb_add_rmsnorm_q8_dev": (_i, [_vp, _vp, _vp, _i, _i, _f, _i, _vp, _vp, _vp, _vp]),
    "vv_col_absmax_dev": (_i, [_vp, _i, _i, _vp, _vp]),
    "vv_lm_head_gemv_dev": (_i, [_vp, _vp, _vp, _i, _i, _vp]),
    "vv_argmax_dev": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp]),
    "vvb_lm_head_scratch_bytes": (_sz, [_i]),
    "vvb_lm_head_argmax_dev": (_i, [_vp, _vp, _f, _vp, _i, _i, _vp, _vp, _sz, _vp, _vp, _vp]),
    "vvb_lm_head_argmax_static_dev": (_i, [_vp, _vp, _f, _vp, _i, _i, _vp, _vp, _vp, _vp]),
    "vvb_add_rmsnorm_dev": (_i, [_vp, _vp, _vp, _vp, _i, _i, _f, _vp]),
    "vvb_rope_qk_dev": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _vp, _f, _vp]),
    "vvb_embedding_rmsnorm_dev": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp]),
    "vvb_rope_qk_append_dev": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _f, _i, _vp]),
    "vvb_rope_qk_append_fp8_dev": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _f,
                                        _i, _i, _vp]),
    "vvb_swiglu_dev": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "vvb_residual_add_dev": (_i, [_vp, _vp, _sz, _vp]),
    "vvb_layer_chain_dev": (_i, [C.POINTER(LayerChain), _vp]),
    "vvb_shard_rows": (_i, [C.c_int64, _i, _i, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "vvb_host_ctx_create": (_i, [C.POINTER(_vp), _i, _i, _i, _i, _i, _i, _i]),
    "vvb_host_ctx_destroy": (None, [_vp]),
    "vvb_layer_chain_host": (_i, [_vp, C.POINTER(LayerChain)]),
    "vvb_host_ctx_last_traffic": (None, [_vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "vvb_host_ctx_last_ms": (C.c_float, [_vp]),
    "vvb_host_multi_create": (_i, [C.POINTER(_vp), C.POINTER(_i), _i, _i, _i, _i, _i, _i, _i]),
    "vvb_host_multi_destroy": (None, [_vp]),
    "vvb_host_multi_devices": (_i, [_vp]),
    "vvb_layer_chain_host_multi": (_i, [_vp, C.POINTER(LayerChain)]),
    "vvb_host_multi_last_ms": (C.c_float, [_vp]),
    "vvb_host_multi_last_traffic": (None, [_vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "vvb_version": (C.c_char_p, []),
    "vvb_status_string": (C.c_char_p, [_i]),
    "vvb_launch_count": (C.c_uint64, []),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(_lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def _ptr(t):
    """Device address of a tensor argument (None -> NULL)."""
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


def _stream(s):
    if s is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    if isinstance(s, int):
        return s
    return s.cuda_stream


def version() -> str:
    return _lib.vvb_version().decode()


def status_string(status: int) -> str:
    return _lib.vvb_status_string(int(status)).decode()


def launch_count() -> int:
    return int(_lib.vvb_launch_count())


def check(status: int, what: str = "vvb200") -> None:
    if status != VV_OK:
        raise VvbError(status, what)


# ------------------------------------------------------------------ group 1
def vv_embedding_dev(table, ids, output, seq_len, hidden_size, stream=None) -> int:
    return _lib.vv_embedding_dev(_ptr(table), _ptr(ids), _ptr(output), seq_len, hidden_size, _stream(stream))


def vv_rmsnorm_dev(input, weight, output, seq_len, hidden_size, eps, stream=None) -> int:
    return _lib.vv_rmsnorm_dev(_ptr(input), _ptr(weight), _ptr(output), seq_len, hidden_size, eps, _stream(stream))


def vv_rope_dev(x, seq_len, n_heads, head_dim, position_offset, d_position, theta, stream=None) -> int:
    return _lib.vv_rope_dev(_ptr(x), seq_len, n_heads, head_dim, position_offset, _ptr(d_position), theta,
                            _stream(stream))


def vv_swiglu_dev(gate, up, output, n_elements, stream=None) -> int:
    return _lib.vv_swiglu_dev(_ptr(gate), _ptr(up), _ptr(output), n_elements, _stream(stream))


def vv_swiglu_fused_dev(gate_up, output, rows, inter, stream=None) -> int:
    return _lib.vv_swiglu_fused_dev(_ptr(gate_up), _ptr(output), rows, inter, _stream(stream))


def vv_residual_add_dev(x, y, total, stream=None) -> int:
    return _lib.vv_residual_add_dev(_ptr(x), _ptr(y), total, _stream(stream))


def vv_bias_add_dev(output, bias, M, N, stream=None) -> int:
    return _lib.vv_bias_add_dev(_ptr(output), _ptr(bias), M, N, _stream(stream))


def vv_fp32_to_fp16_dev(in_fp32, out_fp16, n, stream=None) -> int:
    return _lib.vv_fp32_to_fp16_dev(_ptr(in_fp32), _ptr(out_fp16), n, _stream(stream))


def vv_fp16_to_fp32_dev(in_fp16, out_fp32, n, stream=None) -> int:
    return _lib.vv_fp16_to_fp32_dev(_ptr(in_fp16), _ptr(out_fp32), n, _stream(stream))


# per-token int8 activations (include/vibevoice/device.h:297-331)
VV_Q8_NATURAL, VV_Q8_NIBBLE, VV_Q8_W4_GEMV, VV_Q8_W4_MMA = 0, 1, 2, 3
VV_ACT_QUANT_MAX_K, VV_ACT_QUANT_MIN_K = 22528, 256


def vv_act_quant_dev(x, M, K, layout, xq, sx, xsum, stream=None) -> int:
    return _lib.vv_act_quant_dev(_ptr(x), M, K, layout, _ptr(xq), _ptr(sx), _ptr(xsum), _stream(stream))


def vv_rmsnorm_q8_dev(x, weight, M, K, eps, layout, xq, sx, xsum, stream=None) -> int:
    return _lib.vv_rmsnorm_q8_dev(_ptr(x), _ptr(weight), M, K, eps, layout, _ptr(xq), _ptr(sx), _ptr(xsum),
                                  _stream(stream))


def vv_swiglu_q8_dev(gate, up, M, K, layout, xq, sx, xsum, stream=None) -> int:
    return _lib.vv_swiglu_q8_dev(_ptr(gate), _ptr(up), M, K, layout, _ptr(xq), _ptr(sx), _ptr(xsum),
                                 _stream(stream))


def vvb_add_rmsnorm_q8_dev(hidden_inout, delta, weight, M, K, eps, layout, xq, sx, xsum, stream=None) -> int:
    return _lib.vvb_add_rmsnorm_q8_dev(_ptr(hidden_inout), _ptr(delta), _ptr(weight), M, K, eps, layout,
                                       _ptr(xq), _ptr(sx), _ptr(xsum), _stream(stream))


def vv_lm_head_gemv_dev(x, W, logits, V, K, stream=None) -> int:
    return _lib.vv_lm_head_gemv_dev(_ptr(x), _ptr(W), _ptr(logits), V, K, _stream(stream))


def vv_argmax_dev(logits, V, scratch_v, scratch_i, out_token, out_value, stream=None) -> int:
    return _lib.vv_argmax_dev(_ptr(logits), V, _ptr(scratch_v), _ptr(scratch_i), _ptr(out_token), _ptr(out_value),
                              _stream(stream))


def vvb_lm_head_scratch_bytes(V: int) -> int:
    return int(_lib.vvb_lm_head_scratch_bytes(V))


def vvb_lm_head_argmax_dev(x, final_norm_w, eps, W, V, K, logits, scratch, scratch_bytes, out_token, out_value,
                           stream=None) -> int:
    return _lib.vvb_lm_head_argmax_dev(_ptr(x), _ptr(final_norm_w), eps, _ptr(W), V, K, _ptr(logits), _ptr(scratch),
                                       scratch_bytes, _ptr(out_token), _ptr(out_value), _stream(stream))


VVB_LM_HEAD_STATIC_MAX_V = 262144


def vvb_lm_head_argmax_static_dev(x, final_norm_w, eps, W, V, K, logits, out_token, out_value, stream=None) -> int:
    """The fused head + argmax with its scratch inside the library (no device
    memory from the caller, none allocated); V <= VVB_LM_HEAD_STATIC_MAX_V.
    Calls on one GPU must not overlap: they share that scratch."""
    return _lib.vvb_lm_head_argmax_static_dev(_ptr(x), _ptr(final_norm_w), eps, _ptr(W), V, K, _ptr(logits),
                                              _ptr(out_token), _ptr(out_value), _stream(stream))


def vv_col_absmax_dev(x, M, K, acc, stream=None) -> int:
    return _lib.vv_col_absmax_dev(_ptr(x), M, K, _ptr(acc), _stream(stream))


# ------------------------------------------------------------------ group 2
def vvb_add_rmsnorm_dev(hidden_inout, delta, weight, normed_out, rows, hidden_size, eps, stream=None) -> int:
    return _lib.vvb_add_rmsnorm_dev(_ptr(hidden_inout), _ptr(delta), _ptr(weight), _ptr(normed_out),
                                    rows, hidden_size, eps, _stream(stream))


def vvb_rope_qk_dev(q, k, rows, n_q_heads, n_kv_heads, head_dim, position_offset, d_position, theta,
                    stream=None) -> int:
    return _lib.vvb_rope_qk_dev(_ptr(q), _ptr(k), rows, n_q_heads, n_kv_heads, head_dim, position_offset,
                                _ptr(d_position), theta, _stream(stream))


def vvb_rope_qk_append_dev(q, k, v, q_bias, k_bias, v_bias, k_cache, v_cache, rows, n_q_heads, n_kv_heads, head_dim,
                           position_offset, cache_offset, d_position, theta, keep_k=0, stream=None) -> int:
    return _lib.vvb_rope_qk_append_dev(_ptr(q), _ptr(k), _ptr(v), _ptr(q_bias), _ptr(k_bias), _ptr(v_bias),
                                       _ptr(k_cache), _ptr(v_cache), rows, n_q_heads, n_kv_heads, head_dim,
                                       position_offset, cache_offset, _ptr(d_position), theta, keep_k,
                                       _stream(stream))


VVB_KV_FP16, VVB_KV_FP8_E4M3, VVB_KV_FP8_E5M2 = 0, 1, 2
VVB_KV_TQ4, VVB_KV_TQ3, VVB_KV_TQ2, VVB_KV_TQ1_5 = 3, 4, 5, 6


def vvb_kv_append_dev(q, k, v, k_store, v_store, rows, n_q_heads, n_kv_heads, head_dim, *, q_bias=None, k_bias=None,
                      v_bias=None, k_ref=None, page_table=None, d_position=None, position_offset=0, cache_offset=0,
                      theta=1e6, kv_format=0, keep_k=0, k_meta=None, v_meta=None, stream=None) -> int:
    """Bias adds + RoPE + KV-cache append (FP16, FP8 or TurboQuant; contiguous or paged) in one launch."""
    a = KvAppend(_ptr(q), _ptr(k), _ptr(v), _ptr(q_bias), _ptr(k_bias), _ptr(v_bias), _ptr(k_store), _ptr(v_store),
                 _ptr(k_ref), _ptr(page_table), _ptr(d_position), rows, n_q_heads, n_kv_heads, head_dim,
                 position_offset, cache_offset, theta, kv_format, keep_k, _ptr(k_meta), _ptr(v_meta))
    return _lib.vvb_kv_append_dev(C.byref(a), _stream(stream))


def vvb_kv_rotate_dev(x, n_heads, head_dim, rows, stream=None) -> int:
    """Q before attention over a TurboQuant cache: sign pattern, 128-point Hadamard transform, 1/sqrt(128); in place."""
    return _lib.vvb_kv_rotate_dev(_ptr(x), n_heads, head_dim, rows, _stream(stream))


def vvb_kv_unrotate_dev(x, n_heads, head_dim, rows, stream=None) -> int:
    """The attention output after it: the inverse of vvb_kv_rotate_dev; in place."""
    return _lib.vvb_kv_unrotate_dev(_ptr(x), n_heads, head_dim, rows, _stream(stream))


def vvb_rope_qk_append_fp8_dev(q, k, v, q_bias, k_bias, v_bias, k_store, v_store, k_ref, rows, n_q_heads,
                               n_kv_heads, head_dim, position_offset, cache_offset, d_position, theta, kv_format,
                               keep_k=0, stream=None) -> int:
    return _lib.vvb_rope_qk_append_fp8_dev(_ptr(q), _ptr(k), _ptr(v), _ptr(q_bias), _ptr(k_bias), _ptr(v_bias),
                                           _ptr(k_store), _ptr(v_store), _ptr(k_ref), rows, n_q_heads,
                                           n_kv_heads, head_dim, position_offset, cache_offset,
                                           _ptr(d_position), theta, kv_format, keep_k, _stream(stream))


def vvb_embedding_rmsnorm_dev(table, ids, hidden_out, weight, normed_out, rows, hidden_size, vocab, eps,
                              stream=None) -> int:
    return _lib.vvb_embedding_rmsnorm_dev(_ptr(table), _ptr(ids), _ptr(hidden_out), _ptr(weight),
                                          _ptr(normed_out), rows, hidden_size, vocab, eps, _stream(stream))


def vvb_swiglu_dev(gate, up, output, n_elements, stream=None) -> int:
    return _lib.vvb_swiglu_dev(_ptr(gate), _ptr(up), _ptr(output), n_elements, _stream(stream))


def vvb_residual_add_dev(x, y, total, stream=None) -> int:
    return _lib.vvb_residual_add_dev(_ptr(x), _ptr(y), total, _stream(stream))


def make_chain(hidden, delta, norm_w, normed, q, k, gate, up, rows, hidden_size, n_q_heads, n_kv_heads,
               head_dim, inter, position_offset=0, eps=1e-6, theta=1e6) -> LayerChain:
    """Fill a vvb_layer_chain_t from tensors (device tensors for
    vvb_layer_chain_dev, pinned host tensors for HostPipeline.run)."""
    return LayerChain(_ptr(hidden), _ptr(delta), _ptr(norm_w), _ptr(normed), _ptr(q), _ptr(k), _ptr(gate),
                      _ptr(up), rows, hidden_size, n_q_heads, n_kv_heads, head_dim, inter, position_offset,
                      eps, theta)


def vvb_layer_chain_dev(chain: LayerChain, stream=None) -> int:
    return _lib.vvb_layer_chain_dev(C.byref(chain), _stream(stream))


def vvb_shard_rows(total_rows: int, parts: int, part: int):
    """(first, count) of the contiguous row block that `part` of `parts` owns."""
    first, count = C.c_int64(), C.c_int64()
    check(_lib.vvb_shard_rows(total_rows, parts, part, C.byref(first), C.byref(count)), "vvb_shard_rows")
    return first.value, count.value


class HostPipeline:
    """vvb_host_ctx_t: runs the layer chain on tensors that live in (pinned)
    host memory, overlapping uploads, kernels and downloads slice by slice."""

    def __init__(self, device, max_slice_rows, hidden_size, n_q_heads, n_kv_heads, head_dim, inter):
        self._ctx = _vp()
        check(_lib.vvb_host_ctx_create(C.byref(self._ctx), device, max_slice_rows, hidden_size, n_q_heads,
                                       n_kv_heads, head_dim, inter), "vvb_host_ctx_create")

    def run(self, chain: LayerChain) -> int:
        return _lib.vvb_layer_chain_host(self._ctx, C.byref(chain))

    def last_traffic(self):
        a, b = C.c_uint64(), C.c_uint64()
        _lib.vvb_host_ctx_last_traffic(self._ctx, C.byref(a), C.byref(b))
        return a.value, b.value

    def last_ms(self) -> float:
        return float(_lib.vvb_host_ctx_last_ms(self._ctx))

    def close(self):
        if self._ctx:
            _lib.vvb_host_ctx_destroy(self._ctx)
            self._ctx = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class HostPipelineMulti:
    """vvb_host_multi_t: HostPipeline on several GPUs of one box, one host thread
    per device inside the library; rows are sharded with vvb_shard_rows."""

    def __init__(self, devices, max_slice_rows, hidden_size, n_q_heads, n_kv_heads, head_dim, inter):
        devices = list(devices)
        arr = (_i * len(devices))(*devices)
        self._ctx = _vp()
        check(_lib.vvb_host_multi_create(C.byref(self._ctx), arr, len(devices), max_slice_rows, hidden_size,
                                         n_q_heads, n_kv_heads, head_dim, inter), "vvb_host_multi_create")

    def run(self, chain: LayerChain) -> int:
        return _lib.vvb_layer_chain_host_multi(self._ctx, C.byref(chain))

    def devices(self) -> int:
        return int(_lib.vvb_host_multi_devices(self._ctx))

    def last_traffic(self):
        a, b = C.c_uint64(), C.c_uint64()
        _lib.vvb_host_multi_last_traffic(self._ctx, C.byref(a), C.byref(b))
        return a.value, b.value

    def last_ms(self) -> float:
        return float(_lib.vvb_host_multi_last_ms(self._ctx))

    def close(self):
        if self._ctx:
            _lib.vvb_host_multi_destroy(self._ctx)
            self._ctx = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
