"""Golden FP8 KV-cache bytes from the reference's own store kernel.

Needs a CUDA device and oracle/_ref/libvvref_cuda.so (the reference's
src/cuda/kv_quant.cu compiled unmodified by oracle/Makefile). Calls
vv_kv_quant_store_dev (src/cuda/kv_quant.cu:555-566) for both FP8 formats on
  (a) all 65 536 FP16 bit patterns, laid out as K = V = [128 positions, 4 heads, 128],
  (b) seeded random K [64, 4, 128] with a reference key [4, 128] subtracted
      (k_ref given, build_ref false) and V as it is,
and writes tests/golden/fp8_kv_golden.npz. The CPU suite pins the oracle's
restatement (oracle/vvb_oracle.c: orc_fp8_encode, orc_kv_store_fp8) to these
bytes; the reference has no CPU implementation of this format.

    python tests/golden/make_golden_fp8.py [output.npz]
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
LIB = os.path.join(ROOT, "oracle", "_ref", "libvvref_cuda.so")


def main(out_path):
    ref = C.CDLL(LIB)
    vp, i = C.c_void_p, C.c_int
    ref.vv_kv_quant_store_dev.argtypes = [vp, vp, vp, vp, vp, vp, vp, C.c_bool, i, i, i, vp, i, i, vp]
    ref.vv_kv_quant_store_dev.restype = i
    torch.cuda.set_device(0)
    out = {}

    def store(k_np, v_np, kref_np, fmt):
        n_pos, n_kv, hd = k_np.shape
        k = torch.from_numpy(k_np.view(np.int16)).cuda()
        v = torch.from_numpy(v_np.view(np.int16)).cuda()
        ks = torch.zeros(n_pos, n_kv * hd, dtype=torch.uint8, device="cuda")
        vs = torch.zeros_like(ks)
        kr = torch.from_numpy(kref_np.view(np.int16)).cuda() if kref_np is not None else None
        st = ref.vv_kv_quant_store_dev(k.data_ptr(), v.data_ptr(), ks.data_ptr(), vs.data_ptr(), None, None,
                                       kr.data_ptr() if kr is not None else None, False, n_kv, hd, 0, None,
                                       n_pos, fmt, None)
        assert st == 0, st
        torch.cuda.synchronize()
        return ks.cpu().numpy(), vs.cpu().numpy()

    every = np.arange(65536, dtype=np.uint16).reshape(128, 4, 128)
    for fmt, name in ((1, "e4m3"), (2, "e5m2")):
        ks, vs = store(every, every, None, fmt)
        assert np.array_equal(ks, vs)
        out[f"all_halves_{name}"] = ks.reshape(-1)

    rng = np.random.default_rng(20)
    k = (rng.standard_normal((64, 4, 128)) * 1.5).astype(np.float16)
    v = (rng.standard_normal((64, 4, 128)) * 0.02).astype(np.float16)      # small: exercises the subnormal range
    kref = (rng.standard_normal((4, 128)) * 0.5).astype(np.float16)
    out["k"], out["v"], out["k_ref"] = k.view(np.uint16), v.view(np.uint16), kref.view(np.uint16)
    for fmt, name in ((1, "e4m3"), (2, "e5m2")):
        ks, vs = store(k.view(np.uint16), v.view(np.uint16), kref.view(np.uint16), fmt)
        out[f"k_minus_ref_{name}"], out[f"v_{name}"] = ks, vs
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k_: v_.shape for k_, v_ in out.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "fp8_kv_golden.npz"))
