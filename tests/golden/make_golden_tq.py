"""Golden TurboQuant KV-cache bytes from the reference's own store kernel.

Needs a CUDA device and oracle/_ref/libvvref_cuda.so (the reference's
src/cuda/kv_quant.cu compiled unmodified, with its release flags, by
oracle/Makefile). Calls vv_kv_quant_store_dev (src/cuda/kv_quant.cu:555-566)
for the four TurboQuant formats on seeded K [96, 4, 128] with a reference key
[4, 128] subtracted (k_ref given, build_ref false) and V [96, 4, 128] as it is
-- Gaussian rows, rows with an outlier channel, tiny rows, a zero row -- and
writes tests/golden/tq_kv_golden.npz: the inputs, the code bytes and the FP16
sigmas. The CPU suite pins the oracle's restatement (oracle/vvb_oracle.c:
orc_kv_store_tq) to these; the reference has no CPU implementation.

    python tests/golden/make_golden_tq.py [output.npz]
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
LIB = os.path.join(ROOT, "oracle", "_ref", "libvvref_cuda.so")
BPV = {3: 64, 4: 48, 5: 32, 6: 24}


def inputs():
    rng = np.random.default_rng(30)
    k = (rng.standard_normal((96, 4, 128)) * 1.5).astype(np.float16)
    v = (rng.standard_normal((96, 4, 128)) * 0.3).astype(np.float16)
    k[5, :, 17] = 40.0                      # an outlier channel, what the rotation is for
    k[6] *= np.float16(1e-3)                # tiny vectors
    v[7] = 0                                # zero vectors: sigma at its floor
    v[8, 1] = 3.0                           # a constant vector
    kref = (rng.standard_normal((4, 128)) * 0.5).astype(np.float16)
    return k, v, kref


def main(out_path):
    ref = C.CDLL(LIB)
    vp, i = C.c_void_p, C.c_int
    ref.vv_kv_quant_store_dev.argtypes = [vp, vp, vp, vp, vp, vp, vp, C.c_bool, i, i, i, vp, i, i, vp]
    ref.vv_kv_quant_store_dev.restype = i
    torch.cuda.set_device(0)
    k, v, kref = inputs()
    out = {"k": k.view(np.uint16), "v": v.view(np.uint16), "k_ref": kref.view(np.uint16)}
    n_pos, n_kv, hd = k.shape
    dk, dv, dr = (torch.from_numpy(a.view(np.int16)).cuda() for a in (k, v, kref))
    for fmt, name in ((3, "tq4"), (4, "tq3"), (5, "tq2"), (6, "tq1_5")):
        ks = torch.zeros(n_pos, n_kv * BPV[fmt], dtype=torch.uint8, device="cuda")
        vs = torch.zeros_like(ks)
        km = torch.zeros(n_pos, n_kv, dtype=torch.float16, device="cuda")
        vm = torch.zeros_like(km)
        st = ref.vv_kv_quant_store_dev(dk.data_ptr(), dv.data_ptr(), ks.data_ptr(), vs.data_ptr(), km.data_ptr(),
                                       vm.data_ptr(), dr.data_ptr(), False, n_kv, hd, 0, None, n_pos, fmt, None)
        assert st == 0, st
        torch.cuda.synchronize()
        out[f"k_store_{name}"], out[f"v_store_{name}"] = ks.cpu().numpy(), vs.cpu().numpy()
        out[f"k_meta_{name}"], out[f"v_meta_{name}"] = km.cpu().numpy().view(np.uint16), vm.cpu().numpy().view(np.uint16)
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k_: v_.shape for k_, v_ in out.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "tq_kv_golden.npz"))
