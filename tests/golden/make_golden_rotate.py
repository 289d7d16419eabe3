"""Golden outputs of the reference's own Hadamard rotation kernels.

Needs a CUDA device and oracle/_ref/libvvref_cuda.so (the reference's
src/cuda/kv_quant.cu compiled unmodified, with its release flags, by
oracle/Makefile). Calls vv_kv_rotate_dev and vv_kv_unrotate_dev
(src/cuda/kv_quant.cu:473-494) on seeded FP16 x [40, 6, 128] -- Gaussian head
vectors, one with an outlier channel, tiny ones, a zero one, a constant one,
one of the largest halves -- and writes tests/golden/kv_rotate_golden.npz: the
input, the rotated output and the un-rotated output of that same input. The CPU
suite pins the oracle's restatement (oracle/vvb_oracle.c: orc_kv_rotate_f16) to
these bytes; the reference has no CPU implementation of this step.

    python tests/golden/make_golden_rotate.py [output.npz]
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
LIB = os.path.join(ROOT, "oracle", "_ref", "libvvref_cuda.so")


def inputs():
    rng = np.random.default_rng(31)
    x = rng.standard_normal((40, 6, 128)).astype(np.float16)
    x[3, :, 17] = 40.0                      # an outlier channel
    x[4] *= np.float16(1e-3)                # tiny vectors
    x[5, 0] = 0                             # a zero vector
    x[5, 1] = 3.0                           # a constant vector
    x[6, 2] = 65504.0                       # the largest halves: the transform overflows FP16
    x[7, 3] = 6e-8                          # subnormals
    return x


def main(out_path):
    ref = C.CDLL(LIB)
    vp, i = C.c_void_p, C.c_int
    for name in ("vv_kv_rotate_dev", "vv_kv_unrotate_dev"):
        getattr(ref, name).argtypes = [vp, i, i, i, vp]
        getattr(ref, name).restype = i
    x = inputs()
    out = {"x": x.view(np.uint16)}
    for name, key in (("vv_kv_rotate_dev", "rotated"), ("vv_kv_unrotate_dev", "unrotated")):
        d = torch.from_numpy(x.copy()).cuda()
        assert getattr(ref, name)(d.data_ptr(), x.shape[1], 128, x.shape[0], None) == 0
        torch.cuda.synchronize()
        out[key] = d.cpu().numpy().view(np.uint16)
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "kv_rotate_golden.npz"))
