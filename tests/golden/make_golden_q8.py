"""Writes tests/golden/q8_golden.npz from the reference's own int8 activation
quantizer (vv_quant_act_q8_cpu, src/cpu/cpu_int8.c:181-194, compiled unmodified
into oracle/_ref/libvvref_int8.so by `make -C oracle`):

    python tests/golden/make_golden_q8.py

Inputs are FP16-representable rows (the device quantizes FP16 values) at the
reference test's widths (tests/test_int8_linear.c:295-354: K in 1536, 3584) in
all four byte layouts, with the edge rows: all zero, a single non-zero, values
that tie at .5 after scaling, and the largest FP16 value.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "q8_golden.npz")


def main():
    assert oracle.have_reference_int8(), "oracle/_ref/libvvref_int8.so missing: run make -C oracle"
    ref = oracle.reference_int8()
    rng = np.random.default_rng(77)
    g = {}
    for K in (1536, 3584):
        x = rng.standard_normal((6, K)).astype(np.float16)
        x[1] = 0                                   # zero row: sx = 0, q = 0
        x[2] = 0
        x[2, 5] = -3.0                             # one non-zero: q = -127 there
        x[3, :64] = (np.arange(64) - 32) * 0.5     # with amax forced to 127 below: exact .5 ties
        x[3, 64] = 127.0
        x[3, 65:] = np.clip(x[3, 65:], -100, 100)
        x[4, 0] = 65504.0                          # largest FP16
        g[f"x_{K}"] = x
        for layout in range(4):
            xq, sx, xsum = ref.quant_act_q8(x.astype(np.float32), layout)
            g[f"xq_{K}_{layout}"], g[f"sx_{K}_{layout}"], g[f"xsum_{K}_{layout}"] = xq, sx, xsum
    np.savez_compressed(OUT, **g)
    print(f"wrote {OUT}: {len(g)} arrays, {os.path.getsize(OUT)} bytes")


if __name__ == "__main__":
    main()
