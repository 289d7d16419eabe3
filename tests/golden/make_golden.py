"""Writes tests/golden/hotpath_golden.npz from the reference's own CPU kernels.

Run where the reference is mounted and ``make -C oracle`` has produced
``oracle/_ref/libvvref_cpu.so`` (the reference's src/cpu/cpu_kernels.c compiled
unmodified):

    python tests/golden/make_golden.py

Every array the reference computed is stored next to the seeded inputs that
produced it, so the fixtures can be replayed on a machine that has neither the
reference nor numpy's RNG stream of this version. Shapes: the reference's own
known-answer cases (tests/test_cpu_kernels.c:150-183: RMSNorm 4x128, SwiGLU
1024; tests/test_decode_position.c:220-238: RoPE at position 913, 28 heads x
128, theta 1e6) plus the 7B row shapes at a handful of rows.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "hotpath_golden.npz")


def main() -> None:
    assert oracle.have_reference(), "oracle/_ref/libvvref_cpu.so missing: run make -C oracle"
    ref = oracle.reference()
    rng = np.random.default_rng(20240)
    g = {}

    # --- RMSNorm, FP32 in/out, FP16 weight (cpu_kernels.c:1432) ---
    for tag, rows, n, scale in (("a", 4, 128, 3.0), ("b", 3, 3584, 1.0), ("c", 2, 1536, 1.0)):
        x = (rng.standard_normal((rows, n)) * scale).astype(np.float32)
        w = (1.0 + 0.02 * rng.standard_normal(n)).astype(np.float16)
        g[f"rmsnorm_{tag}_x"] = x
        g[f"rmsnorm_{tag}_w"] = w
        g[f"rmsnorm_{tag}_y"] = ref.rmsnorm(x, w, rows, n, np.float32(1e-6))

    # --- residual add + RMSNorm at the FP16 boundary (decoder.c:950-958) ---
    h = rng.standard_normal((5, 3584)).astype(np.float16)
    d = rng.standard_normal((5, 3584)).astype(np.float16)
    w = (1.0 + 0.02 * rng.standard_normal(3584)).astype(np.float16)
    hn, y = oracle.add_rmsnorm_f16(h, d, w, 1e-6, impl=ref)
    g.update(addnorm_h=h, addnorm_d=d, addnorm_w=w, addnorm_h_out=hn, addnorm_y=y)

    # --- RoPE (cpu_kernels.c:1453), FP32 and FP16-boundary ---
    for tag, rows, heads, hd, off, theta in (
            ("a", 3, 28, 128, 913, 1e6),      # test_decode_position's case
            ("b", 6, 4, 128, 0, 1e6),
            ("c", 4, 2, 128, 14445, 1e6),     # tail of the 14449-token prompt
            ("d", 3, 2, 64, 131000, 1e4)):    # long context, other head_dim/theta
        x = rng.standard_normal((rows, heads, hd)).astype(np.float16)
        g[f"rope_{tag}_x"] = x
        g[f"rope_{tag}_meta"] = np.array([off, theta], np.float64)
        g[f"rope_{tag}_y32"] = ref.rope(x.astype(np.float32), rows, heads, hd, off, np.float32(theta))
        g[f"rope_{tag}_y16"] = oracle.rope_f16(x, off, theta, impl=ref)

    # --- SwiGLU (cpu_kernels.c:1536) ---
    gate = (rng.standard_normal(1024) * 4.0).astype(np.float32)
    up = rng.standard_normal(1024).astype(np.float32)
    g.update(swiglu_a_g=gate, swiglu_a_u=up, swiglu_a_y=ref.swiglu(gate, up))
    gate16 = np.concatenate([rng.standard_normal(4096) * 2.0,
                             np.array([0.0, -0.0, 65504.0, -65504.0, 6e-8, -6e-8, 11.0, -17.5, -30.0, 88.0])
                             ]).astype(np.float16)
    up16 = rng.standard_normal(gate16.size).astype(np.float16)
    g.update(swiglu_b_g=gate16, swiglu_b_u=up16, swiglu_b_y=oracle.swiglu_f16(gate16, up16, impl=ref))

    # --- residual add (cpu_kernels.c:1550) ---
    x = rng.standard_normal(1000).astype(np.float32)
    yv = rng.standard_normal(1000).astype(np.float32)
    g.update(resadd_x=x, resadd_y=yv, resadd_out=ref.residual_add(x, yv))

    # --- embedding gather (cpu_kernels.c:1560) ---
    table = (0.02 * rng.standard_normal((97, 256))).astype(np.float16)
    table[3, :4] = np.array([0.0, -0.0, 6e-8, 65504.0], np.float16)   # zero, -0, subnormal, max
    ids = np.array([0, 96, 3, 3, 41, 7, 96, 1], np.int32)
    g.update(embed_table=table, embed_ids=ids, embed_out=ref.embedding(table, ids, ids.size, 256))

    np.savez_compressed(OUT, **g)
    print(f"wrote {OUT}: {len(g)} arrays, {os.path.getsize(OUT)} bytes")


if __name__ == "__main__":
    main()
