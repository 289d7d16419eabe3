"""The reference's own test programs, run with this library in place of the
seven CUDA files it replaces.

oracle/build_reftests.sh compiles the reference's C sources, its other CUDA
kernels (GEMMs, attention, KV cache) and five of its tests, unmodified, and
links them against vibevoice.c_b200/lib/libvvb200.a instead of
src/cuda/{rmsnorm,rope,swiglu,embedding,conv_vae,act_quant,lm_head}.cu. Each
program prints its own verdict and exits non-zero on a failed check:

  test_int8_linear      tests/test_int8_linear.c:57-109,295-354: the fused int8
                        producers bit-exact against vv_quant_act_q8_cpu, fused ==
                        unfused, every GEMM path fed by them
  test_decode_position  tests/test_decode_position.c:220-238: RoPE at a device-side
                        position == the host-side position, byte for byte
  test_prefill_append   tests/test_prefill_append.c:181-285: a two-layer decoder on
                        the GPU (norm, RoPE, SwiGLU, residual adds from
                        src/inference/decoder.c) against its CPU path
  test_skinny           tests/test_skinny.c:179-197: GEMM outputs through vv_bias_add_dev
  test_w4a16            tests/test_w4a16.c:405-500: INT4 linear layers, bias added by
                        vv_bias_add_dev (src/cuda/w4a16.cu:930)

Skipped where the programs were not built (the reference is not present on a
GPU box; the prebuilt programs travel with the tree).
"""
import os
import subprocess

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "oracle", "_ref", "tests")
PROGRAMS = ["test_int8_linear", "test_decode_position", "test_prefill_append", "test_skinny", "test_w4a16"]


@pytest.mark.parametrize("name", PROGRAMS)
def test_reference_program_passes_on_this_library(name, tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    exe = os.path.join(BIN, name)
    if not os.path.exists(exe):
        pytest.skip(f"{name} was not built (oracle/build_reftests.sh needs the reference's sources)")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    (tmp_path / f"reference_{name}.log").write_text(out)
    tail = "\n".join(out.splitlines()[-25:])
    assert r.returncode == 0, tail
    # a program that found no device reports a skip and exits 0: that is not a pass
    assert "no device available" not in out and "no GPU" not in out, tail
    assert "FAIL" not in out, tail
