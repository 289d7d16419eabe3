"""The C-ABI library: loads without a GPU, exports every symbol the header
declares, validates arguments before touching CUDA, and the row partition.
No compute call is made here."""
import ctypes as C
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "vvb200.h")


@pytest.fixture(scope="module")
def vv():
    import vvb200
    return vvb200


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vvb?_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_reference_op_names():
    names = declared_functions()
    for ref_name in ("vv_embedding_dev", "vv_rmsnorm_dev", "vv_rope_dev", "vv_swiglu_dev", "vv_swiglu_fused_dev",
                     "vv_residual_add_dev", "vv_bias_add_dev", "vv_fp32_to_fp16_dev", "vv_fp16_to_fp32_dev"):
        assert ref_name in names


def test_library_exports_every_declared_symbol(vv):
    lib = C.CDLL(vv.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in vvb200.h but not exported"
        assert n in vv.SIGNATURES, f"{n} has no ctypes signature in the binding"
    dyn = subprocess.run(["nm", "-D", "--defined-only", vv.LIB_PATH], capture_output=True, text=True).stdout
    for n in names:
        assert re.search(rf" T {n}$", dyn, flags=re.M), n


def test_header_compiles_as_c11_and_cxx(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "vvb200.h"\nint main(void){ return VV_OK; }\n')
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-pedantic", f"-I{ROOT}/include", "-c", str(src), "-o",
                    str(tmp_path / "t.o")], check=True)
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", f"-I{ROOT}/include", "-x", "c++", "-c", str(src), "-o",
                    str(tmp_path / "t2.o")], check=True)


# the reference tree: VV_REFERENCE_DIR, else a directory named "reference" beside this repository
REF_INCLUDE = os.environ.get("VV_REFERENCE_DIR", os.path.join(os.path.dirname(ROOT), "reference")) + "/include"


@pytest.mark.skipif(not os.path.exists(REF_INCLUDE + "/vibevoice/device.h"), reason="reference headers not mounted")
def test_declarations_agree_with_the_reference_headers(tmp_path):
    """One translation unit includes the reference's own device.h and then
    vvb200.h: a C compiler rejects any redeclaration whose type differs, so this
    compiles only if every drop-in signature (and the status enum it returns)
    is the reference's. The unit also takes each function's address through the
    reference's prototype and links against the static archive."""
    names = ["vv_embedding_dev", "vv_rmsnorm_dev", "vv_rope_dev", "vv_swiglu_dev", "vv_swiglu_fused_dev",
             "vv_residual_add_dev", "vv_bias_add_dev", "vv_fp32_to_fp16_dev", "vv_fp16_to_fp32_dev",
             "vv_act_quant_dev", "vv_rmsnorm_q8_dev", "vv_swiglu_q8_dev", "vv_col_absmax_dev",
             "vv_lm_head_gemv_dev", "vv_argmax_dev"]
    src = tmp_path / "both.c"
    src.write_text('#include "vibevoice/device.h"\n#include "vvb200.h"\n#include <stdio.h>\n'
                   "int main(void) {\n  const void* fns[] = {" + ", ".join(f"(const void*){n}" for n in names) +
                   "};\n  printf(\"%d\\n\", (int)(sizeof fns / sizeof fns[0]));\n"
                   "  return VV_Q8_LAYOUT_COUNT == 4 && VV_ACT_QUANT_MAX_K == 22528 && VV_ERR_CUDA_LAUNCH == -102 ? 0 : 1;\n}\n")
    obj = tmp_path / "both.o"
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", f"-I{REF_INCLUDE}", f"-I{ROOT}/include", "-c", str(src),
                    "-o", str(obj)], check=True)
    exe = tmp_path / "both"
    lib = os.path.join(ROOT, "vibevoice.c_b200", "lib", "libvvb200.a")
    subprocess.run(["g++", str(obj), lib, "-L/usr/local/cuda/lib64", "-lcudart_static", "-lpthread", "-ldl", "-lrt",
                    "-lm", "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout
    assert out.strip() == str(len(names))


def test_version_and_status_strings(vv):
    assert vv.version().startswith("vvb200 ") and "sm_100a" in vv.version()
    assert vv.status_string(0) == "ok"
    assert vv.status_string(vv.VV_ERR_NULL_PTR) == "null pointer"
    assert vv.status_string(-12345) == "unknown status"


def test_status_codes_match_the_reference_enum(vv):
    """include/vibevoice/types.h:18-58."""
    assert (vv.VV_OK, vv.VV_ERR_INVALID_ARG, vv.VV_ERR_NULL_PTR, vv.VV_ERR_UNSUPPORTED) == (0, -1, -2, -7)
    assert (vv.VV_ERR_CUDA, vv.VV_ERR_CUDA_OOM, vv.VV_ERR_CUDA_LAUNCH) == (-100, -101, -102)
    text = open(HEADER).read()
    for name, val in (("VV_ERR_INVALID_ARG", -1), ("VV_ERR_NULL_PTR", -2), ("VV_ERR_UNSUPPORTED", -7),
                      ("VV_ERR_CUDA_LAUNCH", -102)):
        assert re.search(rf"{name}\s*=\s*{val}\b", text)


def test_argument_validation_needs_no_gpu(vv):
    """NULL tensors and negative sizes are rejected before any CUDA call, with
    the reference's codes (src/cuda/rmsnorm.cu:86, rope.cu:93, swiglu.cu:83,
    embedding.cu:63). Fake non-null addresses are never dereferenced."""
    P = 0x1000
    assert vv.vv_rmsnorm_dev(None, P, P, 1, 8, 1e-6, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv.vv_rmsnorm_dev(P, None, P, 1, 8, 1e-6, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv.vv_rmsnorm_dev(P, P, None, 1, 8, 1e-6, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv.vv_rmsnorm_dev(P, P, P, -1, 8, 1e-6, stream=0) == vv.VV_ERR_INVALID_ARG
    assert vv.vv_rmsnorm_dev(P, P, P, 0, 8, 1e-6, stream=0) == vv.VV_OK
    assert vv.vv_rope_dev(None, 1, 1, 128, 0, None, 1e6, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv.vv_rope_dev(P, 0, 1, 128, 0, None, 1e6, stream=0) == vv.VV_OK
    assert vv.vv_rope_dev(P, 1, 1, 1024, 0, None, 1e6, stream=0) == vv.VV_ERR_UNSUPPORTED
    assert vv.vv_rope_dev(P, -1, 1, 128, 0, None, 1e6, stream=0) == vv.VV_ERR_INVALID_ARG
    assert vv.vv_swiglu_dev(None, P, P, 8, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv.vv_swiglu_dev(P, P, P, -8, stream=0) == vv.VV_ERR_INVALID_ARG
    assert vv.vv_swiglu_dev(P, P, P, 0, stream=0) == vv.VV_OK
    assert vv.vv_swiglu_fused_dev(None, P, 1, 8, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv.vv_embedding_dev(P, None, P, 1, 8, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv.vv_embedding_dev(P, P, P, 0, 8, stream=0) == vv.VV_OK
    assert vv.vv_residual_add_dev(P, None, 8, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv.vv_residual_add_dev(P, P, 0, stream=0) == vv.VV_OK
    assert vv.vv_bias_add_dev(None, P, 1, 8, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv.vv_fp32_to_fp16_dev(None, P, 8, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv.vv_fp16_to_fp32_dev(P, None, 8, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv.vvb_add_rmsnorm_dev(None, P, P, P, 1, 8, 1e-6, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv.vvb_add_rmsnorm_dev(P, P, P, P, 0, 8, 1e-6, stream=0) == vv.VV_OK
    assert vv.vvb_rope_qk_dev(None, P, 1, 28, 4, 128, 0, None, 1e6, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv.vvb_rope_qk_dev(P, None, 1, 28, 4, 128, 0, None, 1e6, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv.vvb_rope_qk_dev(None, None, 1, 0, 0, 128, 0, None, 1e6, stream=0) == vv.VV_OK
    assert vv.vvb_embedding_rmsnorm_dev(P, P, P, None, P, 1, 8, 10, 1e-6, stream=0) == vv.VV_ERR_NULL_PTR
    assert vv._lib.vvb_layer_chain_dev(None, 0) == vv.VV_ERR_NULL_PTR
    assert vv._lib.vvb_layer_chain_host(None, None) == vv.VV_ERR_NULL_PTR
    assert vv._lib.vvb_layer_chain_host_multi(None, None) == vv.VV_ERR_NULL_PTR
    import ctypes as C
    m = C.c_void_p()
    assert vv._lib.vvb_host_multi_create(None, None, 2, 64, 3584, 28, 4, 128, 18944) == vv.VV_ERR_NULL_PTR
    assert vv._lib.vvb_host_multi_create(C.byref(m), None, 0, 64, 3584, 28, 4, 128, 18944) == vv.VV_ERR_INVALID_ARG
    assert vv._lib.vvb_host_multi_create(C.byref(m), None, 65, 64, 3584, 28, 4, 128, 18944) == vv.VV_ERR_INVALID_ARG
    assert vv._lib.vvb_host_multi_devices(None) == 0 and vv._lib.vvb_host_multi_last_ms(None) == 0.0
    vv._lib.vvb_host_multi_destroy(None)                 # a no-op, like free(NULL)
    # the fused KV-cache append, in its three forms
    assert vv._lib.vvb_kv_append_dev(None, 0) == vv.VV_ERR_NULL_PTR
    kv = lambda **kw: vv.vvb_kv_append_dev(kw.pop("q", P), kw.pop("k", P), P, kw.pop("ks", P), P, kw.pop("rows", 1),
                                           28, 4, 128, stream=0, **kw)
    assert kv(q=None) == vv.VV_ERR_NULL_PTR and kv(k=None) == vv.VV_ERR_NULL_PTR and kv(ks=None) == vv.VV_ERR_NULL_PTR
    assert kv(rows=-1) == vv.VV_ERR_INVALID_ARG and kv(cache_offset=-1) == vv.VV_ERR_INVALID_ARG
    assert kv(kv_format=7) == vv.VV_ERR_UNSUPPORTED and kv(kv_format=-1) == vv.VV_ERR_UNSUPPORTED
    assert kv(kv_format=3) == vv.VV_ERR_NULL_PTR          # TurboQuant needs the two sigma arrays
    assert kv(rows=0) == vv.VV_OK and kv(rows=0, kv_format=2, page_table=P) == vv.VV_OK
    assert vv.vvb_rope_qk_append_dev(P, P, None, None, None, None, P, P, 1, 28, 4, 128, 0, 0, None, 1e6, 0, 0) \
        == vv.VV_ERR_NULL_PTR
    assert vv.vvb_rope_qk_append_fp8_dev(P, P, P, None, None, None, P, P, None, 1, 28, 4, 128, 0, 0, None, 1e6, 0, 0, 0) \
        == vv.VV_ERR_UNSUPPORTED                                     # kv_format 0 is the FP16 cache: the other call
    assert vv.vvb_rope_qk_append_fp8_dev(P, P, P, None, None, None, P, P, None, 0, 28, 4, 128, 0, 0, None, 1e6, 1, 0, 0) \
        == vv.VV_OK
    ctx = C.c_void_p()
    assert vv._lib.vvb_host_ctx_create(C.byref(ctx), 0, 0, 8, 1, 1, 16, 8) == vv.VV_ERR_INVALID_ARG
    assert vv._lib.vvb_host_ctx_create(None, 0, 1, 8, 1, 1, 16, 8) == vv.VV_ERR_NULL_PTR


def test_no_cuda_device_is_an_error_not_a_fallback(vv):
    """Without a usable device a real launch must fail with a status code --
    the library has no CPU path to fall back on."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    P = 0x1000
    st = vv.vv_swiglu_dev(P, P, P, 1024, stream=0)
    assert st in (vv.VV_ERR_CUDA_LAUNCH, vv.VV_ERR_CUDA)


def test_shard_rows_partition(vv):
    """ceil(T/n)-row blocks; T = 14449 gives 7225+7224, 3613*3+3610, 1807*7+1800."""
    T = 14449
    expect = {1: [14449], 2: [7225, 7224], 4: [3613, 3613, 3613, 3610], 8: [1807] * 7 + [1800]}
    for n, counts in expect.items():
        got = [vv.vvb_shard_rows(T, n, g) for g in range(n)]
        assert [c for _, c in got] == counts
        assert got[0][0] == 0
        for (f0, c0), (f1, _) in zip(got, got[1:]):
            assert f0 + c0 == f1
        assert got[-1][0] + got[-1][1] == T
    # more parts than rows: trailing parts are empty, nothing is lost or doubled
    got = [vv.vvb_shard_rows(3, 8, g) for g in range(8)]
    assert sum(c for _, c in got) == 3 and all(c in (0, 1) for _, c in got)
    assert vv.vvb_shard_rows(0, 4, 2) == (0, 0)
    first, count = C.c_int64(), C.c_int64()
    assert vv._lib.vvb_shard_rows(10, 0, 0, C.byref(first), C.byref(count)) == vv.VV_ERR_INVALID_ARG
    assert vv._lib.vvb_shard_rows(10, 2, 2, C.byref(first), C.byref(count)) == vv.VV_ERR_INVALID_ARG
    assert vv._lib.vvb_shard_rows(-1, 2, 0, C.byref(first), C.byref(count)) == vv.VV_ERR_INVALID_ARG
    assert vv._lib.vvb_shard_rows(10, 2, 0, None, C.byref(count)) == vv.VV_ERR_NULL_PTR


def test_product_does_not_reference_the_oracle():
    """Nothing under the package or include/ may import, link or mention the
    CPU checkers."""
    pkg = os.path.join(ROOT, "vibevoice.c_b200")
    for base, _, files in os.walk(pkg):
        if os.sep + "build" in base or os.sep + "lib" in base or "__pycache__" in base:
            continue
        for f in files:
            if f.endswith((".py", ".c", ".cu", ".cuh", ".h")) or f == "Makefile":
                text = open(os.path.join(base, f), errors="ignore").read()
                assert "oracle" not in text.lower(), os.path.join(base, f)
    ldd = subprocess.run(["ldd", os.path.join(pkg, "lib", "libvvb200.so")], capture_output=True, text=True).stdout
    assert "oracle" not in ldd and "vvref" not in ldd
