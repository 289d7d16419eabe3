"""The entry point for callers that cannot allocate device memory:
vvb_lm_head_argmax_static_dev keeps its argmax partials in an array inside the
library instead of taking scratch from the caller.

This file is named to be collected last, so that a run which stops at the first
failure has already run every other test. It must also pass alone in a fresh
process: nothing here relies on an earlier test having warmed the library up
(the very first call below is the one that looks up the array's address).

Checked on two calls in a row, through the C-ABI, against the entry point that
takes caller scratch (vvb_lm_head_argmax_dev). Both run the same kernels in the
same order, so token, winning value and logits must be bit-identical; the second
call uses a shorter head, so stale partials of the first call are still sitting
in the array when it runs and must not be read.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def vv():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import vvb200
    torch.cuda.set_device(0)
    return vvb200


def run_both(vv, V, K, seed, planted, device_memory_must_not_move):
    g = torch.Generator(device="cuda").manual_seed(seed)
    h = (3 * torch.randn(K, generator=g, device="cuda")).half()
    gamma = (1 + 0.1 * torch.randn(K, generator=g, device="cuda")).half()
    w = (0.02 * torch.randn(V, K, generator=g, device="cuda")).half()
    w[planted] = (0.05 * torch.sign(h.float() * gamma.float())).half()      # a clear winner

    nbytes = vv.vvb_lm_head_scratch_bytes(V)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    lg_ref = torch.empty(V, dtype=torch.float32, device="cuda")
    tok_ref = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    val_ref = torch.zeros(1, dtype=torch.float32, device="cuda")
    assert vv.vvb_lm_head_argmax_dev(h, gamma, 1e-6, w, V, K, lg_ref, scratch, nbytes, tok_ref, val_ref) == vv.VV_OK

    lg = torch.empty(V, dtype=torch.float32, device="cuda")
    tok = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    val = torch.zeros(1, dtype=torch.float32, device="cuda")
    # torch's own counter sees only torch's allocator; the free bytes the driver reports
    # (cudaMemGetInfo) also move for a cudaMalloc or cudaMallocAsync made inside the library.
    # The very first call on a device may load the library's module lazily, which takes device
    # memory once, so the driver's figure is held still from the second call on.
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before, _ = torch.cuda.mem_get_info()
    assert vv.vvb_lm_head_argmax_static_dev(h, gamma, 1e-6, w, V, K, lg, tok, val) == vv.VV_OK
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert torch.cuda.memory_allocated() == before
    if device_memory_must_not_move:
        assert free_after == free_before, (free_before, free_after)
    assert int(tok.item()) == int(tok_ref.item()) == planted
    assert torch.equal(val.view(torch.int32), val_ref.view(torch.int32))
    assert torch.equal(lg.view(torch.int32), lg_ref.view(torch.int32))
    return int(tok.item())


def test_static_scratch_entry_point_matches_the_caller_scratch_one_twice_in_a_row(vv):
    # first call: the 7B model's head, 152064 rows of 3584
    assert run_both(vv, 152064, 3584, seed=11, planted=150001, device_memory_must_not_move=False) == 150001
    # second call straight after, a much shorter head: the array still holds the first call's partials
    assert run_both(vv, 4000, 1536, seed=12, planted=17, device_memory_must_not_move=True) == 17
    # and a third, back at the full head
    assert run_both(vv, 152064, 3584, seed=13, planted=9, device_memory_must_not_move=True) == 9


def test_static_scratch_entry_point_limits_and_errors(vv):
    x = torch.zeros(64, dtype=torch.float16, device="cuda")
    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    too_tall = vv.VVB_LM_HEAD_STATIC_MAX_V + 1
    assert vv.vvb_lm_head_argmax_static_dev(x, None, 0.0, x, too_tall, 64, None, tok, None) == vv.VV_ERR_OVERFLOW
    assert vv.vvb_lm_head_argmax_static_dev(None, None, 0.0, x, 1, 64, None, tok, None) == vv.VV_ERR_NULL_PTR
    assert vv.vvb_lm_head_argmax_static_dev(x, None, 0.0, x, 1, 64, None, None, None) == vv.VV_ERR_NULL_PTR
    assert vv.vvb_lm_head_argmax_static_dev(x, None, 0.0, x, 0, 64, None, tok, None) == vv.VV_ERR_INVALID_ARG
    assert vv.vvb_lm_head_argmax_static_dev(x, None, 0.0, x, 1, 12, None, tok, None) == vv.VV_ERR_UNSUPPORTED
    # a one-row head, no norm, no logits, no value: the smallest legal call
    w = torch.ones(1, 64, dtype=torch.float16, device="cuda")
    assert vv.vvb_lm_head_argmax_static_dev(x, None, 0.0, w, 1, 64, None, tok, None) == vv.VV_OK
    torch.cuda.synchronize()
    assert int(tok.item()) == 0
