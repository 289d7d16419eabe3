"""Ordering under programmatic dependent launch.

Every kernel of the library is launched with the programmatic stream
serialization attribute and waits for the grid before it at its first
instruction. These tests put the library's kernels in dependency chains with
kernels that are NOT the library's (torch element-wise kernels, memsets and
copies, which know nothing of the attribute) -- the situation inside the
reference's engine, where GEMMs and attention sit between these ops
(src/inference/decoder.c:806-990) -- directly on a stream and replayed from a
CUDA graph, many times over with fresh data, and demand the bytes of a fully
synchronised run. A kernel that started reading before its producer had
finished, or a foreign kernel that overtook one of ours, would show as a
mismatch.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

H, NQ, NKV, HD, INTER = 3584, 28, 4, 128, 18944


@pytest.fixture(scope="module")
def vv():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import vvb200
    torch.cuda.set_device(0)
    return vvb200


def ok(st):
    assert st == 0, st


class Chain:
    """hidden -> [torch: delta = hidden * a] -> add+norm -> [torch: gate = normed-tile * b]
    -> swiglu in place -> [torch: q = gate slice + c] -> rope -> [torch copy] -> residual add.
    Each arrow is a true data dependency between a foreign kernel and one of ours."""

    def __init__(self, vv, rows):
        self.vv, self.rows = vv, rows
        g = torch.Generator(device="cuda").manual_seed(rows)
        mk = lambda *s: torch.randn(*s, device="cuda", generator=g).half()
        self.seed_hidden = mk(rows, H)
        self.hidden = torch.empty_like(self.seed_hidden)
        self.delta = torch.empty(rows, H, device="cuda", dtype=torch.float16)
        self.normed = torch.empty(rows, H, device="cuda", dtype=torch.float16)
        self.w = (1 + 0.05 * torch.randn(H, device="cuda", generator=g)).half()
        self.gate = torch.empty(rows, INTER, device="cuda", dtype=torch.float16)
        self.up = mk(rows, INTER)
        self.q = torch.empty(rows, NQ, HD, device="cuda", dtype=torch.float16)
        self.k = mk(rows, NKV, HD)
        self.k_work = torch.empty_like(self.k)
        self.acc = torch.empty(rows, NQ * HD, device="cuda", dtype=torch.float16)
        self.reps = INTER // H + 1

    def step(self, stream, sync_between):
        vv, rows = self.vv, self.rows
        s = stream.cuda_stream
        fence = (lambda: torch.cuda.synchronize()) if sync_between else (lambda: None)
        with torch.cuda.stream(stream):
            self.hidden.copy_(self.seed_hidden); fence()                                  # foreign
            torch.mul(self.hidden, 0.5, out=self.delta); fence()                          # foreign
            ok(vv.vvb_add_rmsnorm_dev(self.hidden, self.delta, self.w, self.normed, rows, H, 1e-6, s)); fence()
            self.gate.copy_(self.normed.repeat(1, self.reps)[:, :INTER]); fence()         # foreign
            ok(vv.vv_swiglu_dev(self.gate, self.up, self.gate, rows * INTER, s)); fence()
            torch.add(self.gate[:, :NQ * HD].reshape(rows, NQ, HD), 0.25, out=self.q); fence()   # foreign
            self.k_work.copy_(self.k); fence()                                            # foreign
            ok(vv.vvb_rope_qk_dev(self.q, self.k_work, rows, NQ, NKV, HD, 11, None, 1e6, s)); fence()
            self.acc.copy_(self.q.reshape(rows, NQ * HD)); fence()                        # foreign
            ok(vv.vv_residual_add_dev(self.acc, self.normed[:, :NQ * HD].contiguous(), rows * NQ * HD, s)); fence()
            self.acc.mul_(2.0); fence()                                                   # foreign

    def result(self):
        torch.cuda.synchronize()
        return [t.cpu().numpy().view(np.uint16).copy() for t in (self.hidden, self.normed, self.gate, self.q, self.k_work, self.acc)]


@pytest.mark.parametrize("rows", [1, 3, 64, 700])
def test_stream_order_with_foreign_kernels(vv, rows):
    c = Chain(vv, rows)
    st = torch.cuda.Stream()
    c.step(st, sync_between=True)
    want = c.result()
    for it in range(25):
        c.step(st, sync_between=False)
    got = c.result()
    for a, b in zip(got, want):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("rows", [1, 64, 700])
def test_graph_replay_with_foreign_kernels(vv, rows):
    c = Chain(vv, rows)
    st = torch.cuda.Stream()
    c.step(st, sync_between=True)
    want = c.result()
    # new inputs for the captured run: the graph must recompute everything from seed_hidden
    c.step(st, sync_between=False)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=st):
        c.step(st, sync_between=False)
        c.step(st, sync_between=False)          # back to back: the second pass overwrites the first
    for _ in range(20):
        for t in (c.hidden, c.normed, c.gate, c.q, c.k_work, c.acc, c.delta):
            t.fill_(7.0)                        # stale data a premature read would pick up
        g.replay()
        got = c.result()
        for a, b in zip(got, want):
            assert np.array_equal(a, b)


def test_decode_sequence_replay_matches_eager(vv):
    """The one-token launch sequence (norm -> bias+RoPE+append -> add+norm -> SwiGLU, 8 layers,
    then final norm + head + argmax) where every kernel consumes what the one before produced:
    graph replay == the same calls with a device synchronisation after each."""
    L, V, max_len = 8, 4096, 32
    g = torch.Generator(device="cuda").manual_seed(5)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g).half()
    w = (1 + 0.05 * torch.randn(H, device="cuda", generator=g)).half()
    head = (0.02 * torch.randn(V, H, device="cuda", generator=g)).half()
    hid0, up = mk(1, H), mk(1, INTER)
    hid, nrm = torch.empty_like(hid0), torch.empty(1, H, device="cuda", dtype=torch.float16)
    q, k, v = (torch.empty(1, n, HD, device="cuda", dtype=torch.float16) for n in (NQ, NKV, NKV))
    gate = torch.empty(1, INTER, device="cuda", dtype=torch.float16)
    kc = [torch.zeros(max_len, NKV * HD, device="cuda", dtype=torch.float16) for _ in range(L)]
    vc = [torch.zeros(max_len, NKV * HD, device="cuda", dtype=torch.float16) for _ in range(L)]
    dpos = torch.tensor([5], device="cuda", dtype=torch.int32)
    nb = vv.vvb_lm_head_scratch_bytes(V)
    scratch = torch.empty(nb, device="cuda", dtype=torch.uint8)
    tok, val = torch.zeros(1, device="cuda", dtype=torch.int32), torch.zeros(1, device="cuda")

    def token(s, fence):
        hid.copy_(hid0); fence()
        ok(vv.vv_rmsnorm_dev(hid, w, nrm, 1, H, 1e-6, s)); fence()
        for l in range(L):
            # stand-ins for the engine's projections: slices of the normed row (foreign kernels)
            q.copy_(nrm[:, :NQ * HD].reshape(1, NQ, HD)); k.copy_(nrm[:, :NKV * HD].reshape(1, NKV, HD))
            v.copy_(nrm[:, NKV * HD:2 * NKV * HD].reshape(1, NKV, HD)); fence()
            ok(vv.vvb_rope_qk_append_dev(q, k, v, None, None, None, kc[l], vc[l], 1, NQ, NKV, HD, 0, 0,
                                         dpos, 1e6, 0, s)); fence()
            ok(vv.vvb_add_rmsnorm_dev(hid, q.reshape(1, NQ * HD), w, nrm, 1, H, 1e-6, s)); fence()
            gate.copy_(nrm.repeat(1, INTER // H + 1)[:, :INTER]); fence()
            ok(vv.vvb_swiglu_dev(gate, up, gate, INTER, s)); fence()
            ok(vv.vvb_add_rmsnorm_dev(hid, gate[:, :H].contiguous(), w, nrm, 1, H, 1e-6, s)); fence()
        ok(vv.vvb_lm_head_argmax_dev(hid, w, 1e-6, head, V, H, None, scratch, nb, tok, val, s)); fence()

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        token(stream.cuda_stream, torch.cuda.synchronize)
    torch.cuda.synchronize()
    want = (int(tok.item()), float(val.item()), hid.cpu().numpy().view(np.uint16).copy(),
            kc[L - 1].cpu().numpy().view(np.uint16).copy())
    with torch.cuda.stream(stream):
        token(stream.cuda_stream, lambda: None)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            token(stream.cuda_stream, lambda: None)
    for _ in range(30):
        tok.zero_(); hid.fill_(3.0); nrm.fill_(3.0); gate.fill_(3.0)
        graph.replay()
        torch.cuda.synchronize()
        assert int(tok.item()) == want[0] and float(val.item()) == want[1]
        assert np.array_equal(hid.cpu().numpy().view(np.uint16), want[2])
        assert np.array_equal(kc[L - 1].cpu().numpy().view(np.uint16), want[3])
