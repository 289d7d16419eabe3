"""GPU tests of the host-buffer pipeline, of concurrent callers on their own
streams, and of the chain under CUDA-graph replay."""
import threading

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


def make_inputs(rows, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g).half()
    return dict(h=mk(rows, H), d=mk(rows, H), w=(1 + 0.02 * torch.randn(H, generator=g)).half(),
                q=mk(rows, NQ, HD), k=mk(rows, NKV, HD), gate=mk(rows, INTER), up=mk(rows, INTER))


def run_on_device(vv, t, rows, first, stream=None):
    dv = {k: v.cuda() for k, v in t.items()}
    n = torch.empty_like(dv["h"])
    c = vv.make_chain(dv["h"], dv["d"], dv["w"], n, dv["q"], dv["k"], dv["gate"], dv["up"], rows, H, NQ, NKV, HD,
                      INTER, first, 1e-6, 1e6)
    assert vv.vvb_layer_chain_dev(c, stream) == 0
    torch.cuda.synchronize()
    return {"h": dv["h"].cpu(), "n": n.cpu(), "q": dv["q"].cpu(), "k": dv["k"].cpu(), "gate": dv["gate"].cpu()}


@pytest.mark.parametrize("rows,slice_rows", [(1, 64), (700, 256), (1000, 1000), (2500, 1024)])
def test_host_pipeline_matches_device_path(vv, orc, rows, slice_rows):
    """vvb_layer_chain_host on pinned host tensors gives the bytes of the
    device-resident path, whatever the slicing, and reports its traffic."""
    first = 321
    t = make_inputs(rows, rows)
    want = run_on_device(vv, t, rows, first)
    pin = {k: v.clone().pin_memory() for k, v in t.items()}
    n = torch.empty(rows, H, dtype=torch.float16).pin_memory()
    pipe = vv.HostPipeline(0, slice_rows, H, NQ, NKV, HD, INTER)
    c = vv.make_chain(pin["h"], pin["d"], pin["w"], n, pin["q"], pin["k"], pin["gate"], pin["up"], rows, H, NQ, NKV,
                      HD, INTER, first, 1e-6, 1e6)
    assert pipe.run(c) == 0
    for got, key in ((pin["h"], "h"), (n, "n"), (pin["q"], "q"), (pin["k"], "k"), (pin["gate"], "gate")):
        assert torch.equal(got.view(torch.int16), want[key].view(torch.int16)), key
    h2d, d2h = pipe.last_traffic()
    assert h2d == rows * 2 * (2 * H + (NQ + NKV) * HD + 2 * INTER) + 2 * H
    assert d2h == rows * 2 * (2 * H + (NQ + NKV) * HD + INTER)
    assert pipe.last_ms() > 0
    # against the oracle too (a few rows)
    sel = slice(0, min(rows, 5))
    wh, wn = orc.add_rmsnorm_f16(t["h"][sel].numpy(), t["d"][sel].numpy(), t["w"].numpy(), 1e-6)
    assert np.array_equal(pin["h"][sel].numpy().view(np.uint16), wh.view(np.uint16))
    assert orc.ulp_distance(n[sel].numpy(), wn).max() <= 2
    pipe.close()


def test_host_pipeline_rejects_wrong_shape_and_null(vv):
    pipe = vv.HostPipeline(0, 64, H, NQ, NKV, HD, INTER)
    t = make_inputs(4, 1)
    pin = {k: v.pin_memory() for k, v in t.items()}
    n = torch.empty(4, H, dtype=torch.float16).pin_memory()
    bad = vv.make_chain(pin["h"], pin["d"], pin["w"], n, pin["q"], pin["k"], pin["gate"], pin["up"], 4, H, NQ, NKV, HD,
                        INTER // 2, 0, 1e-6, 1e6)
    assert pipe.run(bad) == vv.VV_ERR_INVALID_ARG
    null = vv.make_chain(None, pin["d"], pin["w"], n, pin["q"], pin["k"], pin["gate"], pin["up"], 4, H, NQ, NKV, HD,
                         INTER, 0, 1e-6, 1e6)
    assert pipe.run(null) == vv.VV_ERR_NULL_PTR
    empty = vv.make_chain(pin["h"], pin["d"], pin["w"], n, pin["q"], pin["k"], pin["gate"], pin["up"], 0, H, NQ, NKV,
                          HD, INTER, 0, 1e-6, 1e6)
    assert pipe.run(empty) == vv.VV_OK
    pipe.close()


def test_concurrent_callers_on_their_own_streams(vv):
    """Four host threads, each with its own stream and buffers, hammer the ops
    at once; every result must equal the serial answer byte for byte
    (tests/test_concurrent_decode.c:1-22: guards against shared scratch)."""
    rows, iters, nthreads = 33, 40, 4
    inputs = [make_inputs(rows, 100 + i) for i in range(nthreads)]
    serial = [run_on_device(vv, inputs[i], rows, 50 * i) for i in range(nthreads)]
    errors = []

    def worker(i):
        try:
            torch.cuda.set_device(0)
            s = torch.cuda.Stream()
            with torch.cuda.stream(s):
                for _ in range(iters):
                    dv = {k: v.cuda(non_blocking=False) for k, v in inputs[i].items()}
                    n = torch.empty_like(dv["h"])
                    c = vv.make_chain(dv["h"], dv["d"], dv["w"], n, dv["q"], dv["k"], dv["gate"], dv["up"], rows, H,
                                      NQ, NKV, HD, INTER, 50 * i, 1e-6, 1e6)
                    assert vv.vvb_layer_chain_dev(c, s) == 0
                    s.synchronize()
                    got = {"h": dv["h"], "n": n, "q": dv["q"], "k": dv["k"], "gate": dv["gate"]}
                    for key, val in got.items():
                        if not torch.equal(val.cpu().view(torch.int16), serial[i][key].view(torch.int16)):
                            errors.append((i, key))
        except Exception as e:  # noqa: BLE001
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(nthreads)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert not errors, errors[:5]


def test_chain_replays_under_a_cuda_graph(vv):
    rows = 257
    t = make_inputs(rows, 9)
    want = run_on_device(vv, t, rows, 10)
    dv = {k: v.cuda() for k, v in t.items()}
    src = {k: v.clone() for k, v in dv.items()}
    n = torch.empty_like(dv["h"])
    c = vv.make_chain(dv["h"], dv["d"], dv["w"], n, dv["q"], dv["k"], dv["gate"], dv["up"], rows, H, NQ, NKV, HD, INTER,
                      10, 1e-6, 1e6)
    s = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        assert vv.vvb_layer_chain_dev(c, s) == 0
        s.synchronize()
        with torch.cuda.graph(g, stream=s):
            assert vv.vvb_layer_chain_dev(c, s) == 0
    for _ in range(2):
        for k in ("h", "q", "k", "gate"):
            dv[k].copy_(src[k])
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        for key, val in (("h", dv["h"]), ("n", n), ("q", dv["q"]), ("k", dv["k"]), ("gate", dv["gate"])):
            assert torch.equal(val.cpu().view(torch.int16), want[key].view(torch.int16)), key


@pytest.mark.parametrize("rows,devices", [(1000, [0, 0, 0]), (5, [0, 0, 0, 0, 0, 0, 0, 0]), (2500, [0, 1]), (0, [0, 0])])
def test_host_multi_matches_one_device(vv, rows, devices):
    """vvb_layer_chain_host_multi: one pipeline and one host thread per listed
    device, rows sharded by vvb_shard_rows with the shard's first row as RoPE's
    offset; the bytes are those of the one-device path. Listing a device more
    than once puts several pipelines on it (which exercises the sharding and the
    threads on a single GPU); [0, 1] needs two GPUs. More devices than rows
    leaves the last shards empty."""
    if max(devices) >= torch.cuda.device_count():
        pytest.skip("needs more visible GPUs")
    first = 77
    t = make_inputs(max(rows, 1), rows + 3)
    if rows == 0:
        t = {k: (v[:0] if k != "w" else v) for k, v in t.items()}
    want = run_on_device(vv, t, rows, first) if rows else None
    pin = {k: v.clone().pin_memory() for k, v in t.items()}
    n = torch.empty(rows, H, dtype=torch.float16).pin_memory()
    pipe = vv.HostPipelineMulti(devices, 256, H, NQ, NKV, HD, INTER)
    assert pipe.devices() == len(devices)
    c = vv.make_chain(pin["h"], pin["d"], pin["w"], n, pin["q"], pin["k"], pin["gate"], pin["up"], rows, H, NQ, NKV,
                      HD, INTER, first, 1e-6, 1e6)
    for _ in range(2):                                       # a context is reusable
        for k in ("h", "q", "k", "gate"):
            pin[k].copy_(t[k])
        assert pipe.run(c) == 0
        if rows:
            for got, key in ((pin["h"], "h"), (n, "n"), (pin["q"], "q"), (pin["k"], "k"), (pin["gate"], "gate")):
                assert torch.equal(got.view(torch.int16), want[key].view(torch.int16)), key
    h2d, d2h = pipe.last_traffic()
    assert d2h == rows * 2 * (2 * H + (NQ + NKV) * HD + INTER)
    busy = sum(1 for g in range(len(devices)) if vv.vvb_shard_rows(rows, len(devices), g)[1] > 0)
    assert h2d == rows * 2 * (2 * H + (NQ + NKV) * HD + 2 * INTER) + 2 * H * busy   # gamma goes to every device with rows
    pipe.close()
    torch.cuda.set_device(0)
