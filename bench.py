#!/usr/bin/env python
"""bench.py -- the layer chain (residual add + RMSNorm, RoPE on Q/K, SwiGLU) at
long-prompt prefill: T = 14449 tokens of the Qwen2-7B shape, token-sharded over
the GPUs of one box with no collective on the data path.

  python bench.py [--gpus N] [--steps K] [--warmup W]        # this library
  python bench.py --impl reference [...]                     # the reference's CPU kernels

A step is one pass of the three kernels over the rank's rows. `value` is
aggregate tokens/s with inputs resident in HBM (CUDA events, max over ranks);
`e2e` is the same metric through the host-buffer API with the host->device and
device->host copies of every step inside the timed region. `roofline` is for
the one kernel of the timed region (the chain's three operations share a
grid); `chain_ops_separately` times the three entry points alone, and on one
GPU `kernels` lists every kernel family at the shapes of the benchmark
configurations (bench_kernels.py), the one-token decode sequence included.
Every K-step pass is repeated (at least 15 times, and until the timed passes
add up to a quarter of a second); `ms_per_step` is the median pass.
For N > 1 launch under torch.distributed.run (one rank per GPU); a bare
`--gpus N` re-launches itself that way.

Synthetic data: seeded N(0,1) FP16 activations, gamma ~ N(1, 0.02), in the
model's shapes; there are no weights on this path.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "vibevoice.c_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

# Qwen2-7B decoder shape and the prompt length of the reference's long-file run
T_TOTAL, H, NQ, NKV, HD, INTER = 14449, 3584, 28, 4, 128, 18944
EPS, THETA, SEED = 1e-6, 1e6, 1
# algorithmic bytes per token: every tensor read once and written once, FP16
BYTES_ADDNORM = 4 * H * 2                 # read h, delta; write h', normed      28 672
BYTES_ROPE = 2 * (NQ + NKV) * HD * 2      # read + write Q and K                 16 384
BYTES_SWIGLU = 3 * INTER * 2              # read gate, up; write out            113 664
BYTES_CHAIN = BYTES_ADDNORM + BYTES_ROPE + BYTES_SWIGLU   #                     158 720
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per token per launch seen by ncu (dram__bytes_read.sum +
# dram__bytes_write.sum at T = 14449, one launch of each kernel). Reads equal
# the algorithmic reads; writes are ~55 MB short of the algorithmic writes
# because the last lines written are still dirty in L2 when the kernel ends.
# Scaled by rows for other sizes.
NCU_DRAM_BYTES_PER_TOKEN = {"layer_chain": 155230, "swiglu": 110050, "add_rmsnorm": 24590, "rope_qk": 12265}
CPU_SAMPLE_ROWS = 4096


def measured_hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Polls SM clock and throttle reasons of one GPU through NVML (read-only)
    while the benchmark runs."""

    def __init__(self, uuid: str | None, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid) if uuid else pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append((time.perf_counter(), nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self, t0=None, t1=None):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=1.0)
        inside = [m for (t, m) in self.samples if t0 is None or (t0 <= t <= t1)]
        use = inside if len(inside) >= 3 else [m for _, m in self.samples]
        return {
            "sm_mhz": statistics.median(use) if use else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(use),
            "window": "timed region" if len(inside) >= 3 else "warm-up + timed passes",
        }


# --------------------------------------------------------------------------- CPU legs
def cpu_chain_run(rows: int, steps: int, warmup: int):
    """The reference's CPU path for one layer's elementwise chain on FP32
    activations (src/inference/decoder.c:1463-1473): residual add, RMSNorm,
    RoPE on Q and K, SwiGLU in place. Uses the compiled reference kernels when
    present, else the restatement. Returns (tokens/s, info)."""
    import ctypes as C
    import numpy as np
    import oracle
    rng = np.random.default_rng(SEED)
    f = lambda *s: rng.standard_normal(s, dtype=np.float32)
    h, d, q, k, gate, up = f(rows, H), f(rows, H), f(rows, NQ, HD), f(rows, NKV, HD), f(rows, INTER), f(rows, INTER)
    w = (1 + 0.02 * rng.standard_normal(H)).astype(np.float16)
    normed = np.empty_like(h)
    fp = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    if oracle.have_reference():
        ref = oracle.reference()
        L, kind = ref.lib, "reference"
        threads = ref.threads()          # physical cores, pinned (cpu_kernels.c:303-327)
        simd, cores = ref.simd_name(), ref.physical_cores()

        def step():
            L.vv_residual_add_cpu(fp(h), fp(d), h.size)
            L.vv_rmsnorm_cpu(fp(h), w.ctypes.data, fp(normed), rows, H, C.c_float(EPS))
            L.vv_rope_cpu(fp(q), rows, NQ, HD, 0, C.c_float(THETA))
            L.vv_rope_cpu(fp(k), rows, NKV, HD, 0, C.c_float(THETA))
            L.vv_swiglu_cpu(fp(gate), fp(up), fp(gate), gate.size)
    else:
        R = oracle.restated()
        L, kind = R.lib, "port"
        threads, simd, cores = R.threads(), "scalar", os.cpu_count()
        u16 = C.POINTER(C.c_uint16)

        def step():
            L.orc_residual_add(fp(h), fp(d), h.size)
            L.orc_rmsnorm(fp(h), w.view(np.uint16).ctypes.data_as(u16), fp(normed), rows, H, C.c_float(EPS))
            L.orc_rope(fp(q), rows, NQ, HD, 0, C.c_float(THETA))
            L.orc_rope(fp(k), rows, NKV, HD, 0, C.c_float(THETA))
            L.orc_swiglu(fp(gate), fp(up), fp(gate), gate.size)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    info = {"kind": kind, "cores": threads, "physical_cores": cores, "simd": simd,
            "sample": f"{rows} of {T_TOTAL} rows per pass, {steps} passes after {warmup} warm-up, FP32 activations "
                      f"(the CPU path's type; 2x the FP16 bytes)", "ms_per_pass": 1e3 * dt / steps}
    return rows * steps / dt, info


def run_reference_arm(args):
    """`--impl reference`: the reference's CPU kernels on the box's host cores.
    Rank 0 alone works. The timing runs in a child process whose environment
    has the OpenMP variables removed: torch.distributed.run exports
    OMP_NUM_THREADS=1 to its ranks, and vv_cpu_threads() honours that
    variable (src/cpu/cpu_kernels.c:303-327), which would put the whole CPU
    baseline on one core."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    info = cpu_chain_subprocess(T_TOTAL, args.steps, args.warmup)
    value = info.get("value")
    line = {
        "impl": "reference", "metric": "layer_chain_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": info.get("ms_per_pass"),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": info,
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def cpu_chain_subprocess(rows, steps, warmup):
    """Times the CPU leg in a child process: the reference pins its OpenMP team
    (and the calling thread) to cores, which must not leak into this process,
    and the child must not inherit a launcher's OMP_NUM_THREADS."""
    env = {k: v for k, v in os.environ.items()
           if not (k.startswith("OMP_") or k.startswith("GOMP_") or k.startswith("KMP_") or k == "MKL_NUM_THREADS")}
    env["CUDA_VISIBLE_DEVICES"] = ""
    try:
        out = subprocess.run([sys.executable, os.path.abspath(__file__), "--cpu-worker", f"{rows},{steps},{warmup}"],
                             capture_output=True, text=True, timeout=900, check=True, env=env).stdout
        return json.loads(out.strip().splitlines()[-1])
    except Exception as e:  # the GPU line is still valid without it
        return {"value": None, "unit": "tokens/s", "error": f"{type(e).__name__}: {e}"[:300]}


def cpu_worker(spec):
    rows, steps, warmup = (int(x) for x in spec.split(","))
    value, info = cpu_chain_run(rows, steps, warmup)
    print(json.dumps({"value": value, "unit": "tokens/s", "cores": info["cores"], "kind": info["kind"],
                      "sample": info["sample"], "simd": info["simd"], "physical_cores": info["physical_cores"],
                      "ms_per_pass": info["ms_per_pass"],
                      "omp_num_threads_env": os.environ.get("OMP_NUM_THREADS")}))


def workload_config(n_gpus, scaling="strong", rows=T_TOTAL):
    return {
        "workload": "Qwen2-7B layer chain at long-prompt prefill: add+RMSNorm [T,3584], RoPE Q [T,28,128] K [T,4,128] "
                    "at positions 0..T-1, SwiGLU [T,18944] in place; T=14449, fp16 ~ N(0,1), seed 1",
        "rows_total": rows * (n_gpus if scaling == "weak" else 1),
        "sharding": f"contiguous token rows over {n_gpus} GPU(s), no collective",
        "eps": EPS, "theta": THETA,
        "l2": "inputs larger than L2: every rank's working set exceeds the 126 MB L2 and each pass streams it once",
    }


# --------------------------------------------------------------------------- GPU arm
MIN_REPEATS = 15            # K-step passes timed in one process
MIN_REGION_S = 0.25         # and as many more as it takes for the timed passes to add up to this


def run_native(args):
    import torch
    import torch.distributed as dist
    import vvb200 as vv

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE {world}"
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()

    def reduce(values, op):
        """Element-wise max / sum over ranks of a list of floats (one collective)."""
        if world == 1:
            return list(values)
        t = torch.tensor(list(values), dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM)
        return t.tolist()

    total_rows = args.rows * (world if args.scaling == "weak" else 1)
    first, rows = vv.vvb_shard_rows(total_rows, world, rank)

    # The same seeded tensors on every rank count; each rank draws its own rows
    # (seed, first row) -- values do not affect timing, parity is tested elsewhere.
    gen = torch.Generator(device=dev).manual_seed(SEED + 1000 * rank)
    mk = lambda *s: torch.randn(*s, generator=gen, device=dev).half()
    h, d = mk(rows, H), mk(rows, H)
    w = (1 + 0.02 * torch.randn(H, generator=gen, device=dev)).half()
    q, k = mk(rows, NQ, HD), mk(rows, NKV, HD)
    gate, up = mk(rows, INTER), mk(rows, INTER)
    normed = torch.empty_like(h)
    h0, g0 = h.clone(), gate.clone()
    chain = vv.make_chain(h, d, w, normed, q, k, gate, up, rows, H, NQ, NKV, HD, INTER, first, EPS, THETA)
    stream = torch.cuda.current_stream()

    def restore():
        # the chain works in place; start every pass from the same values
        h.copy_(h0)
        gate.copy_(g0)

    def launch_chain(on_stream):
        vv.check(vv.vvb_layer_chain_dev(chain, on_stream), "vvb_layer_chain_dev")

    # One step = the chain's launches. A timed pass is K steps; the K steps are captured once
    # into ONE CUDA graph and a pass replays it: the kernels of consecutive steps then follow
    # each other as they do inside an engine's captured layer sequence (programmatic edges, the
    # next kernel scheduled while this one drains), not a host-side graph launch apart -- which
    # costs some 3 us a step and is a tenth of a 45 us step when the prompt is sharded over eight.
    K = args.steps
    graph, nodes_per_pass = None, 0
    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            launch_chain(side)                      # warm the library before capture
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            n0 = vv.launch_count()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(K):
                    launch_chain(side)
            nodes_per_pass = vv.launch_count() - n0
        stream.wait_stream(side)

    def run_pass():
        """Exactly K steps."""
        if graph is not None:
            graph.replay()
        else:
            for _ in range(K):
                launch_chain(stream)

    sampler = None
    if rank == 0:
        uuid = None
        try:
            uuid = "GPU-" + str(torch.cuda.get_device_properties(local).uuid)
        except Exception:
            pass
        sampler = ClockSampler(uuid, local)
        sampler.start()

    warm = max(args.warmup, 3)
    warm_passes = -(-warm // K)                  # warm-up runs whole passes: at least `warm` steps
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(warm_passes):
        run_pass()
    e1.record(stream)
    torch.cuda.synchronize()
    est_ms = max(reduce([e0.elapsed_time(e1) / (warm_passes * K)], "max")[0], 1e-3)
    repeats = args.repeats or min(2000, max(MIN_REPEATS, int(MIN_REGION_S * 1e3 / (K * est_ms)) + 1))

    # ---- timed passes: EXACTLY K steps under one CUDA-event pair, a barrier and a
    # synchronize on both sides, `repeats` times; ms_per_step is the median pass
    # (each pass: max over ranks) / K
    launches0 = vv.launch_count()
    pass_ms = []
    t_region0 = time.perf_counter()
    for _ in range(repeats):
        restore()
        torch.cuda.synchronize()
        barrier()
        e0.record(stream)
        run_pass()
        e1.record(stream)
        torch.cuda.synchronize()
        barrier()
        pass_ms.append(e0.elapsed_time(e1))
    t_region1 = time.perf_counter()
    launches = (vv.launch_count() - launches0) if graph is None else nodes_per_pass * repeats
    pass_ms = reduce(pass_ms, "max")
    launches_all = int(reduce([float(launches)], "sum")[0])

    # ---- span pass: repeats x K steps back to back, host clock from the barrier's
    # return to every rank synchronised: start skew between GPUs is inside it
    restore()
    torch.cuda.synchronize()
    barrier()
    t0 = time.perf_counter()
    for _ in range(repeats):
        run_pass()
    torch.cuda.synchronize()
    barrier()
    span_s = reduce([time.perf_counter() - t0], "max")[0]
    clocks = sampler.stop(t_region0, t_region1) if sampler else None

    # ---- the chain's three operations launched separately at this rank's rows (same protocol)
    restore()
    per = separate_ops(torch, vv, (h, d, w, normed, q, k, gate, up), rows, first, stream, reduce, barrier)

    # ---- e2e: host buffers through the pipeline API, copies inside the timed region
    e2e_line = None
    if not args.no_e2e:
        e2e_line = run_e2e(args, vv, torch, (h0, d, w, q, k, g0, up), rows, first, local, total_rows,
                           barrier, reduce)

    kernels = None
    if world == 1 and not args.no_kernels:
        del h, d, q, k, gate, up, normed, h0, g0
        torch.cuda.empty_cache()
        import bench_kernels
        kernels = bench_kernels.run(*measured_hbm_peak())

    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return
    emit(args, world, total_rows, pass_ms, span_s, repeats, per, launches_all, clocks, e2e_line, kernels)


def separate_ops(torch, vv, tensors, rows, first, stream, reduce, barrier):
    """add+RMSNorm, RoPE and SwiGLU as three entry points, each ALONE: 20 launches
    back to back under one event pair (no event between launches), five times,
    median. One operation's own tensors are smaller than the whole chain's and, on
    a shard of the prompt, fit the 126 MB L2; so each operation rotates over as
    many copies of its tensors as it takes for 2.5x the L2 to lie between two
    uses of the same copy (1 copy where one already exceeds that)."""
    h, d, w, normed, q, k, gate, up = tensors
    L2_BYTES = 126e6

    def copies(ts):
        per = sum(t.numel() * t.element_size() for t in ts)
        n = max(1, min(24, int(2.5 * L2_BYTES / max(per, 1)) + 1)) if per < 2.5 * L2_BYTES else 1
        return [ts] + [tuple(t.clone() for t in ts) for _ in range(n - 1)]

    sets = {"add_rmsnorm": copies((h, d, normed)), "rope_qk": copies((q, k)), "swiglu": copies((gate, up))}
    ops = {
        "add_rmsnorm": lambda s: vv.check(vv.vvb_add_rmsnorm_dev(s[0], s[1], w, s[2], rows, H, EPS, stream)),
        "rope_qk": lambda s: vv.check(vv.vvb_rope_qk_dev(s[0], s[1], rows, NQ, NKV, HD, first, None, THETA, stream)),
        "swiglu": lambda s: vv.check(vv.vvb_swiglu_dev(s[0], s[1], s[0], rows * INTER, stream)),
    }
    out = {}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name, fn in ops.items():
        ring = sets[name]
        for i in range(max(3, len(ring))):
            fn(ring[i % len(ring)])
        res = []
        for _ in range(5):
            torch.cuda.synchronize()
            barrier()
            e0.record(stream)
            for i in range(20):
                fn(ring[i % len(ring)])
            e1.record(stream)
            torch.cuda.synchronize()
            res.append(e0.elapsed_time(e1) / 20)
        out[name] = statistics.median(reduce(res, "max"))
        out[name + "_copies"] = len(ring)
        del ring
        sets[name] = None
    return out


class numa_local:
    """While inside: this thread runs on the CPUs of the NUMA node the GPU hangs off, so the pages
    of host buffers allocated AND first touched inside land in that node's memory (Linux places a
    page on the node of the thread that first touches it). The affinity is put back on exit. A box
    that does not say where the GPU sits (no sysfs entry, node -1, one node) is left alone."""

    def __init__(self, torch, local):
        self.info = {"gpu_numa_node": None, "bound": False}
        self.saved = None
        self.cpus = set()
        try:
            pr = torch.cuda.get_device_properties(local)
            bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
            node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read())
            self.info["gpu_numa_node"] = node
            if node >= 0:
                cpus = set()
                for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
                    lo, _, hi = part.partition("-")
                    cpus.update(range(int(lo), int(hi or lo) + 1))
                self.cpus = cpus & os.sched_getaffinity(0)
            else:
                self.cpus = set()
        except Exception:            # no such device property, no sysfs entry, an unreadable list
            self.cpus = set()

    def __enter__(self):
        if self.cpus and self.cpus != os.sched_getaffinity(0):
            self.saved = os.sched_getaffinity(0)
            os.sched_setaffinity(0, self.cpus)
            self.info["bound"] = True
            self.info["cpus_on_node"] = len(self.cpus)
        return self

    def __exit__(self, *exc):
        if self.saved is not None:
            os.sched_setaffinity(0, self.saved)
        return False



def copy_ceiling(torch, local, h2d_bytes, d2h_bytes, barrier, reduce, rounds=3):
    """What the box's host<->device path gives this rank while every rank does
    the same: plain cudaMemcpyAsync of the step's byte counts from and to pinned
    memory, uploads on one stream and downloads on another, no kernels. The
    copies go in 64 MiB pieces (one call per piece)."""
    piece = 64 << 20
    with numa_local(torch, local):
        hb = torch.zeros(piece, dtype=torch.uint8).pin_memory()
        hb2 = torch.zeros(piece, dtype=torch.uint8).pin_memory()
    db = torch.empty(piece, dtype=torch.uint8, device="cuda")
    db2 = torch.empty(piece, dtype=torch.uint8, device="cuda")
    s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))

    def one_round():
        torch.cuda.synchronize()
        barrier()
        e0.record(s_up)
        s_down.wait_event(e0)
        left = h2d_bytes
        with torch.cuda.stream(s_up):
            while left > 0:
                n = min(piece, left)
                db[:n].copy_(hb[:n], non_blocking=True)
                left -= n
            e1.record(s_up)
        left = d2h_bytes
        with torch.cuda.stream(s_down):
            while left > 0:
                n = min(piece, left)
                hb2[:n].copy_(db2[:n], non_blocking=True)
                left -= n
            e2.record(s_down)
        torch.cuda.synchronize()
        return max(e0.elapsed_time(e1), e0.elapsed_time(e2))

    one_round()
    ms = statistics.median(reduce([one_round() for _ in range(rounds)], "max"))
    return ms


def run_e2e(args, vv, torch, tensors, rows, first, local, total_rows, barrier, reduce):
    h0, d, w, q, k, g0, up = tensors
    pin = lambda t: t.cpu().pin_memory()
    with numa_local(torch, local) as numa:
        hh, hd_, hw, hq, hk, hg, hu = (pin(t) for t in (h0, d, w, q, k, g0, up))
        hn = torch.zeros_like(hh).pin_memory()
    pipe = vv.HostPipeline(local, args.slice_rows, H, NQ, NKV, HD, INTER)
    hchain = vv.make_chain(hh, hd_, hw, hn, hq, hk, hg, hu, rows, H, NQ, NKV, HD, INTER, first, EPS, THETA)
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    for _ in range(2):
        vv.check(pipe.run(hchain), "vvb_layer_chain_host")
    dev_ms, wall_ms = [], []
    for _ in range(e2e_steps):
        barrier()
        t0 = time.perf_counter()
        vv.check(pipe.run(hchain), "vvb_layer_chain_host")
        wall_ms.append(1e3 * (time.perf_counter() - t0))
        dev_ms.append(pipe.last_ms())
    h2d, d2h = pipe.last_traffic()
    barrier()
    dev_ms = reduce(dev_ms, "max")           # per step: the slowest rank
    wall_ms = reduce(wall_ms, "max")
    h2d_all, d2h_all = (int(x) for x in reduce([float(h2d), float(d2h)], "sum"))
    pipe.close()
    del pipe
    ms = statistics.median(dev_ms)
    ceiling_ms = copy_ceiling(torch, local, h2d, d2h, barrier, reduce)
    return {"value": total_rows / (ms * 1e-3), "unit": "tokens/s",
            "h2d_bytes_per_step": h2d_all, "d2h_bytes_per_step": d2h_all, "steps": e2e_steps,
            "ms_per_step": ms, "ms_min": min(dev_ms), "ms_max": max(dev_ms),
            "wall_ms_per_step": statistics.median(wall_ms),
            "ceiling": {"value": total_rows / (ceiling_ms * 1e-3), "unit": "tokens/s", "ms_per_step": ceiling_ms,
                        "what": "every rank copying its step's bytes host->device and device->host at once with "
                                "plain cudaMemcpyAsync from/to pinned memory, no kernels"},
            "frac_of_ceiling": ceiling_ms / ms,
            "host_buffers": {"pinned": True, "numa": numa.info,
                             "what": "allocated and first touched on the CPUs of the GPU's NUMA node when the box "
                                     "names one"},
            "api": "vvb_layer_chain_host (pinned host tensors; uploads, kernels and downloads pipelined in "
                   f"{args.slice_rows}-row slices)"}


def emit(args, world, total_rows, pass_ms, span_s, repeats, per, launches_all, clocks, e2e_line, kernels):
    peak, peak_kind = measured_hbm_peak()
    K = args.steps
    rows_max = -(-total_rows // world)       # the slowest rank holds ceil(T/N) rows
    ms_step = statistics.median(pass_ms) / K
    ops = {}
    for name, bpt in (("add_rmsnorm", BYTES_ADDNORM), ("rope_qk", BYTES_ROPE), ("swiglu", BYTES_SWIGLU)):
        gbs = bpt * rows_max / (per[name] * 1e-3) / 1e9
        ops[name] = {"us": per[name] * 1e3, "GB/s": gbs, "frac_of_" + peak_kind: gbs / peak,
                     "frac_of_nominal_8TBs": gbs / 8000.0, "algorithmic_bytes_per_launch": bpt * rows_max,
                     "buffer_sets": per.get(name + "_copies", 1)}
    # The timed region launches ONE kernel per step (layer_chain_kernel: the three operations share a
    # grid), so that kernel is the dominant one; `chain_ops_separately` times the three entry points alone.
    chain_gbs = BYTES_CHAIN * rows_max / (ms_step * 1e-3) / 1e9
    traffic = NCU_DRAM_BYTES_PER_TOKEN["layer_chain"]
    value = total_rows / (ms_step * 1e-3)
    value_span = total_rows * repeats * K / span_s
    line = {
        "metric": "layer_chain_tokens_per_s", "value": value,
        "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f16 storage, f32 arithmetic (f64 sum of squares)", "data": "synthetic",
        "config": workload_config(world, args.scaling, args.rows),
        "timing": {"repeats": repeats, "what": "each repeat = exactly K steps under one CUDA-event pair, barrier + "
                   "synchronize on both sides, max over ranks; ms_per_step = median repeat / K",
                   "ms_per_step_min": min(pass_ms) / K, "ms_per_step_max": max(pass_ms) / K,
                   "spread": (max(pass_ms) - min(pass_ms)) / statistics.median(pass_ms),
                   "timed_region_s": sum(pass_ms) * 1e-3,
                   "value_span": value_span, "span_s": span_s,
                   "span_what": "host clock from a barrier's return to every rank synchronised, over "
                                f"{repeats * K} steps issued back to back (start skew between GPUs is inside it)",
                   "span_over_events": value_span / value},
        "roofline": {"bound": "hbm", "kernel": "layer_chain_kernel (add+RMSNorm | RoPE Q,K | SwiGLU in one grid)",
                     "achieved": chain_gbs, "peak": peak, "unit": "GB/s", "frac": chain_gbs / peak,
                     "peak_kind": "of " + peak_kind, "frac_of_nominal_8TBs": chain_gbs / 8000.0,
                     "algorithmic_bytes_per_launch": BYTES_CHAIN * rows_max,
                     "traffic": None if traffic is None else traffic * rows_max,
                     "timing": "CUDA events around K launches on the launching stream "
                               "(ms_per_step is the kernel's average duration, launch gaps included)"},
        "chain_ops_separately": ops,
        "e2e": e2e_line,
        "gpu_launches": launches_all,
        "launch_mode": ("direct" if args.no_graph else "one CUDA graph replay per timed pass of K steps") +
                       f" ({launches_all // max(1, K * repeats * world)} kernel launch(es) per step per GPU: the chain's "
                       "three operations share one grid); gpu_launches counts all timed repeats",
        "clocks": clocks,
    }
    if kernels is not None:
        line["kernels"] = kernels["cases"]
        line["kernels_method"] = kernels["method"]
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_chain_subprocess(CPU_SAMPLE_ROWS, 20, 2)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--scaling", choices=["strong", "weak"], default="strong",
                    help="strong: T=14449 rows in total (the named config); weak: 14449 rows per GPU")
    ap.add_argument("--slice-rows", type=int, default=1024, help="rows per slice of the host-buffer pipeline")
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every step directly instead of replaying a graph")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer pass (profiling runs)")
    ap.add_argument("--rows", type=int, default=T_TOTAL,
                    help="token rows in total (default: the named config's 14449; smaller for profiler captures)")
    ap.add_argument("--workload", choices=["chain", "kernels"], default="chain",
                    help="chain: the benchmark line (config 5); kernels: one line of per-kernel timings at the "
                         "shapes of configs 1-4 and for the int8 activation quantizers (1 GPU)")
    ap.add_argument("--case", default=None, help="--workload kernels: run only the cases whose name contains this")
    ap.add_argument("--plain-launches", action="store_true",
                    help="--workload kernels: four direct launches per case, no graphs, no timing (profiler captures)")
    ap.add_argument("--repeats", type=int, default=0,
                    help="timed K-step passes (default: at least 15, and enough for a 0.25 s timed region)")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel list of the 1-GPU line")
    ap.add_argument("--cpu-worker", default=None, help=argparse.SUPPRESS)
    args = ap.parse_args()

    if args.cpu_worker:
        return cpu_worker(args.cpu_worker)
    if args.gpus > 1 and "RANK" not in os.environ:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 1000),
               os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.workload == "kernels":
        import torch
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
        torch.cuda.set_device(0)
        import bench_kernels
        return bench_kernels.main(*measured_hbm_peak(), only=args.case, plain=args.plain_launches)
    return run_native(args)


if __name__ == "__main__":
    main()
