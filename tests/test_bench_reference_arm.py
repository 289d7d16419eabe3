"""`bench.py --impl reference` -- the reference's CPU kernels timed as the
baseline arm -- as the benchmark driver launches it: under a
torch.distributed.run-style environment, which exports OMP_NUM_THREADS=1 to
every rank. The arm must still use the box's cores (it times the CPU kernels in
a child process whose environment has the OpenMP variables removed), rank 0
alone prints the line and the other ranks exit 0 without work."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_arm(rank, world):
    env = dict(os.environ, OMP_NUM_THREADS="1", RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
               MASTER_ADDR="127.0.0.1", MASTER_PORT="29591")
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", str(world),
                           "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600, env=env)


def test_reference_arm_ignores_the_launchers_omp_setting():
    r = run_arm(0, 2)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["steps"] == 1
    assert line["metric"] == "layer_chain_tokens_per_s" and line["higher_is_better"] is True
    base = line["cpu_baseline"]
    assert base["value"] == line["value"] > 0
    assert base["omp_num_threads_env"] is None          # the child did not inherit OMP_NUM_THREADS=1
    want = base["physical_cores"] if base["kind"] == "reference" else os.cpu_count()
    assert base["cores"] == want and (want == 1 or base["cores"] > 1)
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_other_ranks_do_nothing():
    r = run_arm(1, 2)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_numa_placement_scope_restores_the_affinity(tmp_path, monkeypatch):
    """bench.py places its pinned host buffers on the GPU's NUMA node by narrowing the thread's CPU
    affinity while it allocates them; a box that names no node is left alone, and the affinity is
    back to what it was on leaving the scope either way."""
    sys.path.insert(0, ROOT)
    import importlib
    bench = importlib.import_module("bench")
    before = os.sched_getaffinity(0)

    class NoGpu:                           # torch.cuda.get_device_properties raises without a device
        class cuda:
            @staticmethod
            def get_device_properties(_):
                raise RuntimeError("no CUDA device")
    with bench.numa_local(NoGpu, 0) as scope:
        assert scope.info == {"gpu_numa_node": None, "bound": False}
        assert os.sched_getaffinity(0) == before
    assert os.sched_getaffinity(0) == before

    # a scope that does narrow the affinity (to one of the CPUs this process may use) undoes it
    scope = bench.numa_local(NoGpu, 0)
    scope.cpus = {min(before)}
    with scope:
        assert os.sched_getaffinity(0) == ({min(before)} if len(before) > 1 else before)
    assert os.sched_getaffinity(0) == before
