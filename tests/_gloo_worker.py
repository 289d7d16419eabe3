"""Worker for tests/test_sharding_gloo.py: one CPU rank of a gloo group.

Each rank takes its row block from vvb_shard_rows (the library's C host code),
runs the CPU oracle on that block with the block's first row as RoPE's position
offset, and the ranks gather their blocks on rank 0, which compares the
concatenation with the oracle run over all rows at once. That is the whole
multi-GPU algorithm of this path (no exchange step) with the kernels swapped
for the oracle, so it runs without a GPU.
"""
import datetime
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "vibevoice.c_b200"))
import oracle  # noqa: E402
import vvb200 as vv  # noqa: E402


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    T, H, NQ, HD, INTER = 301, 256, 4, 128, 512
    rng = np.random.default_rng(5)                     # same tensors on every rank
    h = rng.standard_normal((T, H)).astype(np.float16)
    d = rng.standard_normal((T, H)).astype(np.float16)
    w = (1 + 0.02 * rng.standard_normal(H)).astype(np.float16)
    q = rng.standard_normal((T, NQ, HD)).astype(np.float16)
    g = rng.standard_normal((T, INTER)).astype(np.float16)
    u = rng.standard_normal((T, INTER)).astype(np.float16)

    first, count = vv.vvb_shard_rows(T, world, rank)
    if mode == "fail" and rank == 1:
        # a rank that dies between steps: the others must see an error, not hang
        os._exit(3)
    sl = slice(first, first + count)
    hn, nn = oracle.add_rmsnorm_f16(h[sl], d[sl], w, 1e-6)
    qn = oracle.rope_f16(q[sl], first, 1e6)            # the shard's first row is its position offset
    on = oracle.swiglu_f16(g[sl], u[sl])
    mine = {"first": first, "count": count, "h": hn, "n": nn, "q": qn, "o": on}
    gathered = [None] * world
    try:
        dist.all_gather_object(gathered, mine)
    except Exception as e:                              # noqa: BLE001
        print(f"rank {rank}: collective failed: {type(e).__name__}", flush=True)
        sys.exit(7)
    if rank == 0:
        assert [p["first"] for p in gathered] == sorted(p["first"] for p in gathered)
        assert sum(p["count"] for p in gathered) == T
        cat = lambda k: np.concatenate([p[k] for p in gathered], axis=0)
        wh, wn = oracle.add_rmsnorm_f16(h, d, w, 1e-6)
        assert np.array_equal(cat("h").view(np.uint16), wh.view(np.uint16))
        assert np.array_equal(cat("n").view(np.uint16), wn.view(np.uint16))
        assert np.array_equal(cat("q").view(np.uint16), oracle.rope_f16(q, 0, 1e6).view(np.uint16))
        assert np.array_equal(cat("o").view(np.uint16), oracle.swiglu_f16(g, u).view(np.uint16))
        print("sharded == whole", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
