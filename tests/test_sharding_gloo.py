"""Token-row sharding on CPU with two (and three) gloo ranks: the N > 1 path
of this library is a row partition with no exchange step, so it is exercised
here with the oracle standing in for the kernels."""
import os
import socket
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(world, mode):
    port = free_port()
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="2", GLOO_SOCKET_IFNAME="lo")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "_gloo_worker.py"), mode],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n<timeout>"
        outs.append((p.returncode, out))
    return outs


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_rows_reassemble_to_the_whole(world):
    outs = launch(world, "ok")
    for rc, out in outs:
        assert rc == 0, out
    assert "sharded == whole" in outs[0][1]


def test_a_rank_that_exits_is_an_error_not_a_hang():
    outs = launch(2, "fail")
    assert outs[1][0] == 3
    assert outs[0][0] != 0 and "<timeout>" not in outs[0][1], outs[0][1]
