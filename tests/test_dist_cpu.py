"""Multi-process tests on CPU (gloo): layout, TP / EP baselines, pipeline stages, data parallel."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(what: str, nproc: int, port: int):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "cpu_dist_worker.py"), what]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "CPU_DIST_WORKER_OK" in r.stdout, r.stderr[-4000:]


@pytest.mark.parametrize("what,nproc,port", [("groups", 4, 29701), ("tp", 2, 29702), ("ep", 2, 29703), ("pp", 3, 29704), ("dp", 2, 29705), ("cp", 3, 29706), ("hybrid", 2, 29707), ("m3ep", 3, 29708)])
def test_cpu_ranks(what, nproc, port):
    _launch(what, nproc, port)
