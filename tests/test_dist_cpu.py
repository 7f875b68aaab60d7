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


@pytest.mark.parametrize("what,nproc,port", [("groups", 4, 29701), ("tp", 2, 29702), ("ep", 2, 29703), ("pp", 3, 29704), ("dp", 2, 29705), ("cp", 3, 29706), ("hybrid", 2, 29707), ("m3ep", 3, 29708), ("cpmerge", 4, 29709), ("cpmerge", 3, 29710)])
def test_cpu_ranks(what, nproc, port):
    _launch(what, nproc, port)


def test_ring_attention_benchmark_runs_on_cpu_ranks():
    """The context-parallel decode-attention cost benchmark on 2 gloo ranks: one JSON line with the read, the three merges and the
    projection table; the projection helpers on their own."""
    import json
    from gemm_b200.utils import ringbench
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1", "--master-port", "29711",
           "-m", "gemm_b200.utils.ringbench", "--seq", "256", "--batch", "2", "--qh", "8", "--kvh", "2", "--iters", "3", "--warmup", "1"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="1"), cwd=os.path.dirname(HERE))
    assert r.returncode == 0, r.stderr[-3000:]
    line = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])
    assert line["world"] == 2 and line["config"]["positions_per_rank"] == 128 and line["payload_bytes"] == 2 * 8 * 129 * 4
    assert line["ring_rel_err"] < 1e-2 and line["tree_rel_err"] < 1e-2 and len(line["projection"]) == 7
    rows = ringbench.projection(read_ms=8.0, hop_ms=0.5, round_ms=1.0, world=2)
    assert rows[0] == {"n": 1, "read_ms": 16.0, "ring_ms": 0.0, "tree_ms": 0.0} and rows[3] == {"n": 8, "read_ms": 2.0, "ring_ms": 3.5, "tree_ms": 3.0}
    assert ringbench.crossover(rows, "ring_ms") == 8 and ringbench.crossover(rows, "tree_ms") == 8
    assert ringbench.crossover(ringbench.projection(100.0, 0.001, 0.001, 1), "ring_ms") is None
