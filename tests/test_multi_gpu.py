"""Multi-GPU tests: fabric collectives and expert parallelism, run as child processes (one per GPU)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(what: str, nproc: int, port: int):
    env = dict(os.environ)
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "multi_gpu_worker.py"), what]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    if r.returncode != 0:
        log_dir = os.environ.get("GB_TEST_LOG_DIR", "")        # where to leave the workers' output of a failed run
        if log_dir and os.path.isdir(log_dir):
            with open(os.path.join(log_dir, f"multi_gpu_{what}.log"), "w") as f:
                f.write(r.stdout + "\n---- stderr ----\n" + r.stderr)
    assert r.returncode == 0 and "MULTI_GPU_WORKER_OK" in r.stdout, (r.stdout[-3000:], r.stderr[-6000:])


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
def test_fabric_collectives():
    _launch("collectives", min(_ngpu(), 8), 29611)


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
def test_expert_parallel_matches_single_gpu():
    _launch("ep", min(_ngpu(), 8), 29612)


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
def test_tensor_parallel_matches_single_gpu():
    _launch("tp", 2, 29613)


@pytest.mark.skipif(_ngpu() < 4, reason="needs at least 4 GPUs")
def test_tensor_parallel_four_ranks_replicated_kv_heads():
    _launch("tp4", 4, 29615)


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
def test_tensor_parallel_attention_with_expert_parallel_experts():
    _launch("hybrid", 2, 29616)


@pytest.mark.skipif(_ngpu() < 2, reason="needs at least 2 GPUs")
def test_context_parallel_decode_attention():
    _launch("cp", min(_ngpu(), 8), 29614)
