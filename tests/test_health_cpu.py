"""Failure detection with failures made on the host (no GPU involved): a rank that leaves, raises or stalls is noticed by
the others through the heartbeat store before their next collective."""
import os
import socket
import subprocess
import sys

import pytest

from gemm_b200.parallel.health import Heartbeat, PeerLost

WORKER = os.path.join(os.path.dirname(__file__), "health_worker.py")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(world, mode):
    port = _free_port()
    procs = [subprocess.Popen([sys.executable, WORKER, str(r), str(world), str(port), mode], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=60)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append((p.returncode, o))
    return outs


class _DictStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_heartbeat_logic_in_process():
    st = _DictStore()
    a, b = Heartbeat(st, 0, 2), Heartbeat(st, 1, 2)
    a.beat(0)
    with pytest.raises(PeerLost) as ei:
        a.check(timeout_s=0.05)
    assert ei.value.ranks == [1]
    b.beat(0)
    a.check(timeout_s=0.05)
    a.beat(1)
    b.leave()
    with pytest.raises(PeerLost) as ei:
        a.check(timeout_s=0.05)
    assert "left" in str(ei.value)


def test_all_ranks_finish_without_failure():
    outs = _run(2, "none")
    assert all(rc == 0 and "DONE" in o for rc, o in outs), outs


@pytest.mark.parametrize("mode", ["leave", "raise", "stall"])
def test_survivors_notice_a_lost_rank(mode):
    world = 3
    outs = _run(world, mode)
    for r in range(world - 1):
        rc, o = outs[r]
        assert rc == 3 and f"PEERLOST [{world - 1}] at step 3" in o, (mode, r, outs)
