"""Child process of tests/test_health_cpu.py: ranks step together under heartbeats; one of them fails on the host."""
import os
import sys
import time
from datetime import timedelta

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from gemm_b200.parallel.health import Heartbeat, PeerLost, guarded  # noqa: E402


def main():
    rank, world, port, mode = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=timedelta(seconds=20))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=timedelta(seconds=20))
    hb = Heartbeat(store, rank, world)
    x = torch.ones(4)
    try:
        for step in range(6):
            if rank == world - 1 and step == 3:
                if mode == "leave":          # orderly: between steps, nothing in flight
                    hb.leave()
                    print(f"rank {rank} LEFT at step {step}", flush=True)
                    time.sleep(1.0)          # keep the process (and a store hosted here) alive while the others notice
                    return 0
                if mode == "raise":          # an exception on the host: the rank never reaches the step
                    raise RuntimeError("injected host failure")
                if mode == "stall":          # never joins the step
                    time.sleep(6)
            def one_step():
                y = x.clone()
                dist.all_reduce(y)
                return float(y[0])
            got = guarded(hb, step, one_step, timeout_s=1.5, device=False)
            assert got == world
        print(f"rank {rank} DONE", flush=True)
        return 0
    except PeerLost as e:
        print(f"rank {rank} PEERLOST {e.ranks} at step {hb.step}", flush=True)
        if rank == 0:
            time.sleep(2.0)      # this rank hosts the store: stay until the other survivors have read the heartbeats too
        return 3
    except RuntimeError as e:
        print(f"rank {rank} FAILED {e}", flush=True)
        return 4


if __name__ == "__main__":
    code = main()
    sys.stdout.flush()
    os._exit(code)           # no process-group teardown: a survivor must not wait for the rank that is gone
