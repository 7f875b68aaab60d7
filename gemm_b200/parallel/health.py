"""Failure detection for multi-rank jobs: host-side heartbeats plus the device-side status word.

The reference's one-sided collectives spin on sequence numbers and, after 60 s (all-reduce) or 300 s (barrier), print
rank / wanted / got and ``exit(1)`` (a64fx/utofu-tests/tp_allreduce.h:122-134, a64fx/llm/tp_runner.c:656-659); its socket
back end has no timeout at all once connected (common/comm.h:348-409).  Here a lost peer is noticed in two places:

* **On the host, before the next launch.**  Every rank publishes the step it is about to run in the job's key-value store
  (``Heartbeat.beat``); ``Heartbeat.check`` makes sure that every peer has reached that step within a deadline and has not
  announced that it is leaving, and raises ``PeerLost`` otherwise.  A rank that leaves on purpose (``leave``) does so
  between steps, with none of its kernels or collectives in flight.  A store that stops answering (rank 0 hosts it) counts
  as the loss of rank 0.
* **On the device, inside a kernel that waits for a peer.**  Every wait on a peer's flag is bounded (``kPeerBudgetNs``);
  when it runs out the kernel records (where, peer, wanted, seen) in the status word and returns normally, so the CUDA
  context stays usable.  ``check_device`` turns a non-zero status word into ``DeviceWaitTimeout``.

``guarded`` bundles both around one step of an engine.
"""
from __future__ import annotations

import time
from typing import Callable, Iterable, List, Optional

from .. import _native


class PeerLost(RuntimeError):
    def __init__(self, ranks: Iterable[int], why: str):
        self.ranks = sorted(ranks)
        super().__init__(f"lost rank(s) {self.ranks}: {why}")


class DeviceWaitTimeout(RuntimeError):
    def __init__(self, status: dict):
        self.status = status
        super().__init__(f"a kernel gave up waiting: {status}")


class Heartbeat:
    """Liveness of ``world`` ranks over a ``torch.distributed`` store (TCPStore / FileStore / the default store of a group)."""

    LEFT = b"left"

    def __init__(self, store, rank: int, world: int, prefix: str = "gb_hb"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix
        self.step = -1

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        """Publish that this rank is about to run ``step``."""
        self.step = step
        self.store.set(self._key(self.rank), str(step))

    def leave(self) -> None:
        """Announce an orderly departure (call between steps, after the stream has been synchronised)."""
        self.store.set(self._key(self.rank), self.LEFT)

    def peer_state(self, r: int) -> Optional[bytes]:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            return bytes(self.store.get(self._key(r)))
        except Exception as e:                       # the store itself is gone: its host (rank 0) died
            raise PeerLost([0], f"key-value store unreachable ({type(e).__name__})") from None

    def check(self, step: Optional[int] = None, timeout_s: float = 5.0, poll_s: float = 0.01) -> None:
        """Return once every peer has published a step >= ``step`` (default: this rank's); raise ``PeerLost`` for peers
        that left, and for peers that did not get there within ``timeout_s``."""
        want = self.step if step is None else step
        deadline = time.monotonic() + timeout_s
        pending: List[int] = [r for r in range(self.world) if r != self.rank]
        while True:
            still = []
            for r in pending:
                st = self.peer_state(r)
                if st == self.LEFT:
                    raise PeerLost([r], "it announced that it left the job")
                if st is None or int(st) < want:
                    still.append(r)
            if not still:
                return
            if time.monotonic() > deadline:
                raise PeerLost(still, f"no heartbeat for step {want} within {timeout_s} s")
            pending = still
            time.sleep(poll_s)


def check_device(clear: bool = True) -> None:
    """Synchronise the device and raise ``DeviceWaitTimeout`` if any kernel recorded an expired wait or a failed check."""
    st = _native.read_status(clear=clear)
    if st["code"] != 0:
        raise DeviceWaitTimeout(st)


def guarded(hb: Optional[Heartbeat], step: int, fn: Callable, timeout_s: float = 5.0, device: bool = True):
    """Run one step of a multi-rank job under both detectors: peers must be alive before anything is launched, and the
    status word must be clean afterwards."""
    if hb is not None:
        hb.beat(step)
        hb.check(step, timeout_s)
    out = fn()
    if device:
        check_device()
    return out
