"""Python face of the C++ runtime (csrc/host/runtime.cc): paged-KV block manager, continuous-batching scheduler, profiler."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

from .. import _native


def _lib():
    lib = _native.host()
    if not getattr(lib, "_rt_ready", False):
        lib.gbh_kv_create.restype = ctypes.c_void_p
        lib.gbh_sched_create.restype = ctypes.c_void_p
        lib.gbh_sched_num_preempted.restype = ctypes.c_long
        lib.gbh_prof_summary.restype = ctypes.c_long
        lib._rt_ready = True
    return lib


class KvBlockManager:
    """Pages of the KV cache: allocation per sequence, release, fork with shared full pages."""

    def __init__(self, num_pages: int, page_size: int):
        self.num_pages, self.page_size = num_pages, page_size
        self._h = _lib().gbh_kv_create(num_pages, page_size)

    def new_sequence(self) -> int:
        return _lib().gbh_kv_seq_new(ctypes.c_void_p(self._h))

    def reserve(self, seq: int, tokens: int) -> None:
        if _lib().gbh_kv_seq_reserve(ctypes.c_void_p(self._h), seq, tokens) != 0:
            raise MemoryError(_lib().gbh_last_error().decode())

    def release(self, seq: int) -> None:
        _lib().gbh_kv_seq_release(ctypes.c_void_p(self._h), seq)

    def fork(self, seq: int, tokens: int) -> Tuple[int, Optional[Tuple[int, int]]]:
        """New sequence sharing ``tokens`` cached positions; returns (id, (src_page, dst_page) to copy or None)."""
        a, b = ctypes.c_int(), ctypes.c_int()
        nid = _lib().gbh_kv_seq_fork(ctypes.c_void_p(self._h), seq, tokens, ctypes.byref(a), ctypes.byref(b))
        if nid < 0:
            raise MemoryError(_lib().gbh_last_error().decode())
        return nid, ((a.value, b.value) if a.value >= 0 else None)

    def pages(self, seq: int) -> List[int]:
        buf = (ctypes.c_int * 4096)()
        n = _lib().gbh_kv_seq_pages(ctypes.c_void_p(self._h), seq, buf, 4096)
        if n < 0:
            raise KeyError(seq)
        return list(buf[:n])

    @property
    def num_free(self) -> int:
        return _lib().gbh_kv_num_free(ctypes.c_void_p(self._h))

    def refcount(self, page: int) -> int:
        return _lib().gbh_kv_refcount(ctypes.c_void_p(self._h), page)

    def __del__(self):
        try:
            if self._h:
                _lib().gbh_kv_destroy(ctypes.c_void_p(self._h))
                self._h = None
        except Exception:
            pass


@dataclass
class PlanItem:
    req_id: int
    seq: int
    q_len: int
    ctx_len: int
    is_prefill: bool
    emits_token: bool


class Scheduler:
    """Continuous batching: each ``plan()`` is one engine step (decode tokens first, prompt chunks in the rest of the budget)."""

    def __init__(self, kv: KvBlockManager, max_running: int, max_batch_tokens: int):
        self.kv = kv
        self._h = _lib().gbh_sched_create(ctypes.c_void_p(kv._h), max_running, max_batch_tokens)
        self._cap = max_running + 64

    def add(self, req_id: int, prompt_len: int, max_new_tokens: int) -> None:
        """Queue a request.  Raises ``ValueError`` when prompt + generation (+ look-ahead) can never fit the cache."""
        if _lib().gbh_sched_add(ctypes.c_void_p(self._h), ctypes.c_long(req_id), prompt_len, max_new_tokens) != 0:
            raise ValueError(_lib().gbh_last_error().decode())

    def take_aborted(self) -> List[int]:
        """Requests the scheduler dropped since the last call because the cache can never hold them."""
        buf = (ctypes.c_long * 256)()
        n = _lib().gbh_sched_take_aborted(ctypes.c_void_p(self._h), buf, 256)
        return list(buf[:n])

    def plan(self) -> List[PlanItem]:
        c = self._cap
        rid = (ctypes.c_long * c)()
        arrs = [(ctypes.c_int * c)() for _ in range(5)]
        n = _lib().gbh_sched_plan(ctypes.c_void_p(self._h), rid, *arrs, c)
        return [PlanItem(rid[i], arrs[0][i], arrs[1][i], arrs[2][i], bool(arrs[3][i]), bool(arrs[4][i])) for i in range(min(n, c))]

    def commit(self, finished: Sequence[bool], advance: Optional[Sequence[int]] = None) -> None:
        """``advance[i]``: tokens a decode item produced this step (more than one after accepted draft tokens)."""
        arr = (ctypes.c_int * max(1, len(finished)))(*[1 if f else 0 for f in finished])
        if advance is None:
            _lib().gbh_sched_commit(ctypes.c_void_p(self._h), arr, len(finished))
        else:
            adv = (ctypes.c_int * max(1, len(finished)))(*[int(a) for a in advance])
            _lib().gbh_sched_commit_n(ctypes.c_void_p(self._h), arr, adv, len(finished))

    def set_lookahead(self, extra: int) -> None:
        """Decode items reserve (and are budgeted for) ``extra`` more positions: room for draft tokens of speculative decoding."""
        _lib().gbh_sched_set_lookahead(ctypes.c_void_p(self._h), int(extra))

    @property
    def num_waiting(self) -> int:
        return _lib().gbh_sched_num_waiting(ctypes.c_void_p(self._h))

    @property
    def num_running(self) -> int:
        return _lib().gbh_sched_num_running(ctypes.c_void_p(self._h))

    @property
    def num_preempted(self) -> int:
        return _lib().gbh_sched_num_preempted(ctypes.c_void_p(self._h))

    def __del__(self):
        try:
            if self._h:
                _lib().gbh_sched_destroy(ctypes.c_void_p(self._h))
                self._h = None
        except Exception:
            pass
