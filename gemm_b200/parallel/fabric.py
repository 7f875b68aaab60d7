"""NVLink fabric: a symmetric heap shared by the ranks of one node, and the collectives that run as our own
kernels over peer memory (csrc/fabric/fabric.cu).

Every rank allocates one device buffer of the same size, exports it with CUDA IPC and maps the buffers of
its peers; ``torch.distributed`` is used only to pass the 64-byte handles around (the role the reference's
TCP rendezvous plays in common/comm.h:416-531).  Sub-buffers are carved with a bump allocator, so as long as
all ranks allocate in the same order an offset names the same object everywhere.  A flag pad lives in the
heap too; flags carry epoch numbers kept in device memory, so captured CUDA graphs replay correctly.

This replaces common/comm.h, common/parallel.h's collective calls and a64fx/utofu-tests/tp_allreduce.h.  A
wait that runs out of time does not hang and does not kill the process: the kernel records the failure in the
status word (``gemm_b200._native.read_status``) and returns.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native

_c, _i, _l, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_size_t


class _CudaView:
    """Exposes a raw device pointer through ``__cuda_array_interface__`` so that torch can wrap it."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}
        self._owner = owner


class Fabric:
    def __init__(self, group, device: torch.device, heap_bytes: int = 64 << 20):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device
        if self.world > 8:
            raise ValueError("the fabric covers the GPUs of one NVSwitch domain (at most 8 ranks)")
        lib = _native.cuda()
        self.lib = lib
        self.heap_bytes = (heap_bytes + 4095) // 4096 * 4096
        base = ctypes.c_void_p()
        _native.check(lib.gb_fabric_alloc(_sz(self.heap_bytes), ctypes.byref(base)), "gb_fabric_alloc", n=0)
        self.local_base = base.value
        handle = (ctypes.c_ubyte * 64)()
        _native.check(lib.gb_ipc_get(_c(self.local_base), handle), "gb_ipc_get", n=0)
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.bases: List[int] = []
        for r in range(self.world):
            if r == self.rank:
                self.bases.append(self.local_base)
            else:
                p = ctypes.c_void_p()
                buf = (ctypes.c_ubyte * 64).from_buffer_copy(handles[r])
                _native.check(lib.gb_ipc_open(buf, ctypes.byref(p)), "gb_ipc_open", n=0)
                self.bases.append(p.value)
        self.bases_arr = (ctypes.c_void_p * 8)(*([ctypes.c_void_p(b) for b in self.bases] + [ctypes.c_void_p(0)] * (8 - self.world)))
        self._bump = 0
        self._heap_t = torch.as_tensor(_CudaView(self.local_base, self.heap_bytes, self), device=device)
        # control words (device-local, not shared): epoch counters and completion counters
        self._ctl = torch.zeros(1024, dtype=torch.int32, device=device)
        self._ctl_next = 0
        # a barrier channel
        self._bar_flags = self.alloc(8 * 4)
        self._bar_epoch = self.ctl_word()
        dist.barrier(group=group)
        torch.cuda.synchronize()

    # ------------------------------------------------------------------------------------------ allocation
    def alloc(self, nbytes: int, align: int = 1024) -> int:
        """Offset of a fresh symmetric sub-buffer (same value on every rank when called in the same order)."""
        off = (self._bump + align - 1) // align * align
        if off + nbytes > self.heap_bytes:
            raise MemoryError(f"symmetric heap exhausted: {off + nbytes} > {self.heap_bytes}")
        self._bump = off + nbytes
        return off

    def view(self, off: int, shape, dtype) -> torch.Tensor:
        """Tensor view of this rank's part of a symmetric sub-buffer."""
        n = int(torch.tensor(shape).prod().item()) * torch.empty(0, dtype=dtype).element_size()
        if off < 0 or off + n > self.heap_bytes:
            raise IndexError(f"view [{off}, {off + n}) leaves the symmetric heap of {self.heap_bytes} bytes")
        return self._heap_t[off:off + n].view(dtype).view(*shape)

    def peer_ptr(self, rank: int, off: int) -> int:
        return self.bases[rank] + off

    def ctl_word(self) -> int:
        """Device address of a fresh zeroed 32-bit control word (epoch or completion counter)."""
        if self._ctl_next >= self._ctl.numel():
            raise MemoryError("out of control words")
        p = self._ctl.data_ptr() + 4 * self._ctl_next
        self._ctl_next += 1
        return p

    # ------------------------------------------------------------------------------------------ collectives
    def _stream(self):
        return _c(torch.cuda.current_stream().cuda_stream)

    def barrier(self) -> None:
        """Device-side barrier of the ranks (a kernel on the current stream, no host blocking)."""
        rc = self.lib.gb_fabric_barrier(self.bases_arr, _i(self.world), _i(self.rank), _sz(self._bar_flags), _c(self._bar_epoch),
                                        _c(_native.status_ptr()), self._stream())
        _native.check(rc, "gb_fabric_barrier")

    def make_allreduce(self, max_elems: int, dtype: torch.dtype, chunks: int = 8) -> "OneShotAllReduce":
        return OneShotAllReduce(self, max_elems, dtype, chunks)

    def make_allreduce_large(self, n_elems: int, dtype: torch.dtype, chunks: int = 296) -> "TwoShotAllReduce":
        return TwoShotAllReduce(self, n_elems, dtype, chunks)

    def make_exchange(self, bytes_per_dst: int, chunks: int = 0, handshake: bool = True) -> "PushExchange":
        """``chunks`` = CTAs of the push kernel (0: by size, one per 32 KB per destination, between 8 and 296).  ``handshake``: every
        call first waits until all peers have entered it, so back-to-back calls cannot overwrite a receive buffer that a peer
        still reads; switch it off only where another exchange between two calls already orders the ranks."""
        if chunks <= 0:
            chunks = max(8, min(296, bytes_per_dst // (32 << 10)))
        return PushExchange(self, bytes_per_dst, chunks, handshake)

    def make_argmax(self, max_rows: int) -> "ArgmaxAllReduce":
        return ArgmaxAllReduce(self, max_rows)

    def close(self) -> None:
        torch.cuda.synchronize()
        for r, b in enumerate(self.bases):
            if r != self.rank and b:
                self.lib.gb_ipc_close(_c(b))
        self.bases = []


class OneShotAllReduce:
    """Latency-bound sum all-reduce (decode): push to every peer, sum in rank order -> identical bits on all ranks."""

    def __init__(self, fab: Fabric, max_elems: int, dtype: torch.dtype, chunks: int):
        self.fab, self.dtype, self.chunks = fab, dtype, chunks
        esz = 4 if dtype == torch.float32 else 2
        self.max_elems = (max_elems * esz + 15) // 16 * 16 // esz
        # two slot sets used alternately (by call parity): a rank that is one call ahead never overwrites what a peer still sums
        self.parity_stride = (fab.world * self.max_elems * esz + 1023) // 1024 * 1024
        self.data_off = fab.alloc(2 * self.parity_stride)
        self.flags_off = fab.alloc(fab.world * chunks * 4)
        self.epoch, self.done = fab.ctl_word(), fab.ctl_word()

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        assert x.dtype == self.dtype and x.is_contiguous() and x.numel() <= self.max_elems
        out = out if out is not None else torch.empty_like(x)
        f = self.fab
        rc = f.lib.gb_allreduce_oneshot(f.bases_arr, _i(f.world), _i(f.rank), _sz(self.data_off), _sz(self.flags_off), _c(x.data_ptr()),
                                        _c(out.data_ptr()), _l(x.numel()), _l(self.max_elems), _i(0 if self.dtype == torch.float32 else 1),
                                        _i(self.chunks), _c(self.epoch), _c(self.done), _c(_native.status_ptr()), _sz(self.parity_stride),
                                        f._stream())
        _native.check(rc, "gb_allreduce_oneshot")
        return out


class TwoShotAllReduce:
    """Bandwidth-bound sum all-reduce (prefill): reduce-scatter by peer loads + all-gather by peer stores.
    Input and output live in the symmetric heap (``input_view`` / ``output_view``)."""

    def __init__(self, fab: Fabric, n_elems: int, dtype: torch.dtype, chunks: int):
        self.fab, self.dtype, self.chunks = fab, dtype, chunks
        esz = 4 if dtype == torch.float32 else 2
        unit = 16 * fab.world // esz
        self.n = (n_elems + unit - 1) // unit * unit
        self.in_off = fab.alloc(self.n * esz)
        self.out_off = fab.alloc(self.n * esz)
        self.flags_off = fab.alloc(2 * fab.world * chunks * 4)
        self.epoch, self.done = fab.ctl_word(), fab.ctl_word()
        self.input_view = fab.view(self.in_off, (self.n,), dtype)
        self.output_view = fab.view(self.out_off, (self.n,), dtype)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        n = x.numel()
        assert n <= self.n
        if x.data_ptr() != self.input_view.data_ptr():          # a producer that wrote straight into ``input_view`` skips this copy
            self.input_view[:n].copy_(x.reshape(-1))
        if n < self.n:
            self.input_view[n:].zero_()
        f = self.fab
        rc = f.lib.gb_allreduce_twoshot(f.bases_arr, _i(f.world), _i(f.rank), _sz(self.in_off), _sz(self.out_off), _sz(self.flags_off),
                                        _l(self.n), _i(0 if self.dtype == torch.float32 else 1), _i(self.chunks), _c(self.epoch),
                                        _c(self.done), _c(_native.status_ptr()), f._stream())
        _native.check(rc, "gb_allreduce_twoshot")
        return self.output_view[:n].view(x.shape)


class PushExchange:
    """All-gather (``stride = 0``) or all-to-all (``stride = bytes_per_dst``) by peer stores."""

    def __init__(self, fab: Fabric, bytes_per_dst: int, chunks: int, handshake: bool = True):
        self.fab, self.chunks = fab, chunks
        self.bytes_per_dst = (bytes_per_dst + 15) // 16 * 16
        self.out_off = fab.alloc(fab.world * self.bytes_per_dst)
        self.flags_off = fab.alloc(fab.world * chunks * 4)
        self.ack_off = fab.alloc(8 * 4) if handshake else 0
        self.epoch, self.done = fab.ctl_word(), fab.ctl_word()
        self.out_view = fab.view(self.out_off, (fab.world, self.bytes_per_dst), torch.uint8)

    def _run(self, x: torch.Tensor, stride: int) -> torch.Tensor:
        f = self.fab
        rc = f.lib.gb_push_exchange(f.bases_arr, _i(f.world), _i(f.rank), _sz(self.out_off), _sz(self.flags_off), _c(x.data_ptr()),
                                    _sz(self.bytes_per_dst), _sz(stride), _i(self.chunks), _c(self.epoch), _c(self.done),
                                    _c(_native.status_ptr()), _sz(self.ack_off), f._stream())
        _native.check(rc, "gb_push_exchange")
        return self.out_view

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """``x`` (contiguous, exactly bytes_per_dst bytes) -> uint8 [world, bytes_per_dst] (a view of the heap)."""
        assert x.is_contiguous() and x.numel() * x.element_size() == self.bytes_per_dst
        return self._run(x, 0)

    def all_to_all(self, x: torch.Tensor) -> torch.Tensor:
        """``x`` [world, ...] with bytes_per_dst bytes per destination -> what every rank sent to this one."""
        assert x.is_contiguous() and x.numel() * x.element_size() == self.bytes_per_dst * self.fab.world
        return self._run(x, self.bytes_per_dst)


class ArgmaxAllReduce:
    """(value, index) arg-max over ranks, ties to the lower index: the merge step of a vocabulary-sharded LM head
    (reference: tp_allreduce_argmax, a64fx/utofu-tests/tp_allreduce.h:326-349)."""

    def __init__(self, fab: Fabric, max_rows: int):
        self.fab, self.max_rows = fab, max_rows
        self.parity_stride = (fab.world * max_rows * 8 + 1023) // 1024 * 1024      # two slot sets, alternating by call
        self.data_off = fab.alloc(2 * self.parity_stride)
        self.flags_off = fab.alloc(fab.world * 4)
        self.epoch = fab.ctl_word()

    def __call__(self, val: torch.Tensor, idx: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        rows = val.numel()
        out_i = torch.empty(rows, dtype=torch.int32, device=val.device)
        out_v = torch.empty(rows, dtype=torch.float32, device=val.device)
        f = self.fab
        rc = f.lib.gb_argmax_allreduce(f.bases_arr, _i(f.world), _i(f.rank), _sz(self.data_off), _sz(self.flags_off), _c(val.data_ptr()),
                                       _c(idx.data_ptr()), _c(out_i.data_ptr()), _c(out_v.data_ptr()), _i(rows), _i(self.max_rows),
                                       _c(self.epoch), _c(_native.status_ptr()), _sz(self.parity_stride), f._stream())
        _native.check(rc, "gb_argmax_allreduce")
        return out_i, out_v
