"""Profiler: named op timers with FLOP / byte counts and per-op, per-type, per-component tables (the shape of the
reference's common/profiler.h:44-77,110-249), fed by CUDA events on the GPU and ``perf_counter`` on the CPU.

    with profiler.region("qkv_proj", "gemm", "attention", layer=3, flops=2*m*n*k):
        ...
    print(profiler.summary())

Profiling is off unless ``GEMM_B200_PROFILE=1`` or ``profiler.enable()``; when off, ``region`` costs one branch.
``GEMM_B200_NVTX=1`` (or ``enable_nvtx()``) makes every region an NVTX range as well (``name[layer]``), whether or not the
timers are on, so that a timeline tool shows the model's structure above the kernels."""
from __future__ import annotations

import contextlib
import ctypes
import os
import time
from typing import List

import torch

from .. import _native

_enabled = os.environ.get("GEMM_B200_PROFILE", "0") == "1"
_nvtx = os.environ.get("GEMM_B200_NVTX", "0") == "1"
_pending: List[tuple] = []


def enable_nvtx(on: bool = True) -> None:
    global _nvtx
    _nvtx = on


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = on


def enabled() -> bool:
    return _enabled


@contextlib.contextmanager
def region(name: str, op_type: str = "op", component: str = "model", layer: int = -1, flops: float = 0.0, nbytes: float = 0.0):
    if _nvtx and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name if layer < 0 else f"{name}[{layer}]")
        try:
            with _timed(name, op_type, component, layer, flops, nbytes):
                yield
        finally:
            torch.cuda.nvtx.range_pop()
        return
    with _timed(name, op_type, component, layer, flops, nbytes):
        yield


@contextlib.contextmanager
def _timed(name, op_type, component, layer, flops, nbytes):
    if not _enabled:
        yield
        return
    if torch.cuda.is_available():
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        yield
        b.record()
        _pending.append((name, op_type, component, layer, a, b, flops, nbytes))
    else:
        t0 = time.perf_counter_ns()
        yield
        _native.host().gbh_prof_add(name.encode(), op_type.encode(), component.encode(), layer, ctypes.c_double(time.perf_counter_ns() - t0),
                                    ctypes.c_double(flops), ctypes.c_double(nbytes))


def _flush() -> None:
    if _pending:
        torch.cuda.synchronize()
        for name, op_type, component, layer, a, b, flops, nbytes in _pending:
            _native.host().gbh_prof_add(name.encode(), op_type.encode(), component.encode(), layer, ctypes.c_double(a.elapsed_time(b) * 1e6),
                                        ctypes.c_double(flops), ctypes.c_double(nbytes))
        _pending.clear()


def summary() -> str:
    _flush()
    lib = _native.host()
    lib.gbh_prof_summary.restype = ctypes.c_long
    buf = ctypes.create_string_buffer(1 << 16)
    lib.gbh_prof_summary(buf, ctypes.c_long(1 << 16))
    return buf.value.decode()


def reset() -> None:
    _pending.clear()
    _native.host().gbh_prof_reset()
