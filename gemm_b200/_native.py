"""ctypes bindings of the two in-tree native libraries.

``cuda()`` returns ``libgb_cuda.so`` (sm_100a kernels, C ABI) and ``host()`` returns ``libgb_host.so``
(GGUF / quantisers / tokenizer / KV manager / scheduler / CPU engine).  Neither is ever replaced by a
silent Python fallback: if a library is missing, the first use raises and names the build command.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent / "_lib"
_cuda = None
_host = None


class NativeLibraryMissing(RuntimeError):
    pass


def _load(name: str):
    path = _LIB_DIR / name
    if not path.exists():
        if os.environ.get("GEMM_B200_AUTOBUILD", "1") != "0":
            from . import build as _build
            if name == "libgb_host.so":
                _build.build_host()
            else:
                _build.build_cuda()
    if not path.exists():
        raise NativeLibraryMissing(f"{path} is missing: run `python -m gemm_b200.build`")
    return ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)


def cuda():
    """The CUDA kernel library (loaded once)."""
    global _cuda
    if _cuda is None:
        lib = _load("libgb_cuda.so")
        lib.gb_last_error.restype = ctypes.c_char_p
        lib.gb_status_ptr.restype = ctypes.c_void_p
        _cuda = lib
    return _cuda


def host():
    """The host-side C++ library (loaded once)."""
    global _host
    if _host is None:
        # GEMM_B200_HOST_LIB names another build of the same sources inside _lib/ (the sanitizer build, build.build_host_sanitized)
        lib = _load(os.environ.get("GEMM_B200_HOST_LIB", "libgb_host.so"))
        lib.gbh_last_error.restype = ctypes.c_char_p
        _host = lib
    return _host


def cuda_available() -> bool:
    return (_LIB_DIR / "libgb_cuda.so").exists()


_launches = 0


def check(rc: int, what: str = "kernel launch", n: int = 1):
    """Raise with the library's message if a native call returned non-zero; count its ``n`` kernel launches."""
    global _launches
    if rc != 0:
        msg = cuda().gb_last_error().decode(errors="replace")
        raise RuntimeError(f"{what} failed: {msg}")
    _launches += n


def launch_count() -> int:
    """Kernels of this library launched (or captured into a graph) so far by this process."""
    return _launches


def loaded_libraries():
    """Paths of the native libraries mapped into this process (for diagnostics)."""
    out = []
    with open("/proc/self/maps") as f:
        for line in f:
            if "libgb_" in line:
                p = line.split()[-1]
                if p not in out:
                    out.append(p)
    return out


_status_ptrs = {}


def status_ptr() -> int:
    """Device address of the status word of the current device (bounded waits report into it)."""
    import torch
    dev = torch.cuda.current_device()
    if dev not in _status_ptrs:
        p = cuda().gb_status_ptr()
        if not p:
            raise RuntimeError("gb_status_ptr failed: " + cuda().gb_last_error().decode())
        _status_ptrs[dev] = p
    return _status_ptrs[dev]


STATUS_NAMES = {0: "ok", 1: "mbarrier wait timed out", 2: "flag wait timed out", 3: "bad argument"}


def read_status(clear: bool = True) -> dict:
    """Synchronise and return the status word as a dict (code 0 = no kernel reported a problem)."""
    buf = (ctypes.c_int * 16)()
    check(cuda().gb_status_read(buf, 1 if clear else 0), "gb_status_read")
    return {"code": buf[0], "what": STATUS_NAMES.get(buf[0], "?"), "where": buf[1], "block": buf[2],
            "aux": (buf[3], buf[4], buf[5]), "count": buf[6]}


def assert_status_ok():
    st = read_status()
    if st["code"] != 0:
        raise RuntimeError(f"a kernel reported a failed wait or check: {st}")
