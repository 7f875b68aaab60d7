"""In-tree build of the two native libraries.

* ``_lib/libgb_cuda.so``  — every ``csrc/kernels/*.cu`` and ``csrc/fabric/*.cu`` compiled by nvcc for
  sm_100a only (``-gencode arch=compute_100a,code=sm_100a``); plain C ABI, loaded with ctypes.
* ``_lib/libgb_host.so``  — host-side C++ (GGUF reader/writer, quantisers and CPU dequantisers,
  tokenizer, KV block manager, scheduler, CPU engine); builds without CUDA.

The libraries stay inside the package directory so that a copy of the source tree carries them.
A source is recompiled only when it (or any header) is newer than its object file.

Usage:  ``python -m gemm_b200.build [--force] [--verbose] [--host-only] [--sanitize]``
(``--sanitize`` builds ``_lib/libgb_host_san.so``, the host library under ASan + UBSan, instead).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "_lib"
OBJ = ROOT / "_lib" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
    "-Xptxas", "-v", "-diag-suppress", "177,550",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-march=x86-64-v3", "-pthread", "-Wall",
             "-Wno-unused-function"]


def _nvcc() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def _newest_header(dirs) -> float:
    newest = 0.0
    for d in dirs:
        for ext in ("*.h", "*.cuh", "*.hpp", "*.inc"):
            for p in Path(d).rglob(ext):
                newest = max(newest, p.stat().st_mtime)
    return newest


def _compile(cmd, src, obj, verbose):
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = (r.stdout or "") + (r.stderr or "")
    (obj.parent / (obj.name + ".log")).write_text(log)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {src}\n{' '.join(cmd)}\n{log[-6000:]}")
    if verbose:
        print(log)
    return src


def _build_lib(name, sources, compiler_cmd, link_cmd, hdr_time, force, verbose, tag=""):
    OBJ.mkdir(parents=True, exist_ok=True)
    jobs, objs = [], []
    for src in sources:
        obj = OBJ / (src.stem + tag + ("_cu.o" if src.suffix == ".cu" else "_cc.o"))
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time):
            jobs.append((compiler_cmd + ["-c", str(src), "-o", str(obj)], src, obj))
    out = LIB / name
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            for f in [ex.submit(_compile, c, s, o, verbose) for c, s, o in jobs]:
                print(f"[gemm_b200.build] compiled {f.result().name}")
    if jobs or not out.exists():
        r = subprocess.run(link_cmd + [str(o) for o in objs] + ["-o", str(out)], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {name}\n{r.stdout}\n{r.stderr}")
        print(f"[gemm_b200.build] linked {out}")
    return out


SHARED_HEADER = CSRC / "kernels" / "geometry.cuh"      # inline code the host library compiles too (host/geometry_host.cc)


def build_host(force=False, verbose=False) -> Path:
    srcs = sorted((CSRC / "host").glob("*.cc"))
    hdr = max(_newest_header([CSRC / "host"]), SHARED_HEADER.stat().st_mtime)
    cxx = os.environ.get("CXX", "g++")
    return _build_lib("libgb_host.so", srcs, [cxx] + CXX_FLAGS + ["-I", str(CSRC / "host")],
                      [cxx, "-shared", "-pthread"], hdr, force, verbose)


SAN_FLAGS = ["-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer"]


def build_host_sanitized(force=False, verbose=False) -> Path:
    """``_lib/libgb_host_san.so``: the host library under AddressSanitizer + UndefinedBehaviorSanitizer.  A process uses it with
    ``GEMM_B200_HOST_LIB=libgb_host_san.so`` and the ASan runtime preloaded (``sanitizer_runtime()``); tests/test_host_sanitizers.py
    runs the host-side unit tests that way."""
    srcs = sorted((CSRC / "host").glob("*.cc"))
    hdr = max(_newest_header([CSRC / "host"]), SHARED_HEADER.stat().st_mtime)
    cxx = _sanitizer_compiler()
    if cxx is None:
        raise RuntimeError("no C++ compiler with an AddressSanitizer runtime found")
    flags = [f for f in CXX_FLAGS if f != "-O3"] + SAN_FLAGS
    return _build_lib("libgb_host_san.so", srcs, [cxx] + flags + ["-I", str(CSRC / "host")],
                      [cxx, "-shared", "-pthread", "-fsanitize=address,undefined"], hdr, force, verbose, tag="_san")


def _asan_of(cxx: str) -> str:
    try:
        r = subprocess.run([cxx, "-print-file-name=libasan.so"], capture_output=True, text=True)
    except OSError:
        return ""
    p = r.stdout.strip()
    return os.path.realpath(p) if r.returncode == 0 and os.path.isabs(p) and os.path.exists(p) else ""


def _sanitizer_compiler() -> str | None:
    """The first of $CXX, g++ on PATH and /usr/bin/g++ that ships an ASan runtime (a toolchain without one cannot link the build)."""
    for cand in (os.environ.get("CXX"), shutil.which("g++"), "/usr/bin/g++"):
        if cand and _asan_of(cand):
            return cand
    return None


def sanitizer_runtime() -> str:
    """Path of the ASan runtime that must be loaded before the interpreter (``LD_PRELOAD``); empty if no compiler has one."""
    cxx = _sanitizer_compiler()
    return _asan_of(cxx) if cxx else ""


def build_cuda(force=False, verbose=False) -> Path:
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build the sm_100a kernels")
    srcs = sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "fabric").glob("*.cu"))
    hdr = _newest_header([CSRC / "kernels", CSRC / "fabric"])
    inc = ["-I", str(CSRC / "kernels"), "-I", str(CSRC / "fabric")]
    return _build_lib("libgb_cuda.so", srcs, [nvcc] + NVCC_FLAGS + inc,
                      [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a"], hdr, force, verbose)


def build_all(force=False, verbose=False, host_only=False):
    outs = [build_host(force, verbose)]
    if not host_only:
        outs.append(build_cuda(force, verbose))
    return outs


if __name__ == "__main__":
    if "--sanitize" in sys.argv:
        print(build_host_sanitized(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
        sys.exit(0)
    build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv, host_only="--host-only" in sys.argv)
