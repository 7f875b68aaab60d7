"""The host-side C++ (GGUF reader / writer, dequantisers, tokenizer, block manager, scheduler, CPU engine, geometry helpers, image decoders) under
AddressSanitizer + UndefinedBehaviorSanitizer: ``gemm_b200.build.build_host_sanitized`` compiles the same sources into
``_lib/libgb_host_san.so``, and the unit tests of that code run once more in a child interpreter with the ASan runtime
preloaded and ``GEMM_B200_HOST_LIB`` pointing at the instrumented build.  Any report aborts the child."""
import os
import subprocess
import sys

import pytest

from gemm_b200 import build

HERE = os.path.dirname(os.path.abspath(__file__))
FILES = ["test_runtime_cpu.py", "test_gguf_cpu.py", "test_tokenizer_cpu.py", "test_cpu_engine.py", "test_geometry_cpu.py", "test_image_decode_cpu.py"]

CHILD = r"""
import sys, pytest
from gemm_b200 import _native
_native.host()
maps = open("/proc/self/maps").read()
assert "libgb_host_san.so" in maps and "libgb_host.so" not in maps, "the instrumented library is not the one loaded"
sys.exit(pytest.main(sys.argv[1:] + ["-x", "-q", "-p", "no:cacheprovider"]))
"""


def test_host_unit_tests_pass_under_asan_and_ubsan():
    runtime = build.sanitizer_runtime()
    if not runtime:
        pytest.skip("no compiler with an AddressSanitizer runtime on this machine")
    build.build_host_sanitized()
    env = dict(os.environ)
    env.update(LD_PRELOAD=runtime, GEMM_B200_HOST_LIB="libgb_host_san.so",
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=1",           # the interpreter itself never frees everything
               UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1")
    r = subprocess.run([sys.executable, "-c", CHILD] + [os.path.join(HERE, f) for f in FILES], capture_output=True, text=True,
                       env=env, cwd=os.path.dirname(HERE), timeout=900)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-6000:])
    assert "passed" in r.stdout and "failed" not in r.stdout
