"""The allocation-free arg-max entry point, called through its exported C symbol.

Embedders that may not touch the CUDA allocator (a serving loop that owns all device memory, a plug-in under another
framework's memory manager) use ``gb_argmax_noalloc``: its scratch is a fixed array inside the library.  The test calls it
twice in a row — the scratch is shared between calls and keeps old contents — and checks both results against the regular
two-stage arg-max whose scratch the caller allocates.  The file name sorts last on purpose: it runs after every other test,
and it also passes when run alone in a fresh process.
"""
import ctypes

import pytest
import torch

from gemm_b200 import _native
from gemm_b200.ops import sampling

pytestmark = pytest.mark.gpu


def _call(logits, idx_offset=0):
    lib = _native.cuda()
    fn = lib.gb_argmax_noalloc
    fn.restype = ctypes.c_int
    rows, vocab = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    val = torch.empty(rows, dtype=torch.float32, device=logits.device)
    rc = fn(ctypes.c_void_p(logits.data_ptr()), ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(val.data_ptr()), ctypes.c_int(rows),
            ctypes.c_int(vocab), ctypes.c_long(logits.stride(0)), ctypes.c_int(0 if logits.dtype == torch.float32 else 1),
            ctypes.c_int(idx_offset), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out, val


def test_no_alloc_argmax_matches_regular_entry_point_twice():
    torch.manual_seed(0)
    a = torch.randn(64, 151936, device="cuda")
    a[3, 10] = a[3, 90000] = 99.0                              # tie -> lower column
    b = (torch.randn(7, 50000, device="cuda") * 3).bfloat16()
    for logits, off in ((a, 0), (b, 11)):                      # second call reuses the scratch the first one filled
        rc, out, val = _call(logits, off)
        assert rc == 0, _native.cuda().gb_last_error().decode()
        ref_idx, ref_val = sampling.argmax(logits, idx_offset=off, want_value=True)
        torch.cuda.synchronize()
        assert torch.equal(out, ref_idx)
        assert torch.equal(val, ref_val)
    assert int(_call(a)[1][3]) == 10


def test_no_alloc_argmax_row_of_minus_infinity():
    """A row that is -inf everywhere (a fully masked vocabulary) yields column 0 + offset, like the regular entry point."""
    x = torch.full((3, 70000), float("-inf"), device="cuda")
    x[1, 4242] = -5.0
    rc, out, _ = _call(x, 7)
    assert rc == 0
    ref = sampling.argmax(x, idx_offset=7)
    torch.cuda.synchronize()
    assert out.tolist() == [7, 4249, 7] and torch.equal(out, ref)


def test_no_alloc_argmax_rejects_oversized_batches():
    x = torch.zeros(1025, 8, device="cuda")
    rc, _, _ = _call(x)
    assert rc != 0
    assert "1024" in _native.cuda().gb_last_error().decode()
