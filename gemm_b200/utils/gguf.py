"""GGUF files: reader, writer, ggml (de)quantisation — Python face of csrc/host/gguf.cc and dequant.cc.

Same public surface as the reference's loader (common/gguf_loader.h:146-162: open / close / find_key /
tensor name, data, size) plus what it lacks: a writer and quantisers, which the synthetic checkpoints need.
"""
from __future__ import annotations

import ctypes
from typing import Any, Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native

GGML_TYPES: Dict[str, int] = {
    "F32": 0, "F16": 1, "Q4_0": 2, "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q8_0": 8, "Q8_1": 9, "Q2_K": 10, "Q3_K": 11, "Q4_K": 12,
    "Q5_K": 13, "Q6_K": 14, "Q8_K": 15, "IQ2_XXS": 16, "IQ2_XS": 17, "IQ3_XXS": 18, "IQ1_S": 19, "IQ4_NL": 20, "IQ3_S": 21,
    "IQ2_S": 22, "IQ4_XS": 23, "I8": 24, "I16": 25, "I32": 26, "I64": 27, "F64": 28, "IQ1_M": 29, "BF16": 30, "TQ1_0": 34,
    "TQ2_0": 35, "MXFP4": 39, "NVFP4": 40, "Q1_0": 41,
}
GGML_NAMES = {v: k for k, v in GGML_TYPES.items()}
# the 24 quantisation formats of ggml named by the benchmark description
QUANT_TYPES_24 = ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K", "IQ1_S", "IQ1_M", "IQ2_XXS", "IQ2_XS",
                  "IQ2_S", "IQ3_XXS", "IQ3_S", "IQ4_NL", "IQ4_XS", "TQ1_0", "TQ2_0", "F32", "F16", "BF16"]

KV_U8, KV_I8, KV_U16, KV_I16, KV_U32, KV_I32, KV_F32, KV_BOOL, KV_STR, KV_ARR, KV_U64, KV_I64, KV_F64 = range(13)
_NP_OF_KV = {KV_U8: np.uint8, KV_I8: np.int8, KV_U16: np.uint16, KV_I16: np.int16, KV_U32: np.uint32, KV_I32: np.int32,
             KV_F32: np.float32, KV_BOOL: np.bool_, KV_U64: np.uint64, KV_I64: np.int64, KV_F64: np.float64}


def _lib():
    lib = _native.host()
    if not getattr(lib, "_gguf_ready", False):
        lib.gbh_gguf_open.restype = ctypes.c_void_p
        lib.gbh_gguf_open.argtypes = [ctypes.c_char_p]
        lib.gbh_gguf_tensor_data.restype = ctypes.c_void_p
        lib.gbh_gguf_kv_string.restype = ctypes.c_void_p
        lib.gbh_gguf_kv_array_data.restype = ctypes.c_void_p
        lib.gbh_gguf_writer_new.restype = ctypes.c_void_p
        lib.gbh_row_bytes.restype = ctypes.c_long
        lib.gbh_gguf_n_tensors.restype = ctypes.c_long
        lib.gbh_gguf_n_kv.restype = ctypes.c_long
        lib.gbh_codebook.restype = ctypes.c_void_p
        lib._gguf_ready = True
    return lib


def _err() -> str:
    return _lib().gbh_last_error().decode(errors="replace")


def type_id(t) -> int:
    return GGML_TYPES[t.upper()] if isinstance(t, str) else int(t)


def block_info(t) -> Tuple[int, int]:
    """(elements per block, bytes per block) of a ggml type."""
    blk, nbytes = ctypes.c_int(), ctypes.c_int()
    if _lib().gbh_type_info(type_id(t), ctypes.byref(blk), ctypes.byref(nbytes), None) != 0:
        raise ValueError(_err())
    return blk.value, nbytes.value


def row_bytes(t, n: int) -> int:
    r = _lib().gbh_row_bytes(type_id(t), ctypes.c_long(n))
    if r < 0:
        raise ValueError(f"{n} elements do not fit whole blocks of {t}")
    return r


def dequantize(data, t, n: int) -> torch.Tensor:
    """Decode ``n`` elements of ggml type ``t`` from raw bytes (bytes / numpy / uint8 tensor) to float32."""
    buf = np.frombuffer(data, dtype=np.uint8) if isinstance(data, (bytes, bytearray, memoryview)) else \
        (data.contiguous().numpy() if torch.is_tensor(data) else np.ascontiguousarray(data)).view(np.uint8).reshape(-1)
    need = row_bytes(t, n)
    if buf.size < need:
        raise ValueError(f"need {need} bytes for {n} x {t}, got {buf.size}")
    out = np.empty(n, dtype=np.float32)
    rc = _lib().gbh_dequant_row(type_id(t), ctypes.c_void_p(buf.ctypes.data), ctypes.c_void_p(out.ctypes.data), ctypes.c_long(n))
    if rc != 0:
        raise ValueError(_err())
    return torch.from_numpy(out)


def quantize(x: torch.Tensor, t) -> torch.Tensor:
    """Encode a float tensor (last dim = rows of whole blocks) to raw ggml bytes (uint8 tensor)."""
    xf = x.detach().to(torch.float32).contiguous().cpu().numpy().reshape(-1)
    n = xf.size
    out = np.empty(row_bytes(t, n), dtype=np.uint8)
    rc = _lib().gbh_quantize_row(type_id(t), ctypes.c_void_p(xf.ctypes.data), ctypes.c_void_p(out.ctypes.data), ctypes.c_long(n))
    if rc != 0:
        raise ValueError(_err())
    return torch.from_numpy(out)


def can_quantize(t) -> bool:
    return bool(_lib().gbh_can_quantize(type_id(t)))


def codebook(which: int) -> np.ndarray:
    """IQ codebook ``which`` (0 iq2xxs, 1 iq2xs, 2 iq2s, 3 iq3xxs, 4 iq3s, 5 iq1s (int8), 6 sign table) as a numpy array."""
    n, w = ctypes.c_int(), ctypes.c_int()
    p = _lib().gbh_codebook(which, ctypes.byref(n), ctypes.byref(w))
    arr = np.ctypeslib.as_array((ctypes.c_uint8 * (n.value * w.value)).from_address(p)).reshape(n.value, w.value).copy()
    return arr.view(np.int8) if which == 5 else arr


class GGUFTensor:
    __slots__ = ("name", "shape", "ggml_type", "nbytes", "_ptr", "_owner")

    def __init__(self, name, shape, ggml_type, nbytes, ptr, owner):
        self.name, self.shape, self.ggml_type, self.nbytes, self._ptr, self._owner = name, shape, ggml_type, nbytes, ptr, owner

    @property
    def type_name(self) -> str:
        return GGML_NAMES.get(self.ggml_type, str(self.ggml_type))

    def raw(self) -> np.ndarray:
        """Zero-copy uint8 view of the tensor's bytes inside the mapping."""
        return np.ctypeslib.as_array((ctypes.c_uint8 * self.nbytes).from_address(self._ptr))

    def to_float(self) -> torch.Tensor:
        """float32 tensor with the logical (row-major, outermost-first) shape."""
        n = int(np.prod(self.shape))
        return dequantize(self.raw(), self.ggml_type, n).reshape(self.shape)


class GGUFFile:
    """Read-only view of a GGUF file (memory mapped).  ``metadata`` maps keys to Python values;
    ``tensors`` maps names to ``GGUFTensor``.  Shapes are reported outermost-first (PyTorch order)."""

    def __init__(self, path: str):
        lib = _lib()
        self._h = lib.gbh_gguf_open(path.encode())
        if not self._h:
            raise IOError(_err())
        self.path = path
        h = ctypes.c_void_p(self._h)
        self.version = lib.gbh_gguf_version(h)
        self.alignment = lib.gbh_gguf_alignment(h)
        self.metadata: Dict[str, Any] = {}
        key = ctypes.create_string_buffer(512)
        for i in range(lib.gbh_gguf_n_kv(h)):
            t, et, cnt = ctypes.c_int(), ctypes.c_int(), ctypes.c_uint64()
            lib.gbh_gguf_kv_info(h, i, key, 512, ctypes.byref(t), ctypes.byref(et), ctypes.byref(cnt))
            self.metadata[key.value.decode()] = self._value(i, t.value, et.value, cnt.value)
        self.tensors: Dict[str, GGUFTensor] = {}
        name = ctypes.create_string_buffer(512)
        for i in range(lib.gbh_gguf_n_tensors(h)):
            nd, ty, nb = ctypes.c_int(), ctypes.c_int(), ctypes.c_uint64()
            dims = (ctypes.c_uint64 * 4)()
            lib.gbh_gguf_tensor_info(h, i, name, 512, ctypes.byref(nd), dims, ctypes.byref(ty), ctypes.byref(nb))
            shape = tuple(int(dims[d]) for d in reversed(range(nd.value)))
            ptr = lib.gbh_gguf_tensor_data(h, i)
            self.tensors[name.value.decode()] = GGUFTensor(name.value.decode(), shape, ty.value, nb.value, ptr, self)

    def _value(self, i, t, et, cnt):
        lib, h = _lib(), ctypes.c_void_p(self._h)
        if t == KV_STR:
            ln = ctypes.c_uint64()
            p = lib.gbh_gguf_kv_string(h, i, ctypes.c_long(0), ctypes.byref(ln))
            return ctypes.string_at(p, ln.value).decode(errors="replace")
        if t == KV_ARR:
            if et == KV_STR:
                out, ln = [], ctypes.c_uint64()
                for j in range(cnt):
                    p = lib.gbh_gguf_kv_string(h, i, ctypes.c_long(j), ctypes.byref(ln))
                    out.append(ctypes.string_at(p, ln.value))
                return out            # bytes: token strings need not be valid UTF-8
            p = lib.gbh_gguf_kv_array_data(h, i)
            dt = np.dtype(_NP_OF_KV[et])
            return np.frombuffer(ctypes.string_at(p, cnt * dt.itemsize), dtype=dt).copy()
        v = ctypes.c_double()
        lib.gbh_gguf_kv_scalar(h, i, ctypes.byref(v))
        if t == KV_BOOL:
            return bool(v.value)
        return float(v.value) if t in (KV_F32, KV_F64) else int(v.value)

    def close(self):
        if self._h:
            _lib().gbh_gguf_close(ctypes.c_void_p(self._h))
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GGUFWriter:
    """Builds a GGUF v3 file.  Tensor shapes are given outermost-first (PyTorch order)."""

    def __init__(self, alignment: int = 32):
        self._w = _lib().gbh_gguf_writer_new(alignment)
        self._keep: List[Any] = []

    def add_u32(self, key, v): self._scalar(key, KV_U32, v)
    def add_i32(self, key, v): self._scalar(key, KV_I32, v)
    def add_u64(self, key, v): self._scalar(key, KV_U64, v)
    def add_f32(self, key, v): self._scalar(key, KV_F32, v)
    def add_bool(self, key, v): self._scalar(key, KV_BOOL, 1 if v else 0)

    def _scalar(self, key, t, v):
        if _lib().gbh_gguf_writer_kv_scalar(ctypes.c_void_p(self._w), key.encode(), t, ctypes.c_double(v)) != 0:
            raise ValueError(_err())

    def add_string(self, key: str, s):
        b = s.encode() if isinstance(s, str) else bytes(s)
        _lib().gbh_gguf_writer_kv_string(ctypes.c_void_p(self._w), key.encode(), b, ctypes.c_uint64(len(b)))

    def add_string_array(self, key: str, items: Sequence):
        bs = [x.encode() if isinstance(x, str) else bytes(x) for x in items]
        lens = (ctypes.c_uint64 * len(bs))(*[len(b) for b in bs])
        _lib().gbh_gguf_writer_kv_string_array(ctypes.c_void_p(self._w), key.encode(), b"".join(bs), lens, ctypes.c_uint64(len(bs)))

    def add_array(self, key: str, values, kv_type: int = KV_I32):
        arr = np.ascontiguousarray(np.asarray(values, dtype=_NP_OF_KV[kv_type]))
        _lib().gbh_gguf_writer_kv_array(ctypes.c_void_p(self._w), key.encode(), kv_type, ctypes.c_void_p(arr.ctypes.data), ctypes.c_uint64(arr.size))

    def add_tensor(self, name: str, x: torch.Tensor, t="F32"):
        """Quantise ``x`` (float tensor, logical shape) to ggml type ``t`` and add it."""
        raw = quantize(x, t)
        self.add_raw_tensor(name, raw, tuple(x.shape), t)

    def add_raw_tensor(self, name: str, raw: torch.Tensor, shape: Sequence[int], t):
        raw = raw.contiguous()
        dims = (ctypes.c_uint64 * 4)(*(list(reversed([int(s) for s in shape])) + [1] * (4 - len(shape))))
        rc = _lib().gbh_gguf_writer_tensor(ctypes.c_void_p(self._w), name.encode(), len(shape), dims, type_id(t),
                                           ctypes.c_void_p(raw.data_ptr()), ctypes.c_uint64(raw.numel() * raw.element_size()), 1)
        if rc != 0:
            raise ValueError(_err())

    def write(self, path: str):
        if _lib().gbh_gguf_writer_write(ctypes.c_void_p(self._w), path.encode()) != 0:
            raise IOError(_err())

    def __del__(self):
        try:
            if self._w:
                _lib().gbh_gguf_writer_free(ctypes.c_void_p(self._w))
                self._w = None
        except Exception:
            pass
