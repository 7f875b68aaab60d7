"""Builds the reference project's own CPU decoders / engine with gcc (when its source tree is present) so that
tests can compare against them bit for bit.  Nothing of the reference is copied: it is compiled from its place
and loaded through ctypes; tests that need it are skipped when the tree or gcc is missing."""
import ctypes
import os
import shutil
import subprocess
import tempfile

# the reference checkout: GEMM_REFERENCE_ROOT, or a directory "reference" beside this repository
REF_ROOT = os.environ.get("GEMM_REFERENCE_ROOT",
                          os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"))
_cache = {}


def available() -> bool:
    return os.path.isdir(os.path.join(REF_ROOT, "common")) and shutil.which("gcc") is not None


def _build(name: str, source: str, extra=()):
    if name in _cache:
        return _cache[name]
    d = tempfile.mkdtemp(prefix="gemm_ref_oracle_")
    src = os.path.join(d, name + ".c")
    with open(src, "w") as f:
        f.write(source)
    so = os.path.join(d, name + ".so")
    cmd = ["gcc", "-O2", "-shared", "-fPIC", "-w", "-mavx2", "-mfma", "-mf16c", "-I", os.path.join(REF_ROOT, "common"), src, "-o", so, "-lm", "-lpthread", *extra]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference oracle build failed:\n" + r.stderr[-3000:])
    _cache[name] = ctypes.CDLL(so)
    return _cache[name]


def dequant_lib():
    """ctypes handle exposing the reference's ``dequant_row(type, src, dst, n)``."""
    lib = _build("ref_dequant", '#define GGML_DEQUANT_IMPLEMENTATION\n#include "gguf_loader.h"\n#include "ggml_dequant.h"\n')
    lib.dequant_row.argtypes = [ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
    lib.dequant_row.restype = ctypes.c_int
    return lib


def tokenizer_lib():
    """ctypes handle exposing the reference's gguf_open / bpe_vocab_load / bpe_tokenize."""
    lib = _build("ref_tok", '#define GGUF_LOADER_IMPLEMENTATION\n#include "gguf_loader.h"\n#define BPE_TOKENIZER_IMPLEMENTATION\n#include "bpe_tokenizer.h"\n')
    lib.gguf_open.restype = ctypes.c_void_p
    lib.gguf_open.argtypes = [ctypes.c_char_p, ctypes.c_int]
    lib.bpe_vocab_load.restype = ctypes.c_void_p
    lib.bpe_vocab_load.argtypes = [ctypes.c_void_p]
    lib.bpe_tokenize.restype = ctypes.c_int
    lib.bpe_tokenize.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int]
    return lib


def engine_lib():
    """ctypes handle exposing the reference CPU engine (gguf_open, transformer_load, transformer_forward_logits, ...)."""
    src = ('#define GGUF_LOADER_IMPLEMENTATION\n#include "gguf_loader.h"\n#define GGML_DEQUANT_IMPLEMENTATION\n#include "ggml_dequant.h"\n'
           '#define TRANSFORMER_IMPLEMENTATION\n#include "transformer.h"\n'
           'int ref_n_vocab(transformer_model *m) { return m->n_vocab; }\n')
    lib = _build("ref_engine", src)
    lib.gguf_open.restype = ctypes.c_void_p
    lib.gguf_open.argtypes = [ctypes.c_char_p, ctypes.c_int]
    lib.transformer_load.restype = ctypes.c_void_p
    lib.transformer_load.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.transformer_forward_logits.restype = ctypes.POINTER(ctypes.c_float)
    lib.transformer_forward_logits.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int]
    lib.transformer_set_f64_accum.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.ref_n_vocab.argtypes = [ctypes.c_void_p]
    return lib


def vision_lib():
    """ctypes handle exposing the reference's Qwen3-VL vision encoder (gguf_open, vision_load, vision_encode)."""
    src = ('#define GGUF_LOADER_IMPLEMENTATION\n#include "gguf_loader.h"\n#define GGML_DEQUANT_IMPLEMENTATION\n#include "ggml_dequant.h"\n'
           '#include "transformer.h"\n#define VISION_ENCODER_IMPLEMENTATION\n#include "vision_encoder.h"\n')      # transformer.h declares qtensor
    lib = _build("ref_vision", src)
    lib.gguf_open.restype = ctypes.c_void_p
    lib.gguf_open.argtypes = [ctypes.c_char_p, ctypes.c_int]
    lib.vision_load.restype = ctypes.c_void_p
    lib.vision_load.argtypes = [ctypes.c_void_p]
    lib.vision_encode.restype = ctypes.POINTER(ctypes.c_float)
    lib.vision_encode.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    return lib
