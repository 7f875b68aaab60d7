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
    lib.transformer_forward_embd_logits.restype = ctypes.POINTER(ctypes.c_float)
    lib.transformer_forward_embd_logits.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
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


_M3_SRC = r"""
#define _GNU_SOURCE
__asm__(".macro yield\n.endm");      /* the spin pool's Arm hint instruction: nothing on this machine */
#define GGML_DEQUANT_IMPLEMENTATION
#include "ggml_dequant.h"
/* the reference defines this 8-row kernel for SVE only; on this machine it is eight of its own scalar dot products */
static inline void matvec_bf16_8row(float* dst, const uint16_t* w0, const uint16_t* w1, const uint16_t* w2, const uint16_t* w3, const uint16_t* w4,
                                    const uint16_t* w5, const uint16_t* w6, const uint16_t* w7, const float* x, int n) {
  const uint16_t* w[8] = {w0, w1, w2, w3, w4, w5, w6, w7};
  for (int r = 0; r < 8; r++) dst[r] = vec_dot_bf16_f32(w[r], x, n);
}
#define M3_IMPL
#include "m3.h"
m3_model* ref_m3_new(const int* v) {
  m3_config c = m3_default_config();
  c.n_layers=v[0]; c.n_dense_layers=v[1]; c.hidden=v[2]; c.vocab=v[3]; c.n_heads=v[4]; c.n_kv_heads=v[5]; c.head_dim=v[6]; c.rotary_dim=v[7];
  c.msa_index_dim=v[8]; c.msa_n_index_heads=v[9]; c.msa_block_size=v[10]; c.msa_topk_blocks=v[11]; c.msa_init_block=v[12]; c.msa_local_block=v[13];
  c.n_experts=v[14]; c.n_active=v[15]; c.moe_inter=v[16]; c.dense_inter=v[17]; c.max_pos=v[18];
  return m3_alloc_synth(c, 0, 1, 1, 1);
}
/* which: 0 embed 1 head 2 out_norm | per layer: 10 input_norm 11 post_norm 12 wq 13 wk 14 wv 15 wo 16 q_norm 17 k_norm 18 idx_wq 19 idx_wk
   20 idx_q_norm 21 idx_k_norm 22 gate 23 gate_bias 24 sh_w1 25 sh_w3 26 sh_w2 27 ex_w1[e] 28 ex_w3[e] 29 ex_w2[e] 30 ff_gate 31 ff_up 32 ff_down */
void* ref_m3_tensor(m3_model* m, int l, int which, int e) {
  if (which == 0) return m->embed; if (which == 1) return m->head.w; if (which == 2) return m->out_norm;
  m3_layer* L = &m->layers[l];
  switch (which) {
    case 10: return L->input_norm; case 11: return L->post_norm; case 12: return L->wq.w; case 13: return L->wk.w; case 14: return L->wv.w;
    case 15: return L->wo.w; case 16: return L->q_norm; case 17: return L->k_norm; case 18: return L->idx_wq.w; case 19: return L->idx_wk.w;
    case 20: return L->idx_q_norm; case 21: return L->idx_k_norm; case 22: return L->gate.w; case 23: return L->gate_bias;
    case 24: return L->sh_w1.w; case 25: return L->sh_w3.w; case 26: return L->sh_w2.w; case 27: return L->ex_w1[e].w; case 28: return L->ex_w3[e].w;
    case 29: return L->ex_w2[e].w; case 30: return L->ff_gate.w; case 31: return L->ff_up.w; case 32: return L->ff_down.w;
  }
  return 0;
}
int ref_m3_forward(m3_model* m, int token, int pos, float* logits) {
  int H = m->cfg.hidden;
  float* x = (float*)malloc(H * sizeof(float));
  for (int i = 0; i < H; i++) x[i] = m3_bf2f(m->embed[(size_t)token * H + i]);
  int r = m3_forward_token(m, x, pos);
  memcpy(logits, m->s_logits, (size_t)m->cfg.vocab * sizeof(float));
  free(x);
  return r;
}
"""


def m3_lib():
    """ctypes handle on the reference's MiniMax-M3 engine (common/m3.h) with synthetic weights: its scalar paths, compiled on this
    machine with a stand-in for the Arm SVE header it includes unconditionally (the SVE code itself sits behind feature macros)."""
    stub = tempfile.mkdtemp(prefix="gemm_ref_stub_")
    with open(os.path.join(stub, "arm_sve.h"), "w") as f:
        f.write("#ifndef STUB_ARM_SVE_H\n#define STUB_ARM_SVE_H\ntypedef _Float16 __fp16;\n#endif\n")
    lib = _build("ref_m3", _M3_SRC, extra=("-fopenmp", "-I", stub))
    lib.ref_m3_new.restype = ctypes.c_void_p
    lib.ref_m3_new.argtypes = [ctypes.c_void_p]
    lib.ref_m3_tensor.restype = ctypes.c_void_p
    lib.ref_m3_tensor.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    lib.ref_m3_forward.restype = ctypes.c_int
    lib.ref_m3_forward.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return lib


_GLM5_SRC = r"""
#define _GNU_SOURCE
__asm__(".macro yield\n.endm");
#define GGML_DEQUANT_IMPLEMENTATION
#include "ggml_dequant.h"
static inline void matvec_bf16_8row(float* dst, const uint16_t* w0, const uint16_t* w1, const uint16_t* w2, const uint16_t* w3, const uint16_t* w4,
                                    const uint16_t* w5, const uint16_t* w6, const uint16_t* w7, const float* x, int n) {
  const uint16_t* w[8] = {w0, w1, w2, w3, w4, w5, w6, w7};
  for (int r = 0; r < 8; r++) dst[r] = vec_dot_bf16_f32(w[r], x, n);
}
#define GLM5_IMPL
#include "glm5.h"
glm5_model* ref_glm5_new(const int* v) {
  glm5_config c = glm5_default_config();
  c.n_layers=v[0]; c.n_dense_layers=v[1]; c.hidden=v[2]; c.vocab=v[3]; c.n_heads=v[4]; c.n_kv_heads=v[4]; c.qk_nope_dim=v[5]; c.qk_rope_dim=v[6];
  c.qk_head_dim=v[5]+v[6]; c.head_dim=c.qk_head_dim; c.v_head_dim=v[7]; c.q_lora=v[8]; c.kv_lora=v[9]; c.index_dim=v[10]; c.index_n_heads=v[11];
  c.index_topk_freq=v[12]; c.rotary_dim=v[6]; c.msa_index_dim=v[10]; c.msa_n_index_heads=v[11]; c.msa_block_size=v[13]; c.msa_topk_blocks=v[14];
  c.msa_init_block=v[15]; c.msa_local_block=v[16]; c.n_experts=v[17]; c.n_active=v[18]; c.moe_inter=v[19]; c.dense_inter=v[20]; c.max_pos=v[21];
  return glm5_alloc_synth(c, 0, 1, 1, 1);
}
/* which: 0 embed 1 head 2 out_norm | per layer: 10 input_norm 11 post_norm 12 wq_a 13 wq_b 14 wkv_a 15 wkv_b 16 wo 17 q_a_norm 18 kv_a_norm
   19 idx_wq 20 idx_wk 21 idx_q_norm 22 idx_k_norm 23 gate 24 gate_bias 25 sh_w1 26 sh_w3 27 sh_w2 28 ex_w1[e] 29 ex_w3[e] 30 ex_w2[e]
   31 ff_gate 32 ff_up 33 ff_down */
void* ref_glm5_tensor(glm5_model* m, int l, int which, int e) {
  if (which == 0) return m->embed; if (which == 1) return m->head.w; if (which == 2) return m->out_norm;
  glm5_layer* L = &m->layers[l];
  switch (which) {
    case 10: return L->input_norm; case 11: return L->post_norm; case 12: return L->wq_a.w; case 13: return L->wq_b.w; case 14: return L->wkv_a.w;
    case 15: return L->wkv_b.w; case 16: return L->wo.w; case 17: return L->q_a_norm; case 18: return L->kv_a_norm; case 19: return L->idx_wq.w;
    case 20: return L->idx_wk.w; case 21: return L->idx_q_norm; case 22: return L->idx_k_norm; case 23: return L->gate.w; case 24: return L->gate_bias;
    case 25: return L->sh_w1.w; case 26: return L->sh_w3.w; case 27: return L->sh_w2.w; case 28: return L->ex_w1[e].w; case 29: return L->ex_w3[e].w;
    case 30: return L->ex_w2[e].w; case 31: return L->ff_gate.w; case 32: return L->ff_up.w; case 33: return L->ff_down.w;
  }
  return 0;
}
int ref_glm5_forward(glm5_model* m, int token, int pos, float* logits) {
  int H = m->cfg.hidden;
  float* x = (float*)malloc(H * sizeof(float));
  for (int i = 0; i < H; i++) x[i] = glm5_bf2f(m->embed[(size_t)token * H + i]);
  int r = glm5_forward_token(m, x, pos);
  memcpy(logits, m->s_logits, (size_t)m->cfg.vocab * sizeof(float));
  free(x);
  return r;
}
"""


def glm5_lib():
    """ctypes handle on the reference's GLM-5 engine (common/glm5.h) with synthetic weights, built like ``m3_lib``."""
    stub = tempfile.mkdtemp(prefix="gemm_ref_stub_")
    with open(os.path.join(stub, "arm_sve.h"), "w") as f:
        f.write("#ifndef STUB_ARM_SVE_H\n#define STUB_ARM_SVE_H\ntypedef _Float16 __fp16;\n#endif\n")
    lib = _build("ref_glm5", _GLM5_SRC, extra=("-fopenmp", "-I", stub))
    lib.ref_glm5_new.restype = ctypes.c_void_p
    lib.ref_glm5_new.argtypes = [ctypes.c_void_p]
    lib.ref_glm5_tensor.restype = ctypes.c_void_p
    lib.ref_glm5_tensor.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    lib.ref_glm5_forward.restype = ctypes.c_int
    lib.ref_glm5_forward.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return lib


def gemma4_vision_lib():
    """ctypes handle exposing the reference's Gemma4 vision tower (gguf_open, g4v_load, g4v_encode)."""
    src = ('#define GGUF_LOADER_IMPLEMENTATION\n#include "gguf_loader.h"\n#define GGML_DEQUANT_IMPLEMENTATION\n#include "ggml_dequant.h"\n'
           '#include "transformer.h"\n#define GEMMA4_VISION_IMPLEMENTATION\n#include "gemma4_vision_encoder.h"\n')
    lib = _build("ref_g4v", src)
    lib.gguf_open.restype = ctypes.c_void_p
    lib.gguf_open.argtypes = [ctypes.c_char_p, ctypes.c_int]
    lib.g4v_load.restype = ctypes.c_void_p
    lib.g4v_load.argtypes = [ctypes.c_void_p]
    lib.g4v_encode.restype = ctypes.POINTER(ctypes.c_float)
    lib.g4v_encode.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    return lib


def audio_mel_lib():
    """ctypes handle exposing the reference's Gemma4 audio front end (g4a_mel_init, g4a_mel_extract, g4a_wav_load)."""
    lib = _build("ref_g4a_mel", '#define GEMMA4_AUDIO_MEL_IMPLEMENTATION\n#include "gemma4_audio_mel.h"\n')
    lib.g4a_mel_init.restype = ctypes.c_void_p
    lib.g4a_mel_extract.restype = ctypes.POINTER(ctypes.c_float)
    lib.g4a_mel_extract.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
    lib.g4a_wav_load.restype = ctypes.POINTER(ctypes.c_float)
    lib.g4a_wav_load.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_int)]
    return lib


def audio_encoder_lib():
    """ctypes handle exposing the reference's Gemma4 audio Conformer (g4a_load_safetensors, g4a_encode, g4a_free)."""
    lib = _build("ref_g4a_enc", '#define SAFETENSORS_IMPLEMENTATION\n#include "safetensors.h"\n#define GEMMA4_AUDIO_IMPLEMENTATION\n'
                 '#include "gemma4_audio_encoder.h"\nvoid ref_free(void *p) { free(p); }\n')
    lib.g4a_load_safetensors.restype = ctypes.c_void_p
    lib.g4a_load_safetensors.argtypes = [ctypes.c_char_p]
    lib.g4a_encode.restype = ctypes.POINTER(ctypes.c_float)
    lib.g4a_encode.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
    lib.g4a_free.argtypes = [ctypes.c_void_p]
    lib.ref_free.argtypes = [ctypes.c_void_p]
    return lib
