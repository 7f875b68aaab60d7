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
           'int ref_n_vocab(transformer_model *m) { return m->n_vocab; }\n'
           'int ref_n_deepstack(transformer_model *m) { return m->n_deepstack; }\n'
           'void ref_set_ds_stride(transformer_model *m, int s) { m->ds_embd_stride = s; }\n')
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
    lib.ref_n_deepstack.argtypes = [ctypes.c_void_p]
    lib.ref_set_ds_stride.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.transformer_forward_embd_logits_pos.restype = ctypes.POINTER(ctypes.c_float)
    lib.transformer_forward_embd_logits_pos.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int]
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


# A scalar stand-in for the Arm SVE intrinsics the DS4F header uses unconditionally, at a 512-bit vector length.  Every vector type
# is one 64-byte union (so the reinterpret casts are the identity) and a predicate holds one flag per byte lane.  It exists so that
# the header COMPILES here; the oracle below only calls the header's scalar validation paths.
_SVE_STUB = r"""/* Scalar stand-in for the Arm SVE intrinsics at a 512-bit vector length: every vector type is the same 64-byte union, so the
 * reinterpret casts are the identity; predicates hold one flag per byte lane. */
#ifndef STUB_ARM_SVE_H
#define STUB_ARM_SVE_H
#include <stdint.h>
#include <string.h>
#include <math.h>
typedef _Float16 __fp16;
typedef union { float f[16]; uint32_t u[16]; int32_t s[16]; uint16_t h[32]; int8_t b[64]; uint8_t ub[64]; } svreg_t;
typedef svreg_t svfloat32_t, svuint32_t, svint32_t, svuint16_t, svint16_t, svint8_t, svuint8_t;
typedef struct { uint8_t m[64]; } svbool_t;
static inline uint64_t svcntw(void) { return 16; }
static inline uint64_t svcnth(void) { return 32; }
static inline uint64_t svcntb(void) { return 64; }
static inline svbool_t svptrue_b8(void)  { svbool_t p; memset(p.m, 1, 64); return p; }
static inline svbool_t svptrue_b16(void) { svbool_t p; memset(p.m, 0, 64); for (int i = 0; i < 32; i++) p.m[2 * i] = 1; return p; }
static inline svbool_t svptrue_b32(void) { svbool_t p; memset(p.m, 0, 64); for (int i = 0; i < 16; i++) p.m[4 * i] = 1; return p; }
static inline svbool_t sv_whilelt_b32(long long a, long long b) { svbool_t p; memset(p.m, 0, 64); for (int i = 0; i < 16; i++) p.m[4 * i] = (a + i < b); return p; }
#define svwhilelt_b32(a, b) sv_whilelt_b32((long long)(a), (long long)(b))
#define SV_ON32(pg, i) ((pg).m[4 * (i)])
static inline svreg_t svdup_f32(float x) { svreg_t r; for (int i = 0; i < 16; i++) r.f[i] = x; return r; }
static inline svreg_t svdup_s32(int32_t x) { svreg_t r; for (int i = 0; i < 16; i++) r.s[i] = x; return r; }
static inline svreg_t svdup_u32(uint32_t x) { svreg_t r; for (int i = 0; i < 16; i++) r.u[i] = x; return r; }
static inline svreg_t svld1_f32(svbool_t pg, const float *p) { svreg_t r; for (int i = 0; i < 16; i++) r.f[i] = SV_ON32(pg, i) ? p[i] : 0.0f; return r; }
#define svld1(pg, p) svld1_f32((pg), (p))
static inline svreg_t svld1_s8(svbool_t pg, const int8_t *p) { svreg_t r; for (int i = 0; i < 64; i++) r.b[i] = pg.m[i] ? p[i] : 0; return r; }
static inline svreg_t svld1uh_u32(svbool_t pg, const uint16_t *p) { svreg_t r; for (int i = 0; i < 16; i++) r.u[i] = SV_ON32(pg, i) ? p[i] : 0; return r; }
static inline svreg_t svld1ub_u32(svbool_t pg, const uint8_t *p) { svreg_t r; for (int i = 0; i < 16; i++) r.u[i] = SV_ON32(pg, i) ? p[i] : 0; return r; }
static inline svreg_t svld1sb_s32(svbool_t pg, const int8_t *p) { svreg_t r; for (int i = 0; i < 16; i++) r.s[i] = SV_ON32(pg, i) ? p[i] : 0; return r; }
static inline svreg_t svld1_gather_u32index_u32(svbool_t pg, const uint32_t *base, svreg_t idx) { svreg_t r; for (int i = 0; i < 16; i++) r.u[i] = SV_ON32(pg, i) ? base[idx.u[i]] : 0; return r; }
static inline void svst1_f32(svbool_t pg, float *p, svreg_t v) { for (int i = 0; i < 16; i++) if (SV_ON32(pg, i)) p[i] = v.f[i]; }
#define svst1(pg, p, v) svst1_f32((pg), (p), (v))
static inline void svst1_u16(svbool_t pg, uint16_t *p, svreg_t v) { for (int i = 0; i < 32; i++) if (pg.m[2 * i]) p[i] = v.h[i]; }
static inline void svst1b_s32(svbool_t pg, int8_t *p, svreg_t v) { for (int i = 0; i < 16; i++) if (SV_ON32(pg, i)) p[i] = (int8_t)v.s[i]; }
static inline svreg_t svmla_f32_x(svbool_t pg, svreg_t a, svreg_t x, svreg_t y) { for (int i = 0; i < 16; i++) if (SV_ON32(pg, i)) a.f[i] += x.f[i] * y.f[i]; return a; }
#define svmla_x svmla_f32_x
static inline svreg_t svmul_f32_x(svbool_t pg, svreg_t x, svreg_t y) { for (int i = 0; i < 16; i++) x.f[i] *= y.f[i]; (void)pg; return x; }
#define svmul_x svmul_f32_x
static inline svreg_t svadd_f32_x(svbool_t pg, svreg_t x, svreg_t y) { for (int i = 0; i < 16; i++) x.f[i] += y.f[i]; (void)pg; return x; }
static inline svreg_t svmax_f32_x(svbool_t pg, svreg_t x, svreg_t y) { for (int i = 0; i < 16; i++) x.f[i] = x.f[i] > y.f[i] ? x.f[i] : y.f[i]; (void)pg; return x; }
#define svmax_x svmax_f32_x
static inline svreg_t svabs_f32_x(svbool_t pg, svreg_t x) { for (int i = 0; i < 16; i++) x.f[i] = fabsf(x.f[i]); (void)pg; return x; }
#define svabs_x svabs_f32_x
static inline svreg_t svmax_s32_x(svbool_t pg, svreg_t x, svreg_t y) { for (int i = 0; i < 16; i++) x.s[i] = x.s[i] > y.s[i] ? x.s[i] : y.s[i]; (void)pg; return x; }
static inline svreg_t svmin_s32_x(svbool_t pg, svreg_t x, svreg_t y) { for (int i = 0; i < 16; i++) x.s[i] = x.s[i] < y.s[i] ? x.s[i] : y.s[i]; (void)pg; return x; }
static inline float svaddv_f32(svbool_t pg, svreg_t v) { float s = 0.0f; for (int i = 0; i < 16; i++) if (SV_ON32(pg, i)) s += v.f[i]; return s; }
static inline float svmaxv_f32(svbool_t pg, svreg_t v) { float s = -INFINITY; for (int i = 0; i < 16; i++) if (SV_ON32(pg, i) && v.f[i] > s) s = v.f[i]; return s; }
static inline int64_t svaddv_s32(svbool_t pg, svreg_t v) { int64_t s = 0; for (int i = 0; i < 16; i++) if (SV_ON32(pg, i)) s += v.s[i]; return s; }
static inline svreg_t svdot_s32(svreg_t acc, svreg_t a, svreg_t b) { for (int i = 0; i < 16; i++) for (int j = 0; j < 4; j++) acc.s[i] += (int32_t)a.b[4 * i + j] * (int32_t)b.b[4 * i + j]; return acc; }
#define svdot svdot_s32
#define svreinterpret_f32_u32(v) (v)
#define svreinterpret_u32_f32(v) (v)
#define svreinterpret_u16_u32(v) (v)
#define svreinterpret_s32_u32(v) (v)
#define svreinterpret_u32_s32(v) (v)
static inline svreg_t svlsr_n_u32_x(svbool_t pg, svreg_t v, unsigned n) { for (int i = 0; i < 16; i++) v.u[i] >>= n; (void)pg; return v; }
static inline svreg_t svlsl_n_u32_x(svbool_t pg, svreg_t v, unsigned n) { for (int i = 0; i < 16; i++) v.u[i] <<= n; (void)pg; return v; }
static inline svreg_t svand_n_u32_x(svbool_t pg, svreg_t v, uint32_t n) { for (int i = 0; i < 16; i++) v.u[i] &= n; (void)pg; return v; }
static inline svreg_t sveor_n_u32_x(svbool_t pg, svreg_t v, uint32_t n) { for (int i = 0; i < 16; i++) v.u[i] ^= n; (void)pg; return v; }
static inline svreg_t svorr_u32_x(svbool_t pg, svreg_t v, svreg_t w) { for (int i = 0; i < 16; i++) v.u[i] |= w.u[i]; (void)pg; return v; }
static inline svreg_t svsub_n_s32_x(svbool_t pg, svreg_t v, int32_t n) { for (int i = 0; i < 16; i++) v.s[i] -= n; (void)pg; return v; }
static inline svreg_t svtbl_f32(svreg_t v, svreg_t idx) { svreg_t r; for (int i = 0; i < 16; i++) r.u[i] = idx.u[i] < 16 ? v.u[idx.u[i]] : 0; return r; }
#define svtbl svtbl_f32
static inline svreg_t svuzp1_u16(svreg_t a, svreg_t b) { svreg_t r; for (int i = 0; i < 16; i++) { r.h[i] = a.h[2 * i]; r.h[16 + i] = b.h[2 * i]; } return r; }
static inline svreg_t svzip1_u16(svreg_t a, svreg_t b) { svreg_t r; for (int i = 0; i < 16; i++) { r.h[2 * i] = a.h[i]; r.h[2 * i + 1] = b.h[i]; } return r; }
static inline svreg_t svzip1_f32(svreg_t a, svreg_t b) { svreg_t r; for (int i = 0; i < 8; i++) { r.f[2 * i] = a.f[i]; r.f[2 * i + 1] = b.f[i]; } return r; }
static inline svreg_t svzip2_f32(svreg_t a, svreg_t b) { svreg_t r; for (int i = 0; i < 8; i++) { r.f[2 * i] = a.f[8 + i]; r.f[2 * i + 1] = b.f[8 + i]; } return r; }
static inline svreg_t svcvt_f32_s32_x(svbool_t pg, svreg_t v) { for (int i = 0; i < 16; i++) v.f[i] = (float)v.s[i]; (void)pg; return v; }
static inline svreg_t svcvt_s32_f32_x(svbool_t pg, svreg_t v) { for (int i = 0; i < 16; i++) v.s[i] = (int32_t)v.f[i]; (void)pg; return v; }
#endif
"""

_DS4F_SRC = r"""
#define _GNU_SOURCE
__asm__(".macro yield\n.endm");
#define GGML_DEQUANT_IMPLEMENTATION
/* the e2m1 code points; the kernel header that defines this table is not part of the reference's common/ tree */
static const float ds4f_kvalues_mxfp4_f32[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f, -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};
#include "ds4f.h"
void ref_rotate(float *x, int n) { ds4f_rotate_activation(x, n); }
void ref_fp4(float *x, int n, int block) { ds4f_fp4_act_quant_inplace(x, n, block); }
void ref_compress_prefill(const float *x, int seqlen, int dim, int d, int rd, int ratio, const float *wkv, const float *wgate, const float *ape,
                          const uint16_t *norm_w, const float *rcos, const float *rsin, float eps, int rotate, float *out) {
    ds4f_compress_prefill(x, seqlen, dim, d, rd, ratio, wkv, wgate, ape, norm_w, rcos, rsin, eps, rotate, out);
}
void ref_compress_reset(float *kv_state, float *score_state, int ratio, int d) { ds4f_compress_state_reset(kv_state, score_state, ratio, d); }
int ref_compress_step(const float *x, int dim, int d, int rd, int ratio, int start_pos, const float *wkv, const float *wgate, const float *ape,
                      const uint16_t *norm_w, const float *rcos, const float *rsin, float eps, int rotate, float *kv_state, float *score_state, float *out) {
    return ds4f_compress_step(x, dim, d, rd, ratio, start_pos, wkv, wgate, 0, ape, norm_w, rcos, rsin, eps, rotate, kv_state, score_state, out, NULL);
}
void ref_index_score(const float *q, const float *kvc, const float *weights, int H, int hd, int T, float *score) {
    ds4f_index_score(q, kvc, weights, H, hd, T, score, NULL);
}
void ref_index_topk(const float *score, int T, int thr, int k, int offset, int *sel) { ds4f_index_topk(score, T, thr, k, offset, sel); }
int ref_index_step(const float *x, int dim, const float *qr, int qlora, int H, int hd, int rd, int ratio, int start_pos, int offset, int k,
                   const float *wq_b, const float *wproj, const float *cwkv, const float *cwgate, const float *cape, const uint16_t *cnorm,
                   const float *rcos, const float *rsin, float eps, float *kv_state, float *score_state, float *idx_kv, float *q_scr,
                   float *score_scr, int *sel) {
    return ds4f_index_step(x, dim, qr, qlora, H, hd, rd, ratio, start_pos, offset, k, wq_b, wproj, 0, cwkv, cwgate, cape, cnorm, rcos, rsin, eps,
                           kv_state, score_state, idx_kv, NULL, NULL, NULL, q_scr, score_scr, sel, NULL, 0, 0, 0, NULL, NULL, 0, 1, NULL, NULL);
}
void ref_sparse_attn(const float *q, const float *kv, const float *sink, const int *topk_idxs, int m, int h, int d, int topk, float scale, float *o) {
    ds4f_sparse_attn(q, kv, sink, topk_idxs, m, h, d, topk, scale, o);
}
int ref_window_idx_decode(int window, int start_pos, int *row) { return ds4f_window_idx_decode(window, start_pos, row); }
void ref_rope_apply(float *v, const float *cosb, const float *sinb, int pos, int half, int inverse) { ds4f_rope_apply(v, cosb, sinb, pos, half, inverse); }
"""


def ds4f_lib():
    """ctypes handle on the scalar Tier-B2 building blocks of the reference's DeepSeek-V4-Flash engine (common/ds4f_impl.h: the
    compressor for a whole prompt and token by token, indexer scoring / top-k / the indexer step, the gathered attention with
    sinks, Hadamard rotation, FP4 rounding).  The engine as a whole cannot run here: its matrix kernels live outside common/."""
    stub = tempfile.mkdtemp(prefix="gemm_ref_stub_")
    with open(os.path.join(stub, "arm_sve.h"), "w") as f:
        f.write(_SVE_STUB)
    lib = _build("ref_ds4f", _DS4F_SRC, extra=("-I", stub))
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.ref_rotate.argtypes = [P, I]
    lib.ref_fp4.argtypes = [P, I, I]
    lib.ref_compress_prefill.argtypes = [P, I, I, I, I, I, P, P, P, P, P, P, F, I, P]
    lib.ref_compress_reset.argtypes = [P, P, I, I]
    lib.ref_compress_step.argtypes = [P, I, I, I, I, I, P, P, P, P, P, P, F, I, P, P, P]
    lib.ref_compress_step.restype = I
    lib.ref_index_score.argtypes = [P, P, P, I, I, I, P]
    lib.ref_index_topk.argtypes = [P, I, I, I, I, P]
    lib.ref_index_step.argtypes = [P, I, P, I, I, I, I, I, I, I, I, P, P, P, P, P, P, P, P, F, P, P, P, P, P, P]
    lib.ref_index_step.restype = I
    lib.ref_sparse_attn.argtypes = [P, P, P, P, I, I, I, I, F, P]
    lib.ref_window_idx_decode.argtypes = [I, I, P]
    lib.ref_window_idx_decode.restype = I
    lib.ref_rope_apply.argtypes = [P, P, P, I, I, I]
    return lib


def geometry_lib():
    """ctypes handle on the reference's marching-cubes extractor and Gaussian-splat PLY writer (common/marching_cubes.h,
    common/gs_ply_writer.h)."""
    src = ('#define MARCHING_CUBES_IMPLEMENTATION\n#include "marching_cubes.h"\n#define GS_PLY_WRITER_IMPLEMENTATION\n#include "gs_ply_writer.h"\n'
           '#define T2_FDG_MESH_IMPLEMENTATION\n#include "trellis2_fdg_mesh.h"\n'
           'int ref_fdg(const int *coords, const float *feats, int n, float voxel, const float *aabb, float **verts, int **tris, int *nt) {\n'
           '  t2_fdg_mesh m = t2_fdg_to_mesh(coords, feats, n, voxel, aabb); *verts = m.vertices; *tris = m.triangles; *nt = m.n_tris; return m.n_verts; }\n'
           'int ref_mc(const float *grid, int nx, int ny, int nz, float iso, const float *bounds, float **verts, int **tris, int *nv, int *nt) {\n'
           '  mc_mesh m = mc_marching_cubes(grid, nx, ny, nz, iso, bounds); *verts = m.vertices; *tris = m.triangles; *nv = m.n_verts; *nt = m.n_tris; return 0; }\n')
    lib = _build("ref_geometry", src)
    lib.ref_mc.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.POINTER(ctypes.POINTER(ctypes.c_float)),
                           ctypes.POINTER(ctypes.POINTER(ctypes.c_int)), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
    lib.gs_ply_write.argtypes = [ctypes.c_char_p, ctypes.c_int] + [ctypes.c_void_p] * 6
    lib.ref_fdg.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.POINTER(ctypes.POINTER(ctypes.c_float)),
                            ctypes.POINTER(ctypes.POINTER(ctypes.c_int)), ctypes.POINTER(ctypes.c_int)]
    return lib
