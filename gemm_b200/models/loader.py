"""Checkpoint loading and writing: GGUF (any ggml type, dequantised on load) and Hugging Face safetensors.

Names follow the layouts the reference reads: GGUF ``token_embd / output_norm / output / blk.N.{attn_norm, attn_q, attn_k,
attn_v, attn_q_norm, attn_k_norm, attn_output, ffn_norm, ffn_gate, ffn_up, ffn_down}.weight``, MoE ``blk.N.{ffn_gate_inp,
ffn_gate_exps, ffn_up_exps, ffn_down_exps}.weight`` as 3-D tensors (common/transformer.h:1775-2010), and the HF Qwen3 names
``model.layers.N.self_attn.{q,k,v,o}_proj``, ``mlp.{gate,up,down}_proj``, ``mlp.experts.E.*`` (cuda/llm/cuda_llm_runner.c:12293-12447).
Hyper-parameters come from the GGUF key/values (``<arch>.*``) or, for safetensors, from ``config.json``.
"""
from __future__ import annotations

import ctypes
import json
import os
from typing import Dict, List, Optional

import numpy as np
import torch

from .. import _native
from ..utils import gguf as G
from .config import ARCHS, ModelConfig
from .weights import ModelWeights, RandomSource, build_weights


# ------------------------------------------------------------------------------------------ GGUF
def config_from_gguf(f: G.GGUFFile) -> ModelConfig:
    m = f.metadata
    arch = m.get("general.architecture", "qwen3")
    if arch not in ARCHS:
        raise ValueError(f"unsupported architecture {arch!r} (supported: {ARCHS})")

    def key(name, default=None):
        return m.get(f"{arch}.{name}", default)

    hidden = int(key("embedding_length"))
    n_heads = int(key("attention.head_count"))
    head_dim = int(key("attention.key_length", hidden // n_heads))
    vocab = key("vocab_size")
    if vocab is None:
        vocab = f.tensors["token_embd.weight"].shape[0]
    n_exp = int(key("expert_count", 0) or 0)
    n_layers_probe = int(key("block_count"))
    cfg = ModelConfig(
        arch=arch, n_layers=int(key("block_count")), hidden=hidden, n_heads=n_heads,
        n_kv_heads=int(key("attention.head_count_kv", n_heads)), head_dim=head_dim, ffn=int(key("feed_forward_length", 0) or 0),
        vocab=int(vocab), rms_eps=float(key("attention.layer_norm_rms_epsilon", 1e-6)), rope_theta=float(key("rope.freq_base", 1e6)),
        rope_dim=(int(key("rope.dimension_count")) if key("rope.dimension_count") not in (None, head_dim) else None),
        # any layer: in the hybrid models block 0 is a Delta-Net layer and carries neither tensor
        qk_norm=any(f"blk.{i}.attn_q_norm.weight" in f.tensors for i in range(n_layers_probe)),
        qkv_bias=any(f"blk.{i}.attn_q.bias" in f.tensors for i in range(n_layers_probe)),
        tie_embeddings="output.weight" not in f.tensors, max_seq_len=int(key("context_length", 4096)),
        n_experts=n_exp, n_experts_used=int(key("expert_used_count", 0) or 0), expert_ffn=int(key("expert_feed_forward_length", 0) or 0),
        shared_expert_ffn=int(key("expert_shared_feed_forward_length", 0) or 0),
        full_attention_interval=int(key("attention.full_attention_interval", 0) or 0),
        n_deepstack_layers=int(key("n_deepstack_layers", 0) or 0),
    )
    if cfg.full_attention_interval > 0:            # Qwen3.5 hybrid: the ssm.* family (defaults of common/transformer.h:1699-1704)
        cfg.ssm_d_conv = int(key("ssm.conv_kernel", 4))
        cfg.ssm_head_dim = int(key("ssm.state_size", 128))
        cfg.ssm_n_heads_k = int(key("ssm.group_count", 16))
        cfg.ssm_n_heads_v = int(key("ssm.time_step_rank", 48))
        cfg.attn_output_gate = True
    sections = key("rope.dimension_sections")
    if sections is not None and sum(int(x) for x in sections) > 0:
        cfg.mrope_sections = [int(x) for x in sections]
        cfg.rope_dim = 2 * sum(cfg.mrope_sections)
    return cfg


class GGUFSource:
    """Tensor source over an open GGUF file: every tensor is dequantised to float32 on request."""

    def __init__(self, f: G.GGUFFile, keep_blocks: bool = False):
        self.f = f
        self.keep_blocks = keep_blocks       # hand out Q4_K / Q8_0 matrices as their raw blocks (no conversion at load)
        self._cache_name = None
        self._cache = None

    def get_mat(self, name: str, shape):
        """A 2-D projection matrix: its raw ggml blocks (``models.weights.QBlocks``) when ``keep_blocks`` and the type has a fused
        dequant kernel (Q4_K, Q8_0), else float32 as ``get``."""
        from .weights import QBlocks, QUANT_FMTS
        t = self.f.tensors[name]
        if self.keep_blocks and len(shape) == 2 and int(t.ggml_type) in QUANT_FMTS.values() and tuple(t.shape) == tuple(shape):
            blk, nb = G.block_info(t.ggml_type)
            rows, k = shape
            raw = torch.from_numpy(np.array(t.raw(), copy=True)).reshape(rows, k // blk * nb)
            return QBlocks(raw, int(t.ggml_type), k)
        return self.get(name, shape)

    def has(self, name: str) -> bool:
        return name in self.f.tensors

    def get(self, name: str, shape) -> torch.Tensor:
        t = self.f.tensors[name]
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"{name}: file has shape {t.shape}, model wants {tuple(shape)}")
        return t.to_float()

    def get_expert(self, name: str, e: int, shape) -> torch.Tensor:
        t = self.f.tensors[name]
        if tuple(t.shape[1:]) != tuple(shape):
            raise ValueError(f"{name}: file has per-expert shape {t.shape[1:]}, model wants {tuple(shape)}")
        per = int(np.prod(shape))
        blk, nbytes = G.block_info(t.ggml_type)
        off = e * per // blk * nbytes
        raw = t.raw()[off: off + per // blk * nbytes]
        return G.dequantize(raw, t.ggml_type, per).reshape(tuple(shape))


def load_gguf(path: str, fmt: str = "bf16", device="cuda", tp_rank: int = 0, tp_size: int = 1, ep_rank: int = 0, ep_size: int = 1,
              shard_vocab: bool = False) -> ModelWeights:
    """Load a GGUF checkpoint into the run-time weight format ``fmt``, sharded for this rank.

    ``bf16`` / ``mxfp8`` convert every matrix at load.  ``ggml`` converts nothing it has a kernel for: Q4_K and Q8_0 matrices keep
    the file's blocks (re-ordered into tiles, bit for bit) and are multiplied by the fused dequant-GEMV / dequant-GEMM; tensors
    of other types become bf16.  ``q4_k`` / ``q8_0`` additionally re-quantise the remaining matrices to that format."""
    with G.GGUFFile(path) as f:
        cfg = config_from_gguf(f)
        src = GGUFSource(f, keep_blocks=fmt in ("ggml", "q4_k", "q8_0"))
        return build_weights(cfg, src, fmt, device, tp_rank, tp_size, ep_rank, ep_size, shard_vocab)


def save_gguf(cfg: ModelConfig, src, path: str, wtype: str = "F16", tokens=None, merges=None, token_types=None, pre: str = "qwen2") -> None:
    """Write the tensors of ``src`` (any tensor source) as a GGUF file the reference engine can load.

    Matrices are quantised to ``wtype`` (norms and biases stay F32).  The reference refuses files without a tokenizer
    vocabulary (common/bpe_tokenizer.h:356-360), so a byte-level dummy vocabulary is written when none is given."""
    w = G.GGUFWriter()
    a = cfg.arch
    w.add_string("general.architecture", a)
    w.add_string("general.name", f"synthetic-{a}")
    w.add_u32(f"{a}.block_count", cfg.n_layers)
    w.add_u32(f"{a}.embedding_length", cfg.hidden)
    w.add_u32(f"{a}.attention.head_count", cfg.n_heads)
    w.add_u32(f"{a}.attention.head_count_kv", cfg.n_kv_heads)
    w.add_u32(f"{a}.attention.key_length", cfg.head_dim)
    w.add_u32(f"{a}.attention.value_length", cfg.head_dim)
    w.add_u32(f"{a}.feed_forward_length", cfg.ffn)
    w.add_u32(f"{a}.vocab_size", cfg.vocab)
    w.add_u32(f"{a}.context_length", cfg.max_seq_len)
    w.add_f32(f"{a}.attention.layer_norm_rms_epsilon", cfg.rms_eps)
    w.add_f32(f"{a}.rope.freq_base", cfg.rope_theta)
    if cfg.is_moe:
        w.add_u32(f"{a}.expert_count", cfg.n_experts)
        w.add_u32(f"{a}.expert_used_count", cfg.n_experts_used)
        w.add_u32(f"{a}.expert_feed_forward_length", cfg.expert_ffn)
    if cfg.is_moe and cfg.shared_expert_ffn:
        w.add_u32(f"{a}.expert_shared_feed_forward_length", cfg.shared_expert_ffn)
    if cfg.mrope_sections:
        w.add_array(f"{a}.rope.dimension_sections", [int(x) for x in cfg.mrope_sections])
    elif cfg.rope_dim:
        w.add_u32(f"{a}.rope.dimension_count", cfg.rope_dim)
    if cfg.n_deepstack_layers:
        w.add_u32(f"{a}.n_deepstack_layers", cfg.n_deepstack_layers)
    if cfg.is_hybrid:
        w.add_u32(f"{a}.attention.full_attention_interval", cfg.full_attention_interval)
        w.add_u32(f"{a}.ssm.conv_kernel", cfg.ssm_d_conv)
        w.add_u32(f"{a}.ssm.state_size", cfg.ssm_head_dim)
        w.add_u32(f"{a}.ssm.group_count", cfg.ssm_n_heads_k)
        w.add_u32(f"{a}.ssm.time_step_rank", cfg.ssm_n_heads_v)
        w.add_u32(f"{a}.ssm.inner_size", cfg.ssm_d_inner)
    if tokens is None:
        from ..utils.tokenizer import byte_alphabet
        tokens = byte_alphabet() + [f"<extra_{i}>" for i in range(max(0, cfg.vocab - 256))]
        tokens = tokens[: cfg.vocab]
        merges, token_types = [], [1] * len(tokens)
    w.add_string("tokenizer.ggml.model", "gpt2")
    w.add_string("tokenizer.ggml.pre", pre)
    w.add_string_array("tokenizer.ggml.tokens", tokens)
    w.add_string_array("tokenizer.ggml.merges", merges or [])
    if token_types is not None:
        w.add_array("tokenizer.ggml.token_type", token_types)
    w.add_u32("tokenizer.ggml.eos_token_id", max(0, len(tokens) - 1))
    h, d = cfg.hidden, cfg.head_dim

    def mat(name, shape):
        w.add_tensor(name, src.get(name, shape).float(), wtype)

    def vec(name, shape):
        w.add_tensor(name, src.get(name, shape).float(), "F32")

    mat("token_embd.weight", (cfg.vocab, h))
    vec("output_norm.weight", (h,))
    if not cfg.tie_embeddings:
        mat("output.weight", (cfg.vocab, h))
    for li in range(cfg.n_layers):
        p = f"blk.{li}."
        vec(p + "attn_norm.weight", (h,))
        if cfg.is_ssm_layer(li):
            qd, di, hv = cfg.ssm_qkv_dim, cfg.ssm_d_inner, cfg.ssm_n_heads_v
            mat(p + "attn_qkv.weight", (qd, h)); mat(p + "attn_gate.weight", (di, h))
            mat(p + "ssm_alpha.weight", (hv, h)); mat(p + "ssm_beta.weight", (hv, h)); mat(p + "ssm_out.weight", (h, di))
            vec(p + "ssm_conv1d.weight", (qd, cfg.ssm_d_conv)); vec(p + "ssm_norm.weight", (cfg.ssm_head_dim,))
            vec(p + "ssm_a", (hv,)); vec(p + "ssm_dt.bias", (hv,))
            w.add_tensor(p + "post_attention_norm.weight", src.get(p + "ffn_norm.weight", (h,)).float(), "F32")
            _save_ffn(cfg, src, w, p, wtype, mat)
            continue
        mat(p + "attn_q.weight", ((2 if cfg.attn_output_gate else 1) * cfg.q_dim, h))
        mat(p + "attn_k.weight", (cfg.kv_dim, h)); mat(p + "attn_v.weight", (cfg.kv_dim, h))
        mat(p + "attn_output.weight", (h, cfg.q_dim))
        if cfg.qkv_bias:
            vec(p + "attn_q.bias", (cfg.q_dim,)); vec(p + "attn_k.bias", (cfg.kv_dim,)); vec(p + "attn_v.bias", (cfg.kv_dim,))
        if cfg.qk_norm:
            vec(p + "attn_q_norm.weight", (d,)); vec(p + "attn_k_norm.weight", (d,))
        if cfg.is_hybrid:
            w.add_tensor(p + "post_attention_norm.weight", src.get(p + "ffn_norm.weight", (h,)).float(), "F32")
        else:
            vec(p + "ffn_norm.weight", (h,))
        _save_ffn(cfg, src, w, p, wtype, mat)
    w.write(path)


def _save_ffn(cfg, src, w, p, wtype, mat) -> None:
    h = cfg.hidden
    if cfg.is_moe:
        e, inter = cfg.n_experts, cfg.expert_ffn
        w.add_tensor(p + "ffn_gate_inp.weight", src.get(p + "ffn_gate_inp.weight", (e, h)).float(), "F32")
        for nm, shp in (("ffn_gate_exps.weight", (inter, h)), ("ffn_up_exps.weight", (inter, h)), ("ffn_down_exps.weight", (h, inter))):
            full = torch.stack([src.get_expert(p + nm, ei, shp).float() for ei in range(e)])
            w.add_tensor(p + nm, full, wtype)
        if cfg.shared_expert_ffn:
            fs = cfg.shared_expert_ffn
            mat(p + "ffn_gate_shexp.weight", (fs, h)); mat(p + "ffn_up_shexp.weight", (fs, h)); mat(p + "ffn_down_shexp.weight", (h, fs))
            w.add_tensor(p + "ffn_gate_inp_shexp.weight", src.get(p + "ffn_gate_inp_shexp.weight", (h,)).float(), "F32")
    else:
        mat(p + "ffn_gate.weight", (cfg.ffn, h)); mat(p + "ffn_up.weight", (cfg.ffn, h)); mat(p + "ffn_down.weight", (h, cfg.ffn))


# ------------------------------------------------------------------------------------------ safetensors
_ST_DTYPES = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F8_E4M3": torch.float8_e4m3fn, "U8": torch.uint8,
              "I8": torch.int8, "I32": torch.int32, "I64": torch.int64, "F64": torch.float64, "I16": torch.int16}


def _st_lib():
    lib = _native.host()
    if not getattr(lib, "_st_ready", False):
        lib.gbh_st_open.restype = ctypes.c_void_p
        lib.gbh_st_data.restype = ctypes.c_void_p
        lib.gbh_st_count.restype = ctypes.c_long
        lib.gbh_st_metadata.restype = ctypes.c_char_p
        lib._st_ready = True
    return lib


class SafetensorsFile:
    """Memory-mapped safetensors file; ``tensors[name]`` gives a zero-copy torch view (CPU)."""

    def __init__(self, path: str):
        lib = _st_lib()
        self._h = lib.gbh_st_open(path.encode())
        if not self._h:
            raise IOError(lib.gbh_last_error().decode())
        self.info: Dict[str, tuple] = {}
        name = ctypes.create_string_buffer(1024)
        dt = ctypes.create_string_buffer(8)
        for i in range(lib.gbh_st_count(ctypes.c_void_p(self._h))):
            nd, nb = ctypes.c_int(), ctypes.c_uint64()
            shape = (ctypes.c_int64 * 8)()
            lib.gbh_st_info(ctypes.c_void_p(self._h), i, name, 1024, dt, ctypes.byref(nd), shape, ctypes.byref(nb))
            self.info[name.value.decode()] = (i, dt.value.decode(), tuple(int(shape[d]) for d in range(nd.value)), nb.value)

    def keys(self):
        return self.info.keys()

    def get(self, name: str) -> torch.Tensor:
        i, dt, shape, nb = self.info[name]
        p = _st_lib().gbh_st_data(ctypes.c_void_p(self._h), i)
        if nb == 0:
            return torch.empty(shape, dtype=_ST_DTYPES[dt])
        buf = (ctypes.c_uint8 * nb).from_address(p)
        return torch.frombuffer(buf, dtype=torch.uint8).view(_ST_DTYPES[dt]).reshape(shape)

    def metadata(self, key: str) -> Optional[str]:
        v = _st_lib().gbh_st_metadata(ctypes.c_void_p(self._h), key.encode())
        return v.decode() if v else None

    def close(self):
        if self._h:
            _st_lib().gbh_st_close(ctypes.c_void_p(self._h))
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def save_safetensors(tensors: Dict[str, torch.Tensor], path: str) -> None:
    rev = {v: k for k, v in _ST_DTYPES.items()}
    names = list(tensors)
    ts = [tensors[n].contiguous().cpu() for n in names]
    n = len(names)
    c_names = (ctypes.c_char_p * n)(*[x.encode() for x in names])
    c_dt = (ctypes.c_char_p * n)(*[rev[t.dtype].encode() for t in ts])
    ranks = (ctypes.c_int * n)(*[t.dim() for t in ts])
    flat = [int(s) for t in ts for s in t.shape]
    shapes = (ctypes.c_int64 * max(1, len(flat)))(*flat)
    ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in ts])
    nbytes = (ctypes.c_uint64 * n)(*[t.numel() * t.element_size() for t in ts])
    if _st_lib().gbh_st_write(path.encode(), n, c_names, c_dt, ranks, shapes, ptrs, nbytes) != 0:
        raise IOError(_st_lib().gbh_last_error().decode())


_HF_MAP = {"attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj",
           "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm", "attn_norm": "input_layernorm",
           "ffn_norm": "post_attention_layernorm", "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj",
           "ffn_gate_inp": "mlp.gate"}
_HF_EXPERT = {"ffn_gate_exps": "gate_proj", "ffn_up_exps": "up_proj", "ffn_down_exps": "down_proj"}


def hf_name(gguf_name: str, expert: Optional[int] = None) -> str:
    """HF safetensors name of a GGUF tensor name (Qwen2 / Qwen3 / Qwen3-MoE layout)."""
    if gguf_name == "token_embd.weight":
        return "model.embed_tokens.weight"
    if gguf_name == "output_norm.weight":
        return "model.norm.weight"
    if gguf_name == "output.weight":
        return "lm_head.weight"
    _, li, rest = gguf_name.split(".", 2)
    base, kind = rest.rsplit(".", 1)
    if base in _HF_EXPERT:
        return f"model.layers.{li}.mlp.experts.{expert}.{_HF_EXPERT[base]}.{kind}"
    return f"model.layers.{li}.{_HF_MAP[base]}.{kind}"


E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def mxfp4_dequant(packed: torch.Tensor, scale_e8m0: torch.Tensor) -> torch.Tensor:
    """MXFP4: ``packed`` uint8 [rows, cols / 2] (two e2m1 codes per byte, low nibble = even column), one E8M0 scale per 32
    columns ``[rows, cols / 32]`` -> f32 [rows, cols].  The expert format of DeepSeek-V4-Flash (common/ds4f.h:1-34)."""
    rows, half = packed.shape
    lut = torch.tensor(E2M1_VALUES + tuple(-v for v in E2M1_VALUES), dtype=torch.float32, device=packed.device)
    codes = torch.stack([packed & 0xF, packed >> 4], dim=-1).reshape(rows, half * 2).long()
    scale = (scale_e8m0.to(torch.int32) << 23).view(torch.float32)
    return (lut[codes].reshape(rows, half * 2 // 32, 32) * scale.unsqueeze(-1)).reshape(rows, half * 2)


def mxfp4_quant(w: torch.Tensor):
    """Inverse of ``mxfp4_dequant`` (round to nearest e2m1 after scaling each 32-block so that its maximum is <= 6)."""
    rows, cols = w.shape
    blk = w.float().reshape(rows, cols // 32, 32)
    amax = blk.abs().amax(-1)
    e = torch.where(amax > 0, torch.ceil(torch.log2(amax / 6.0)), torch.zeros_like(amax)).clamp(-126, 127)
    scaled = blk / torch.exp2(e).unsqueeze(-1)
    grid = torch.tensor(E2M1_VALUES, dtype=torch.float32)
    mag = (scaled.abs().unsqueeze(-1) - grid).abs().argmin(-1)
    codes = (mag | ((scaled < 0).long() << 3)).reshape(rows, cols).to(torch.uint8)
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous(), (e + 127).to(torch.uint8)


class SafetensorsSource:
    """Tensor source over a directory of HF safetensors shards (or one file).  Quantised checkpoints are dequantised exactly:

    * MXFP8: ``F8_E4M3`` weight + ``<name>_scale_inv`` E8M0 (uint8) [rows, cols / 32]            -> e4m3 * 2^(s - 127)
    * FP8 with 128 x 128 block scales: ``F8_E4M3`` weight + ``<name>_scale_inv`` F32 / BF16 [rows / 128, cols / 128]
      (the dense format of GLM-5 and DeepSeek-V4-Flash: common/glm5_impl.h:399-471, common/ds4f.h:1-34)
    * MXFP4: ``U8`` weight [rows, cols / 2] + ``<name>_scale`` E8M0 [rows, cols / 32] (DeepSeek-V4-Flash experts)
    """

    def __init__(self, path: str):
        files = [path] if os.path.isfile(path) else sorted(os.path.join(path, x) for x in os.listdir(path) if x.endswith(".safetensors"))
        if not files:
            raise IOError(f"no .safetensors files under {path}")
        self.files = [SafetensorsFile(p) for p in files]
        self.where = {k: f for f in self.files for k in f.keys()}

    def _resolve(self, name: str) -> str:
        """The multimodal checkpoints keep the text model under ``model.language_model.``."""
        if name not in self.where and name.startswith("model.") and ("model.language_model." + name[6:]) in self.where:
            return "model.language_model." + name[6:]
        return name

    def _raw(self, name: str) -> torch.Tensor:
        name = self._resolve(name)
        t = self.where[name].get(name)
        if t.dtype == torch.float8_e4m3fn:
            s = self.where[name + "_scale_inv"].get(name + "_scale_inv")
            rows, cols = t.shape
            if s.dtype == torch.uint8:                                  # MXFP8: E8M0 per 1 x 32
                scale = (s.to(torch.int32) << 23).view(torch.float32)
                return (t.to(torch.float32).reshape(rows, cols // 32, 32) * scale.unsqueeze(-1)).reshape(rows, cols)
            sc = s.to(torch.float32).repeat_interleave(128, 0)[:rows].repeat_interleave(128, 1)[:, :cols]   # f32 per 128 x 128
            return t.to(torch.float32) * sc
        if t.dtype == torch.uint8 and (name + "_scale") in self.where:  # MXFP4
            return mxfp4_dequant(t, self.where[name + "_scale"].get(name + "_scale"))
        return t.to(torch.float32, copy=True)           # a copy also for F32 tensors: the file's mapping ends with this object

    def has(self, name: str) -> bool:
        return self._resolve(hf_name(name)) in self.where

    def get(self, name: str, shape) -> torch.Tensor:
        t = self._raw(hf_name(name))
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"{name}: checkpoint has shape {tuple(t.shape)}, model wants {tuple(shape)}")
        return t

    def get_expert(self, name: str, e: int, shape) -> torch.Tensor:
        return self._raw(hf_name(name, e))


class HFQwen35Source(SafetensorsSource):
    """Qwen3.5 (dense and MoE hybrids) from the Hugging Face layout, served under the GGUF tensor names the model builder asks for.
    What changes on the way (the inverse of what a GGUF converter does; the same rules as ``utils.hf_compare.hf_qwen35_model``):
    RMSNorm weights are stored as ``w`` and used as ``1 + w``; value head ``j`` of a Delta-Net layer belongs to key head ``j // R``
    there and to ``j % Hk`` here, so the value-head blocks of ``in_proj_qkv``, ``in_proj_z``, ``in_proj_a / b``, ``conv1d``, ``A_log``,
    ``dt_bias`` and the columns of ``out_proj`` are permuted; ``ssm_a = -exp(A_log)``; the convolution weight drops its singleton axis;
    experts come one tensor per expert or stacked (``experts.gate_up_proj`` [E, 2 I, H])."""

    _LIN = {"attn_qkv": "in_proj_qkv.weight", "attn_gate": "in_proj_z.weight", "ssm_alpha": "in_proj_a.weight", "ssm_beta": "in_proj_b.weight",
            "ssm_out": "out_proj.weight", "ssm_conv1d": "conv1d.weight", "ssm_norm": "norm.weight"}
    _ATT = {"attn_q": "q_proj", "attn_k": "k_proj", "attn_v": "v_proj", "attn_output": "o_proj", "attn_q_norm": "q_norm", "attn_k_norm": "k_norm"}
    _FFN = {"ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj", "ffn_gate_inp": "mlp.gate",
            "ffn_gate_shexp": "mlp.shared_expert.gate_proj", "ffn_up_shexp": "mlp.shared_expert.up_proj", "ffn_down_shexp": "mlp.shared_expert.down_proj",
            "ffn_gate_inp_shexp": "mlp.shared_expert_gate"}

    def __init__(self, path: str, cfg: ModelConfig):
        super().__init__(path)
        self.cfg = cfg
        self.prefix = "model.language_model." if any(k.startswith("model.language_model.") for k in self.where) else "model."
        hk, hv, ds = cfg.ssm_n_heads_k, cfg.ssm_n_heads_v, cfg.ssm_head_dim
        r = hv // hk
        # our value head i = (i % hk) + hk * (i // hk) sits at their index (i % hk) * r + i // hk
        self.heads = torch.tensor([(i % hk) * r + i // hk for i in range(hv)])
        self.vrows = (self.heads[:, None] * ds + torch.arange(ds)[None, :]).reshape(-1)
        self.chan = torch.cat([torch.arange(2 * hk * ds), 2 * hk * ds + self.vrows])

    def _name(self, name: str) -> str:
        if name == "token_embd.weight":
            return self.prefix + "embed_tokens.weight"
        if name == "output_norm.weight":
            return self.prefix + "norm.weight"
        if name == "output.weight":
            return "lm_head.weight"
        _, li, rest = name.split(".", 2)
        base, _, kind = rest.rpartition(".")
        if not base:                                             # "ssm_a": a bare parameter
            base, kind = rest, ""
        lp = f"{self.prefix}layers.{li}."
        if base == "attn_norm":
            return lp + "input_layernorm.weight"
        if base in ("ffn_norm", "post_attention_norm"):
            return lp + "post_attention_layernorm.weight"
        if base in self._LIN:
            return lp + "linear_attn." + self._LIN[base]
        if base == "ssm_a":
            return lp + "linear_attn.A_log"
        if base == "ssm_dt":
            return lp + "linear_attn.dt_bias"
        if base in self._ATT:
            return lp + "self_attn." + self._ATT[base] + "." + kind
        return lp + self._FFN[base] + "." + kind

    def has(self, name: str) -> bool:
        return self._name(name) in self.where

    def get(self, name: str, shape) -> torch.Tensor:
        t = self._raw(self._name(name))
        base = name.split(".", 2)[2].rpartition(".")[0] if name.startswith("blk.") else name.rpartition(".")[0]
        if name.startswith("blk.") and not base:
            base = name.split(".", 2)[2]
        if base in ("attn_norm", "ffn_norm", "post_attention_norm", "attn_q_norm", "attn_k_norm", "output_norm"):
            t = t + 1.0
        elif base == "attn_qkv":
            t = t[self.chan]
        elif base == "ssm_conv1d":
            t = t.reshape(t.shape[0], -1)[self.chan]
        elif base == "attn_gate":
            t = t[self.vrows]
        elif base in ("ssm_alpha", "ssm_beta"):
            t = t[self.heads]
        elif base == "ssm_out":
            t = t[:, self.vrows]
        elif base == "ssm_a":
            t = -torch.exp(t[self.heads])
        elif base == "ssm_dt":
            t = t[self.heads]
        elif base == "ffn_gate_inp_shexp":
            t = t.reshape(-1)
        t = t.contiguous()
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"{name}: checkpoint has shape {tuple(t.shape)}, model wants {tuple(shape)}")
        return t

    def get_expert(self, name: str, e: int, shape) -> torch.Tensor:
        _, li, rest = name.split(".", 2)
        lp = f"{self.prefix}layers.{li}.mlp.experts."
        which = {"ffn_gate_exps": "gate_proj", "ffn_up_exps": "up_proj", "ffn_down_exps": "down_proj"}[rest.rsplit(".", 1)[0]]
        if f"{lp}{e}.{which}.weight" in self.where:
            return self._raw(f"{lp}{e}.{which}.weight")
        inter = self.cfg.expert_ffn                                 # stacked: [E, 2 I, H] = gate rows then up rows, and [E, H, I]
        if which == "down_proj":
            return self._raw(lp + "down_proj")[e].contiguous()
        gu = self._raw(lp + "gate_up_proj")[e]
        return (gu[:inter] if which == "gate_proj" else gu[inter:]).contiguous()


def _qwen35_config_from_hf(c: dict) -> ModelConfig:
    c = c.get("text_config", c)
    moe = "moe" in c.get("model_type", "")
    rp = c.get("rope_parameters") or {}
    hd = c.get("head_dim", c["hidden_size"] // c["num_attention_heads"])
    factor = rp.get("partial_rotary_factor", c.get("partial_rotary_factor", 1.0))
    types = c.get("layer_types") or []
    interval = (types.index("full_attention") + 1) if "full_attention" in types else int(c.get("full_attention_interval", 4))
    sections = list(rp.get("mrope_section") or [])
    return ModelConfig(
        arch="qwen35moe" if moe else "qwen35", n_layers=c["num_hidden_layers"], hidden=c["hidden_size"], n_heads=c["num_attention_heads"],
        n_kv_heads=c.get("num_key_value_heads", c["num_attention_heads"]), head_dim=hd, ffn=c.get("intermediate_size", 0) or 0, vocab=c["vocab_size"],
        rms_eps=c.get("rms_norm_eps", 1e-6), rope_theta=float(rp.get("rope_theta") or c.get("rope_theta") or 1e7), rope_dim=int(round(hd * factor)),
        qk_norm=True, qkv_bias=False, tie_embeddings=c.get("tie_word_embeddings", False), max_seq_len=c.get("max_position_embeddings", 4096),
        full_attention_interval=interval, ssm_d_conv=c.get("linear_conv_kernel_dim", 4), ssm_n_heads_k=c["linear_num_key_heads"],
        ssm_n_heads_v=c["linear_num_value_heads"], ssm_head_dim=c["linear_key_head_dim"], attn_output_gate=True,
        mrope_sections=(sections + [0] * (4 - len(sections))) if sections else None,
        n_experts=int(c.get("num_experts") or c.get("num_local_experts") or 0) if moe else 0, n_experts_used=c.get("num_experts_per_tok", 0) if moe else 0,
        expert_ffn=c.get("moe_intermediate_size", 0) if moe else 0, shared_expert_ffn=c.get("shared_expert_intermediate_size", 0) if moe else 0,
        norm_topk=True)


def config_from_hf(path: str) -> ModelConfig:
    with open(os.path.join(path, "config.json")) as fh:
        c = json.load(fh)
    mt = c.get("model_type", "qwen3")
    if mt.startswith("qwen3_5"):
        return _qwen35_config_from_hf(c)
    vl_sections, n_deepstack = None, 0
    if mt.startswith("qwen3_vl") or mt.startswith("qwen2_vl") or mt.startswith("qwen2_5_vl"):
        # the text side of a vision-language checkpoint: its own sub-configuration, M-RoPE sections, one DeepStack slice per listed
        # vision layer
        n_deepstack = len((c.get("vision_config") or {}).get("deepstack_visual_indexes") or [])
        tie = c.get("tie_word_embeddings", False)
        c = dict(c.get("text_config", c))
        c.setdefault("tie_word_embeddings", tie)
        sec = list(((c.get("rope_parameters") or c.get("rope_scaling") or {}).get("mrope_section")) or [])
        vl_sections = (sec + [0] * (4 - len(sec))) if sec else None
        mt = {"qwen3_vl_moe": "qwen3_vl_moe", "qwen3_vl_moe_text": "qwen3_vl_moe", "qwen3_vl": "qwen3_vl", "qwen3_vl_text": "qwen3_vl"}.get(mt, "qwen2_vl")
    arch = {"qwen2": "qwen2", "qwen3": "qwen3", "qwen3_moe": "qwen3moe", "qwen3_vl": "qwen3vl", "qwen3_vl_moe": "qwen3vlmoe", "qwen2_vl": "qwen2vl"}.get(mt, "qwen3")
    hidden, heads = c["hidden_size"], c["num_attention_heads"]
    # two generations of config.json: ``rope_theta`` / ``num_experts`` at the top level (the checkpoints on the Hub), or
    # ``rope_parameters.rope_theta`` / ``num_local_experts`` (what current transformers writes)
    rope_theta = c.get("rope_theta") or (c.get("rope_parameters") or {}).get("rope_theta") or 1e6
    n_experts = c.get("num_experts") or c.get("num_local_experts") or 0
    return ModelConfig(arch=arch, n_layers=c["num_hidden_layers"], hidden=hidden, n_heads=heads, n_kv_heads=c.get("num_key_value_heads", heads),
                       head_dim=c.get("head_dim", hidden // heads), ffn=c.get("intermediate_size", 0), vocab=c["vocab_size"],
                       rms_eps=c.get("rms_norm_eps", 1e-6), rope_theta=float(rope_theta), qk_norm=(mt not in ("qwen2", "qwen2_vl")), qkv_bias=(mt in ("qwen2", "qwen2_vl")),
                       tie_embeddings=c.get("tie_word_embeddings", False), max_seq_len=c.get("max_position_embeddings", 4096),
                       n_experts=int(n_experts), n_experts_used=c.get("num_experts_per_tok", 0) if n_experts else 0,
                       expert_ffn=c.get("moe_intermediate_size", 0), norm_topk=c.get("norm_topk_prob", True), mrope_sections=vl_sections,
                       n_deepstack_layers=n_deepstack)


def load_safetensors(path: str, fmt: str = "bf16", device="cuda", cfg: Optional[ModelConfig] = None, **shard) -> ModelWeights:
    """Load an HF checkpoint directory (config.json + *.safetensors)."""
    cfg = cfg or config_from_hf(path)
    src = HFQwen35Source(path, cfg) if cfg.is_hybrid else SafetensorsSource(path)
    return build_weights(cfg, src, fmt, device, **shard)


def save_hf_checkpoint(cfg: ModelConfig, src, path: str, mxfp8: bool = False) -> None:
    """Write ``src`` as an HF-layout directory (one safetensors file + config.json); ``mxfp8`` stores the projection matrices
    as F8_E4M3 + ``_scale_inv`` E8M0 the way MXFP8 checkpoints do."""
    from ..ops import mxfp8 as MX
    os.makedirs(path, exist_ok=True)
    out: Dict[str, torch.Tensor] = {}
    h, d = cfg.hidden, cfg.head_dim

    def put(name, t, quant, expert=None):
        key = hf_name(name, expert)
        if quant and mxfp8:
            q, e = MX.quantize_rowmajor(t.float())
            out[key] = q.view(torch.float8_e4m3fn)
            out[key + "_scale_inv"] = e
        else:
            out[key] = t.to(torch.bfloat16)

    put("token_embd.weight", src.get("token_embd.weight", (cfg.vocab, h)), False)
    put("output_norm.weight", src.get("output_norm.weight", (h,)), False)
    if not cfg.tie_embeddings:
        put("output.weight", src.get("output.weight", (cfg.vocab, h)), False)
    for li in range(cfg.n_layers):
        p = f"blk.{li}."
        for nm, shp, qn in (("attn_norm.weight", (h,), False), ("attn_q.weight", (cfg.q_dim, h), True), ("attn_k.weight", (cfg.kv_dim, h), True),
                            ("attn_v.weight", (cfg.kv_dim, h), True), ("attn_output.weight", (h, cfg.q_dim), True), ("ffn_norm.weight", (h,), False)):
            put(p + nm, src.get(p + nm, shp), qn)
        if cfg.qk_norm:
            put(p + "attn_q_norm.weight", src.get(p + "attn_q_norm.weight", (d,)), False)
            put(p + "attn_k_norm.weight", src.get(p + "attn_k_norm.weight", (d,)), False)
        if cfg.qkv_bias:
            for nm, n in (("attn_q.bias", cfg.q_dim), ("attn_k.bias", cfg.kv_dim), ("attn_v.bias", cfg.kv_dim)):
                put(p + nm, src.get(p + nm, (n,)), False)
        if cfg.is_moe:
            put(p + "ffn_gate_inp.weight", src.get(p + "ffn_gate_inp.weight", (cfg.n_experts, h)), False)
            for e in range(cfg.n_experts):
                put(p + "ffn_gate_exps.weight", src.get_expert(p + "ffn_gate_exps.weight", e, (cfg.expert_ffn, h)), True, e)
                put(p + "ffn_up_exps.weight", src.get_expert(p + "ffn_up_exps.weight", e, (cfg.expert_ffn, h)), True, e)
                put(p + "ffn_down_exps.weight", src.get_expert(p + "ffn_down_exps.weight", e, (h, cfg.expert_ffn)), True, e)
        else:
            put(p + "ffn_gate.weight", src.get(p + "ffn_gate.weight", (cfg.ffn, h)), True)
            put(p + "ffn_up.weight", src.get(p + "ffn_up.weight", (cfg.ffn, h)), True)
            put(p + "ffn_down.weight", src.get(p + "ffn_down.weight", (h, cfg.ffn)), True)
    save_safetensors(out, os.path.join(path, "model.safetensors"))
    mt = {"qwen2": "qwen2", "qwen3": "qwen3", "qwen3moe": "qwen3_moe"}.get(cfg.arch, "qwen3")
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump({"model_type": mt, "architectures": [{"qwen2": "Qwen2ForCausalLM", "qwen3": "Qwen3ForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM"}[mt]],
                   "hidden_size": h, "num_attention_heads": cfg.n_heads, "num_key_value_heads": cfg.n_kv_heads, "head_dim": d,
                   "num_hidden_layers": cfg.n_layers, "intermediate_size": cfg.ffn, "vocab_size": cfg.vocab, "rms_norm_eps": cfg.rms_eps,
                   "rope_theta": cfg.rope_theta, "tie_word_embeddings": cfg.tie_embeddings, "max_position_embeddings": cfg.max_seq_len,
                   "num_experts": cfg.n_experts, "num_experts_per_tok": cfg.n_experts_used, "moe_intermediate_size": cfg.expert_ffn,
                   "norm_topk_prob": cfg.norm_topk}, fh)
