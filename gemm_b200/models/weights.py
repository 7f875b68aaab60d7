"""Weight containers and the synthetic (random-init) checkpoint generator.

A ``LinearWeight`` keeps one projection in the format the kernels consume:

* ``bf16``   row-major ``[N, K]``
* ``mxfp8``  e4m3 bytes + E8M0 scale atoms (``ops.mxfp8.MxTensor``)

Grouped (expert) weights use the same class with ``groups > 0`` and rows stacked expert after expert.
Tensor-parallel and expert-parallel shards are cut when the weights are made or loaded, never at run
time (the reference slices TP rows out of the full matrix on every call, common/transformer.h:4239-4272).

Random init follows the benchmark recipe: N(0, 0.02) for matrices, ones for norms, seeded per tensor so
that a sharded model is a slice of the unsharded one.
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..ops import elementwise as ew
from ..ops import mxfp8
from ..ops.mxfp8 import MxTensor
from .config import ModelConfig


@dataclass
class LinearWeight:
    fmt: str                                  # "bf16" | "mxfp8" | "q4_k" | "q8_0" (ggml blocks kept quantised in HBM)
    n: int                                    # output features (per group)
    k: int
    w: Optional[torch.Tensor] = None          # bf16 [rows, K]
    mx: Optional[MxTensor] = None
    q: Optional["QTensor"] = None             # tiled ggml blocks (``ops.qlinear.QTensor``)
    bias: Optional[torch.Tensor] = None       # f32 [n]
    groups: int = 0                           # > 0: expert-stacked, rows = groups * rows_per_group
    rows_per_group: int = 0
    tiled: bool = False                       # bf16 ``w`` is in the tiled layout (``mx.tiled`` for MXFP8)

    @property
    def is_quant(self) -> bool:
        return self.q is not None

    @property
    def is_tiled(self) -> bool:
        if self.is_quant:
            return True
        return self.tiled if self.fmt == "bf16" else self.mx.tiled

    def tile_(self) -> "LinearWeight":
        """Re-lay the matrix in place into the GEMM kernel's tiled weight layout (``ops.mxfp8.tile_weight``)."""
        if self.is_quant:
            return self                       # ggml blocks are stored in their own tile order from the start
        t = self.w if self.fmt == "bf16" else self.mx.data
        if self.is_tiled or not mxfp8.can_tile(t) or (self.groups and self.rows_per_group % 128):
            return self
        t.copy_(mxfp8.tile_weight(t))
        if self.fmt == "bf16":
            self.tiled = True
        else:
            self.mx.tiled = True
        return self

    def untiled_data(self) -> torch.Tensor:
        """Row-major copy of the stored matrix (bf16 values or e4m3 bytes)."""
        t = self.w if self.fmt == "bf16" else self.mx.data
        return mxfp8.untile_weight(t) if self.is_tiled else t

    @property
    def device(self):
        if self.is_quant:
            return self.q.data.device
        return self.w.device if self.w is not None else self.mx.data.device

    def dequantized(self) -> torch.Tensor:
        """fp32 copy of the full matrix (tests and CPU reference paths)."""
        if self.is_quant:
            return self.q.dequantize()
        if self.fmt == "bf16":
            return self.untiled_data().float()
        return mxfp8.dequantize(self.mx)

    def nbytes(self) -> int:
        if self.is_quant:
            return self.q.nbytes()
        if self.fmt == "bf16":
            return self.w.numel() * 2
        return self.mx.data.numel() + self.mx.sf.numel()

    def to(self, device) -> "LinearWeight":
        return LinearWeight(self.fmt, self.n, self.k, w=self.w.to(device) if self.w is not None else None,
                            mx=self.mx.to(device) if self.mx is not None else None, q=self.q.to(device) if self.q is not None else None,
                            bias=self.bias.to(device) if self.bias is not None else None, groups=self.groups,
                            rows_per_group=self.rows_per_group, tiled=self.tiled)


QUANT_FMTS = {"q4_k": 12, "q8_0": 8}          # run-time formats that keep ggml blocks: name -> ggml type id


@dataclass
class QBlocks:
    """A matrix as row-major ggml blocks (the order of a GGUF file): ``raw`` uint8 ``[rows, row_bytes]``.  Supports what weight
    assembly needs without decoding: row ranges, column ranges on block boundaries, stacking along rows."""
    raw: torch.Tensor
    ggml_type: int
    k: int

    @property
    def shape(self):
        return (self.raw.shape[0], self.k)

    def _geom(self):
        from ..ops import ggml_torch as gt
        return gt.BLOCK[self.ggml_type]

    def rows(self, a: int, b: int) -> "QBlocks":
        return QBlocks(self.raw[a:b], self.ggml_type, self.k)

    def cols(self, a: int, b: int) -> "QBlocks":
        blk, nb = self._geom()
        if a % blk or b % blk:
            raise ValueError(f"column range [{a}, {b}) does not fall on {blk}-element block boundaries")
        return QBlocks(self.raw[:, a // blk * nb: b // blk * nb], self.ggml_type, b - a)

    def to(self, device) -> "QBlocks":
        return QBlocks(self.raw.to(device), self.ggml_type, self.k)

    def contiguous(self) -> "QBlocks":
        return QBlocks(self.raw.contiguous(), self.ggml_type, self.k)


def _mat(src, name: str, shape):
    """A projection matrix from a tensor source: its ggml blocks when the source can hand them out (``get_mat``), else floats."""
    return src.get_mat(name, shape) if hasattr(src, "get_mat") else src.get(name, shape)


def _rows(t, a: int, b: int):
    return t.rows(a, b) if isinstance(t, QBlocks) else t[a:b]


def _cols(t, a: int, b: int):
    return t.cols(a, b) if isinstance(t, QBlocks) else t[:, a:b]


def _cat(parts):
    """Stack matrices along rows; quantised parts must share type and width (a mixed list is decoded to float first)."""
    if all(isinstance(p, QBlocks) for p in parts) and len({(p.ggml_type, p.k) for p in parts}) == 1:
        return QBlocks(torch.cat([p.raw for p in parts]), parts[0].ggml_type, parts[0].k)
    return torch.cat([_to_float(p) for p in parts])


def _to_float(t):
    if isinstance(t, QBlocks):
        from ..ops import ggml_torch as gt
        return gt.dequantize(t.raw.contiguous(), t.ggml_type, t.raw.shape[0], t.k).to(torch.bfloat16)
    return t


def make_linear(w_f, fmt: str, bias: Optional[torch.Tensor] = None, groups: int = 0) -> LinearWeight:
    """Wrap a float / bf16 matrix ``[rows, K]`` (rows = groups * rows_per_group when grouped), or ggml blocks (``QBlocks``).

    ``fmt`` "q4_k" / "q8_0" keeps (or makes) ggml blocks and stores them tiled for the fused dequant kernels; blocks of a type
    without such a kernel, or with a width that is not a multiple of 256, are decoded to bf16.  Expert-stacked matrices have no
    quantised path and are stored as bf16 under these formats."""
    from ..ops.qlinear import QTensor
    if fmt in QUANT_FMTS or fmt == "ggml" or isinstance(w_f, QBlocks):
        rows, k = w_f.shape
        want = QUANT_FMTS.get(fmt)
        if groups == 0 and k % 256 == 0 and (want is not None or fmt == "ggml"):
            if isinstance(w_f, QBlocks) and w_f.ggml_type in QUANT_FMTS.values() and (fmt == "ggml" or w_f.ggml_type == want):
                name = {v: n for n, v in QUANT_FMTS.items()}[w_f.ggml_type]       # the file's own blocks, untouched
                return LinearWeight(name, rows, k, q=QTensor.from_blocks(w_f.raw.contiguous(), w_f.ggml_type, rows, k), bias=bias)
            if want is not None:
                return LinearWeight(fmt, rows, k, q=QTensor.from_float(_to_float(w_f).float(), want), bias=bias)
        w_f = _to_float(w_f)
        if fmt in QUANT_FMTS or fmt == "ggml":
            fmt = "bf16"
    rows, k = w_f.shape
    rpg = rows // groups if groups else 0
    n = rpg if groups else rows
    if fmt == "bf16":
        return LinearWeight("bf16", n, k, w=w_f.to(torch.bfloat16).contiguous(), bias=bias, groups=groups, rows_per_group=rpg)
    if fmt == "mxfp8":
        if w_f.is_cuda:
            mx = ew.mx_quantize(w_f.to(torch.bfloat16).contiguous())
        else:
            mx = mxfp8.quantize(w_f.to(torch.bfloat16).float())
        return LinearWeight("mxfp8", n, k, mx=mx, bias=bias, groups=groups, rows_per_group=rpg)
    raise ValueError(f"unknown weight format {fmt!r}")


@dataclass
class SsmWeights:
    """A Delta-Net layer (GGUF names: attn_qkv, attn_gate, ssm_alpha, ssm_beta, ssm_conv1d, ssm_a, ssm_dt.bias, ssm_norm, ssm_out)."""
    w_in: LinearWeight            # rows [qkv (Q | K | V channels) ; z (d_inner)]
    w_ab: torch.Tensor            # bf16 [2 * n_heads_v, H]: alpha rows then beta rows
    conv_w: torch.Tensor          # f32 [qkv_dim, conv_k]
    a: torch.Tensor               # f32 [n_heads_v]
    dt_bias: torch.Tensor         # f32 [n_heads_v]
    norm: torch.Tensor            # f32 [head_dim]
    w_out: LinearWeight           # [H, d_inner]

    def to(self, device) -> "SsmWeights":
        return SsmWeights(self.w_in.to(device), self.w_ab.to(device), self.conv_w.to(device), self.a.to(device), self.dt_bias.to(device),
                          self.norm.to(device), self.w_out.to(device))


@dataclass
class LayerWeights:
    attn_norm: torch.Tensor
    wqkv: Optional[LinearWeight]                  # rows [Q ; K ; V] (+ [gate] after V when the attention output is gated); None in SSM layers
    wo: Optional[LinearWeight]
    ffn_norm: torch.Tensor
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    w_gate_up: Optional[LinearWeight] = None      # dense FFN, rows [gate ; up]
    w_down: Optional[LinearWeight] = None
    router: Optional[torch.Tensor] = None         # bf16 [E, H]
    router_bias: Optional[torch.Tensor] = None    # f32 [E] (sigmoid router)
    w13: Optional[LinearWeight] = None            # experts, rows per expert [gate ; up] = 2I
    w2: Optional[LinearWeight] = None             # experts, rows per expert = H, K = I
    ssm: Optional[SsmWeights] = None              # Delta-Net layer (then wqkv / wo are None)
    sh_gate_up: Optional[LinearWeight] = None     # shared expert [gate ; up]
    sh_down: Optional[LinearWeight] = None
    sh_gate: Optional[torch.Tensor] = None        # bf16 [1, H]: sigmoid gate of the shared expert (absent = ungated)


@dataclass
class ModelWeights:
    cfg: ModelConfig
    embed: torch.Tensor                           # bf16 [V, H]
    layers: List[LayerWeights]
    final_norm: torch.Tensor
    lm_head: LinearWeight                         # bf16 [V(/tp), H]
    fmt: str = "bf16"
    tp_rank: int = 0
    tp_size: int = 1
    ep_rank: int = 0
    ep_size: int = 1
    vocab_start: int = 0                          # first vocabulary id of the LM-head shard

    def to(self, device) -> "ModelWeights":
        def mv(x):
            return x.to(device) if x is not None else None
        layers = [LayerWeights(attn_norm=mv(l.attn_norm), wqkv=mv(l.wqkv), wo=mv(l.wo), ffn_norm=mv(l.ffn_norm), q_norm=mv(l.q_norm),
                               k_norm=mv(l.k_norm), w_gate_up=mv(l.w_gate_up), w_down=mv(l.w_down), router=mv(l.router),
                               router_bias=mv(l.router_bias), w13=mv(l.w13), w2=mv(l.w2), ssm=mv(l.ssm), sh_gate_up=mv(l.sh_gate_up),
                               sh_down=mv(l.sh_down), sh_gate=mv(l.sh_gate)) for l in self.layers]
        return ModelWeights(cfg=self.cfg, embed=mv(self.embed), layers=layers, final_norm=mv(self.final_norm), lm_head=mv(self.lm_head),
                            fmt=self.fmt, tp_rank=self.tp_rank, tp_size=self.tp_size, ep_rank=self.ep_rank, ep_size=self.ep_size,
                            vocab_start=self.vocab_start)

    def tile_(self) -> "ModelWeights":
        """Put every projection matrix into the tiled weight layout (in place).  An LM head that shares its storage with
        the embedding table (tied embeddings) stays row-major: the embedding lookup reads rows."""
        for l in self.layers:
            for lw in (l.wqkv, l.wo, l.w_gate_up, l.w_down, l.w13, l.w2, l.sh_gate_up, l.sh_down) + ((l.ssm.w_in, l.ssm.w_out) if l.ssm else ()):
                if lw is not None:
                    lw.tile_()
        if self.lm_head.w is not None and self.lm_head.w.data_ptr() != self.embed.data_ptr():
            self.lm_head.tile_()
        return self

    def nbytes(self) -> int:
        tot = self.embed.numel() * 2 + self.lm_head.nbytes()
        for l in self.layers:
            for lw in (l.wqkv, l.wo, l.w_gate_up, l.w_down, l.w13, l.w2, l.sh_gate_up, l.sh_down) + ((l.ssm.w_in, l.ssm.w_out) if l.ssm else ()):
                if lw is not None:
                    tot += lw.nbytes()
        return tot


def ffn_shard(f: int, tp_size: int, tp_rank: int, fmt: str):
    """Column range of the FFN width owned by a tensor-parallel rank.  Formats that keep ggml blocks cut on 256-column boundaries
    (a K-quant super-block cannot be split), with the remainder going to the low ranks as in common/glm5.h:178-202 (its
    block-aligned variant); the others split evenly."""
    if (fmt in QUANT_FMTS or fmt == "ggml") and tp_size > 1 and f % 256 == 0:
        lo, hi = shard_range(f // 256, tp_size, tp_rank)
        return lo * 256, hi * 256
    assert f % tp_size == 0
    f_l = f // tp_size
    return tp_rank * f_l, (tp_rank + 1) * f_l


def shard_range(n: int, parts: int, idx: int):
    """Even split with the remainder to the low ranks (the rule of common/glm5.h:178-202)."""
    q, r = divmod(n, parts)
    lo = idx * q + min(idx, r)
    return lo, lo + q + (1 if idx < r else 0)


class RandomSource:
    """Tensor source of a random-init checkpoint: N(0, 0.02) matrices, unit norms, zero biases... every tensor
    (and every expert) has its own seed derived from its GGUF name, so shards are slices of the same model."""

    def __init__(self, cfg: ModelConfig, seed: int = 0, device="cpu", std: float = 0.02):
        self.cfg, self.seed, self.device, self.std = cfg, seed, torch.device(device), std
        self._gen = torch.Generator(device=self.device)

    def _randn(self, key: str, shape) -> torch.Tensor:
        self._gen.manual_seed((zlib.crc32(key.encode()) ^ (self.seed * 2654435761)) & 0x7FFFFFFF)
        return torch.randn(tuple(shape), generator=self._gen, device=self.device, dtype=torch.float32).mul_(self.std).to(torch.bfloat16)

    def has(self, name: str) -> bool:
        return True

    def get(self, name: str, shape) -> torch.Tensor:
        if name.endswith("norm.weight"):
            return torch.ones(tuple(shape), dtype=torch.bfloat16, device=self.device)
        if name.endswith("ssm_a"):                       # fixed decay constants are negative
            return -(self._randn(name, shape).float().abs() * 20 + 0.5).to(torch.bfloat16)
        if name.endswith("ssm_conv1d.weight") or name.endswith("ssm_alpha.weight") or name.endswith("ssm_beta.weight"):
            return (self._randn(name, shape).float() * 10).to(torch.bfloat16)
        if name.endswith(".bias"):
            return self._randn(name, shape)
        return self._randn(name, shape)

    def get_expert(self, name: str, e: int, shape) -> torch.Tensor:
        return self._randn(f"{name}#{e}", shape)


def _post_attn_norm_name(src, pre: str) -> str:
    """The norm before the FFN: ``ffn_norm`` (Qwen2/3) or ``post_attention_norm`` (Qwen3.5 GGUFs)."""
    if hasattr(src, "has") and not isinstance(src, RandomSource) and not src.has(pre + "ffn_norm.weight") and src.has(pre + "post_attention_norm.weight"):
        return "post_attention_norm.weight"
    return "ffn_norm.weight"


def _build_ffn(cfg, src, pre, lw, fmt, mv, dev, tp_rank, tp_size, ep_rank, ep_size) -> None:
    """Dense FFN or MoE (+ optional shared expert) of one layer into ``lw``."""
    h = cfg.hidden
    if cfg.is_moe:
        e, inter = cfg.n_experts, cfg.expert_ffn
        assert e % ep_size == 0
        e_l = e // ep_size
        lw.router = mv(src.get(pre + "ffn_gate_inp.weight", (e, h)).to(torch.bfloat16))
        if cfg.router == "sigmoid":
            lw.router_bias = torch.zeros(e, dtype=torch.float32, device=dev)
        w13 = torch.empty((e_l * 2 * inter, h), dtype=torch.bfloat16, device=dev)
        w2 = torch.empty((e_l * h, inter), dtype=torch.bfloat16, device=dev)
        for j in range(e_l):
            ge = ep_rank * e_l + j
            w13[j * 2 * inter: j * 2 * inter + inter] = mv(src.get_expert(pre + "ffn_gate_exps.weight", ge, (inter, h)))
            w13[j * 2 * inter + inter:(j + 1) * 2 * inter] = mv(src.get_expert(pre + "ffn_up_exps.weight", ge, (inter, h)))
            w2[j * h:(j + 1) * h] = mv(src.get_expert(pre + "ffn_down_exps.weight", ge, (h, inter)))
        lw.w13 = make_linear(w13, fmt, groups=e_l)
        lw.w2 = make_linear(w2, fmt, groups=e_l)
        del w13, w2
    else:
        f = cfg.ffn
        f0, f1 = ffn_shard(f, tp_size, tp_rank, fmt)
        wg = _rows(_mat(src, pre + "ffn_gate.weight", (f, h)), f0, f1)
        wu = _rows(_mat(src, pre + "ffn_up.weight", (f, h)), f0, f1)
        wd = _cols(_mat(src, pre + "ffn_down.weight", (h, f)), f0, f1)
        lw.w_gate_up = make_linear(mv(_cat([wg, wu])), fmt)
        lw.w_down = make_linear(mv(wd.contiguous()), fmt)
        del wg, wu, wd
    if cfg.is_moe and cfg.shared_expert_ffn > 0:
        fs = cfg.shared_expert_ffn
        lw.sh_gate_up = make_linear(mv(torch.cat([src.get(pre + "ffn_gate_shexp.weight", (fs, h)), src.get(pre + "ffn_up_shexp.weight", (fs, h))])), fmt)
        lw.sh_down = make_linear(mv(src.get(pre + "ffn_down_shexp.weight", (h, fs)).contiguous()), fmt)
        if not hasattr(src, "has") or src.has(pre + "ffn_gate_inp_shexp.weight"):
            lw.sh_gate = mv(src.get(pre + "ffn_gate_inp_shexp.weight", (h,)).to(torch.bfloat16).reshape(1, h).contiguous())


def build_weights(cfg: ModelConfig, src, fmt: str = "bf16", device="cuda", tp_rank: int = 0, tp_size: int = 1, ep_rank: int = 0,
                  ep_size: int = 1, shard_vocab: bool = False, n_layers: Optional[int] = None, layer_range=None,
                  tile: Optional[bool] = None) -> ModelWeights:
    """Assemble ``ModelWeights`` in format ``fmt`` from a tensor source that answers GGUF tensor names
    (``RandomSource``, ``loader.GGUFSource``, ``loader.SafetensorsSource``).  ``tile`` (default: on for CUDA devices) stores
    the projection matrices in the GEMM kernel's tiled layout.

    TP shards attention and the dense FFN Megatron style (q/k/v/gate/up by rows, o/down by columns; KV heads are
    replicated when ``n_kv_heads < tp_size``), EP keeps the experts ``[ep_rank * E/ep_size, (ep_rank+1) * E/ep_size)``."""
    h, d = cfg.hidden, cfg.head_dim
    dev = torch.device(device)
    assert cfg.n_heads % tp_size == 0, "n_heads must divide by the TP size"
    hq_l = cfg.n_heads // tp_size
    if cfg.n_kv_heads >= tp_size:
        assert cfg.n_kv_heads % tp_size == 0
        hkv_l = cfg.n_kv_heads // tp_size
        kv_lo = tp_rank * hkv_l
    else:
        assert tp_size % cfg.n_kv_heads == 0
        hkv_l = 1
        kv_lo = tp_rank // (tp_size // cfg.n_kv_heads)
    q0, q1 = tp_rank * hq_l * d, (tp_rank + 1) * hq_l * d
    k0, k1 = kv_lo * d, (kv_lo + hkv_l) * d

    def mv(t):
        return t.to(dev)

    layers: List[LayerWeights] = []
    nl = n_layers if n_layers is not None else cfg.n_layers
    lo, hi = layer_range if layer_range is not None else (0, nl)       # pipeline stages keep a contiguous slice of layers
    for li in range(lo, hi):
        pre = f"blk.{li}."
        if cfg.is_ssm_layer(li):
            assert tp_size == 1, "Delta-Net layers are not tensor-parallel (the reference replicates them, test_transformer_parallel.c:351-364)"
            qd, di, hv = cfg.ssm_qkv_dim, cfg.ssm_d_inner, cfg.ssm_n_heads_v
            w_in = torch.cat([src.get(pre + "attn_qkv.weight", (qd, h)), src.get(pre + "attn_gate.weight", (di, h))])
            ssm = SsmWeights(
                w_in=make_linear(mv(w_in), fmt),
                w_ab=mv(torch.cat([src.get(pre + "ssm_alpha.weight", (hv, h)), src.get(pre + "ssm_beta.weight", (hv, h))]).to(torch.bfloat16).contiguous()),
                conv_w=mv(src.get(pre + "ssm_conv1d.weight", (qd, cfg.ssm_d_conv)).float().contiguous()),
                a=mv(src.get(pre + "ssm_a", (hv,)).float().contiguous()), dt_bias=mv(src.get(pre + "ssm_dt.bias", (hv,)).float().contiguous()),
                norm=mv(src.get(pre + "ssm_norm.weight", (cfg.ssm_head_dim,)).float().contiguous()),
                w_out=make_linear(mv(src.get(pre + "ssm_out.weight", (h, di)).contiguous()), fmt))
            del w_in
            lw = LayerWeights(attn_norm=mv(src.get(pre + "attn_norm.weight", (h,)).to(torch.bfloat16)), wqkv=None, wo=None,
                              ffn_norm=mv(src.get(pre + _post_attn_norm_name(src, pre), (h,)).to(torch.bfloat16)), ssm=ssm)
            _build_ffn(cfg, src, pre, lw, fmt, mv, dev, tp_rank, tp_size, ep_rank, ep_size)
            layers.append(lw)
            continue
        if cfg.attn_output_gate:
            # attn_q emits [Q_h | gate_h] per head (common/transformer.h:3857-3868): de-interleave, the gate rows go after V
            wqg = src.get(pre + "attn_q.weight", (2 * cfg.q_dim, h)).reshape(cfg.n_heads, 2, d, h)
            wq = wqg[:, 0].reshape(cfg.q_dim, h)[q0:q1]
            wgate = wqg[:, 1].reshape(cfg.q_dim, h)[q0:q1]
        else:
            wq = _rows(_mat(src, pre + "attn_q.weight", (cfg.q_dim, h)), q0, q1)
            wgate = None
        wk = _rows(_mat(src, pre + "attn_k.weight", (cfg.kv_dim, h)), k0, k1)
        wv = _rows(_mat(src, pre + "attn_v.weight", (cfg.kv_dim, h)), k0, k1)
        wo = _cols(_mat(src, pre + "attn_output.weight", (h, cfg.q_dim)), q0, q1)
        bias = None
        if cfg.qkv_bias:
            bias = torch.cat([src.get(pre + "attn_q.bias", (cfg.q_dim,))[q0:q1].float(), src.get(pre + "attn_k.bias", (cfg.kv_dim,))[k0:k1].float(),
                              src.get(pre + "attn_v.bias", (cfg.kv_dim,))[k0:k1].float()]).contiguous()
            bias = mv(bias)
        lw = LayerWeights(
            attn_norm=mv(src.get(pre + "attn_norm.weight", (h,)).to(torch.bfloat16)),
            wqkv=make_linear(mv(_cat([wq, wk, wv] + ([wgate] if wgate is not None else []))), fmt, bias=bias),
            wo=make_linear(mv(wo.contiguous()), fmt),
            ffn_norm=mv(src.get(pre + _post_attn_norm_name(src, pre), (h,)).to(torch.bfloat16)),
            q_norm=mv(src.get(pre + "attn_q_norm.weight", (d,)).to(torch.bfloat16)) if cfg.qk_norm else None,
            k_norm=mv(src.get(pre + "attn_k_norm.weight", (d,)).to(torch.bfloat16)) if cfg.qk_norm else None,
        )
        del wq, wk, wv, wo
        _build_ffn(cfg, src, pre, lw, fmt, mv, dev, tp_rank, tp_size, ep_rank, ep_size)
        layers.append(lw)
    embed_src = _mat(src, "token_embd.weight", (cfg.vocab, h))
    embed = mv(_to_float(embed_src).to(torch.bfloat16))          # the embedding lookup reads bf16 rows
    quant_head = fmt in QUANT_FMTS or fmt == "ggml"
    if cfg.tie_embeddings or not src.has("output.weight"):
        head_full = embed_src if (quant_head and isinstance(embed_src, QBlocks)) else embed
    else:
        head_src = _mat(src, "output.weight", (cfg.vocab, h))
        head_full = head_src if (quant_head and isinstance(head_src, QBlocks)) else mv(_to_float(head_src).to(torch.bfloat16))
    v0, v1 = (0, cfg.vocab)
    if shard_vocab and tp_size > 1:
        v0, v1 = shard_range(cfg.vocab, tp_size, tp_rank)
    head_rows = _rows(head_full, v0, v1).contiguous() if (v0, v1) != (0, cfg.vocab) else head_full
    # the LM head streams the largest matrix of a decode step: under the block formats it stays quantised too
    lm_head = make_linear(mv(head_rows), fmt if quant_head else "bf16")
    mw = ModelWeights(cfg=cfg, embed=embed, layers=layers, final_norm=mv(src.get("output_norm.weight", (h,)).to(torch.bfloat16)),
                      lm_head=lm_head, fmt=fmt, tp_rank=tp_rank, tp_size=tp_size, ep_rank=ep_rank, ep_size=ep_size, vocab_start=v0)
    if tile if tile is not None else dev.type == "cuda":
        mw.tile_()
    return mw


def synthetic_weights(cfg: ModelConfig, fmt: str = "bf16", device="cuda", seed: int = 0, tp_rank: int = 0, tp_size: int = 1,
                      ep_rank: int = 0, ep_size: int = 1, shard_vocab: bool = False, n_layers: Optional[int] = None,
                      layer_range=None) -> ModelWeights:
    """Random-init weights of ``cfg`` (generated on ``device``) in format ``fmt``."""
    return build_weights(cfg, RandomSource(cfg, seed, device), fmt, device, tp_rank, tp_size, ep_rank, ep_size, shard_vocab, n_layers,
                         layer_range)
