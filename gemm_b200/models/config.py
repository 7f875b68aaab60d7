"""Model hyper-parameters and the named shapes used by the benchmarks and tests.

The fields mirror the GGUF keys the reference reads (common/transformer.h:1604-1636 and
cuda/llm/cuda_llm_runner.c:11277-11310): ``<arch>.embedding_length``, ``attention.head_count``,
``attention.head_count_kv``, ``block_count``, ``feed_forward_length``, ``vocab_size``,
``attention.layer_norm_rms_epsilon``, ``rope.freq_base``, ``expert_count``, ``expert_used_count``,
``expert_feed_forward_length``, ``attention.key_length``, ``rope.dimension_count``, the ``ssm.*`` family and
``attention.full_attention_interval`` of the Qwen3.5 hybrids.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, replace
from typing import Dict, List, Optional

ARCHS = ("qwen2", "qwen2vl", "qwen3", "qwen3vl", "qwen3moe", "qwen3vlmoe", "qwen35", "qwen35moe")


@dataclass
class ModelConfig:
    arch: str = "qwen3"
    n_layers: int = 2
    hidden: int = 256
    n_heads: int = 4
    n_kv_heads: int = 2
    head_dim: int = 64
    ffn: int = 512
    vocab: int = 1024
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    rope_dim: Optional[int] = None          # partial rotary (None = head_dim)
    qk_norm: bool = True
    qkv_bias: bool = False                  # Qwen2
    tie_embeddings: bool = False
    max_seq_len: int = 4096
    sliding_window: int = 0
    # MoE
    n_experts: int = 0
    n_experts_used: int = 0
    expert_ffn: int = 0
    norm_topk: bool = True
    router: str = "softmax"                 # or "sigmoid" (MiniMax-M3 / GLM-5 style, with selection bias)
    routed_scale: float = 1.0
    shared_expert_ffn: int = 0              # qwen35moe shared expert (sigmoid-gated)
    # Qwen3.5 hybrid (Delta-Net) layers
    full_attention_interval: int = 0        # every n-th layer is full attention, the rest are SSM layers
    ssm_d_conv: int = 4
    ssm_n_heads_k: int = 0
    ssm_n_heads_v: int = 0
    ssm_head_dim: int = 0
    attn_output_gate: bool = False          # attn_q emits [Q | gate] per head, output *= sigmoid(gate)
    # M-RoPE (Qwen2-VL / Qwen3-VL): sections of rotary pairs assigned to t / h / w
    mrope_sections: Optional[List[int]] = None
    n_deepstack_layers: int = 0

    @property
    def is_moe(self) -> bool:
        return self.n_experts > 0

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def is_hybrid(self) -> bool:
        return self.full_attention_interval > 0

    @property
    def ssm_d_inner(self) -> int:
        return self.ssm_n_heads_v * self.ssm_head_dim

    @property
    def ssm_qkv_dim(self) -> int:
        return 2 * self.ssm_n_heads_k * self.ssm_head_dim + self.ssm_d_inner

    def is_ssm_layer(self, layer: int) -> bool:
        if self.full_attention_interval <= 0:
            return False
        return (layer + 1) % self.full_attention_interval != 0

    def param_count(self) -> int:
        per_layer = self.hidden * (self.q_dim + 2 * self.kv_dim) + self.q_dim * self.hidden
        if self.is_moe:
            per_layer += self.n_experts * 3 * self.hidden * self.expert_ffn + self.n_experts * self.hidden
        else:
            per_layer += 3 * self.hidden * self.ffn
        emb = self.vocab * self.hidden * (1 if self.tie_embeddings else 2)
        return per_layer * self.n_layers + emb

    def to_dict(self) -> Dict:
        return asdict(self)

    def with_(self, **kw) -> "ModelConfig":
        return replace(self, **kw)


def _qwen3(name, **kw) -> ModelConfig:
    return ModelConfig(arch="qwen3", head_dim=128, vocab=151936, **kw)


PRESETS: Dict[str, ModelConfig] = {
    # the five benchmark shapes
    "qwen3-0.6b": _qwen3("0.6b", n_layers=28, hidden=1024, n_heads=16, n_kv_heads=8, ffn=3072, tie_embeddings=True),
    "qwen3-8b": _qwen3("8b", n_layers=36, hidden=4096, n_heads=32, n_kv_heads=8, ffn=12288),
    "qwen3-32b": _qwen3("32b", n_layers=64, hidden=5120, n_heads=64, n_kv_heads=8, ffn=25600),
    "qwen3-30b-a3b": ModelConfig(arch="qwen3moe", n_layers=48, hidden=2048, n_heads=32, n_kv_heads=4, head_dim=128, ffn=6144,
                                 vocab=151936, n_experts=128, n_experts_used=8, expert_ffn=768),
    "qwen3-235b-a22b": ModelConfig(arch="qwen3moe", n_layers=94, hidden=4096, n_heads=64, n_kv_heads=4, head_dim=128, ffn=12288,
                                   vocab=151936, n_experts=128, n_experts_used=8, expert_ffn=1536),
    # small shapes for tests (head_dim 128 so that the tcgen05 attention kernel applies)
    "tiny-dense": ModelConfig(arch="qwen3", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=128, ffn=512, vocab=512),
    "tiny-moe": ModelConfig(arch="qwen3moe", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=128, ffn=512, vocab=512,
                            n_experts=16, n_experts_used=4, expert_ffn=128),
    # hybrid: layers 0 and 2 are Delta-Net layers, 1 and 3 gated full attention; the MoE variant adds a shared expert
    "tiny-qwen35": ModelConfig(arch="qwen35", n_layers=4, hidden=256, n_heads=4, n_kv_heads=2, head_dim=128, ffn=512, vocab=512,
                               rope_dim=64, full_attention_interval=2, ssm_d_conv=4, ssm_n_heads_k=2, ssm_n_heads_v=4, ssm_head_dim=64,
                               attn_output_gate=True, mrope_sections=[11, 11, 10, 0]),
    "tiny-qwen35moe": ModelConfig(arch="qwen35moe", n_layers=4, hidden=256, n_heads=4, n_kv_heads=2, head_dim=128, ffn=512, vocab=512,
                                  rope_dim=64, full_attention_interval=2, ssm_d_conv=4, ssm_n_heads_k=2, ssm_n_heads_v=4, ssm_head_dim=64,
                                  attn_output_gate=True, mrope_sections=[11, 11, 10, 0], n_experts=16, n_experts_used=4, expert_ffn=128, shared_expert_ffn=128),
    "tiny-qwen2": ModelConfig(arch="qwen2", n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=128, ffn=512, vocab=512,
                              qk_norm=False, qkv_bias=True, tie_embeddings=True),
}


def get_config(name: str) -> ModelConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown model preset {name!r}; known: {sorted(PRESETS)}")
    return replace(PRESETS[name])
