"""Roofline estimate of decode and prefill throughput of a model configuration on B200s.

``python -m gemm_b200 estimate --model qwen3-30b-a3b --batch 64 --ctx 2048 --gpus 8 --format mxfp8``

Per decode step the time is the larger of the memory-bound part (bytes every GPU must read from HBM: the weights it
touches once per step, the KV cache of its sequences) and the communication-bound part (bytes it must move over NVLink),
plus a fixed cost per kernel launch; prefill adds the tensor-core time.  Weights amortise over the batch, KV does not;
an MoE layer touches only the experts some token selected: E * (1 - (1 - k/E)^B) of them in expectation.  The numbers
are ceilings (routing, softmax and launch gaps beyond the fixed term are not modelled); ``--derate`` applies an
efficiency factor.  Also reports whether weights + KV fit in HBM.  ``--cp 1,2,4,8`` prints the cost model of context-parallel
decode attention instead (KV shard read time, size of the flash partial, all-gather / ring / tree merge times).

Counterpart in the reference: tools/decode_estimate.py (per-step time = max(memory, communication), fit check, the same
treatment of batch and context), with the platform constants replaced by this machine's measured ones.
"""
from __future__ import annotations

import argparse
import json
from dataclasses import dataclass

from ..models.config import ModelConfig, get_config


@dataclass
class Platform:
    hbm_gbs: float = 6535.0          # measured copy bandwidth
    hbm_gib: float = 180.0
    nvlink_gbs: float = 770.0        # measured peer copy, per direction per GPU
    tensor_tflops: float = 1667.5    # measured cuBLAS bf16 burst
    fp8_speedup: float = 1.15        # measured: block-scaled e4m3 GEMM against the bf16 figure above
    launch_us: float = 4.0           # fixed cost per kernel in a programmatic-dependent-launch chain
    kernels_per_layer: int = 13


def _bytes_per_weight(fmt: str) -> float:
    return {"bf16": 2.0, "mxfp8": 1.0 + 1.0 / 32.0}[fmt]


def layer_params(cfg: ModelConfig):
    """(attention, dense-or-shared FFN, one expert, router) parameter counts of one layer."""
    d = cfg.head_dim
    attn = cfg.hidden * (cfg.n_heads + 2 * cfg.n_kv_heads) * d + cfg.n_heads * d * cfg.hidden
    if cfg.n_experts > 0:
        expert = 3 * cfg.hidden * cfg.expert_ffn
        dense = 3 * cfg.hidden * cfg.shared_expert_ffn
        router = cfg.hidden * cfg.n_experts
    else:
        expert, router = 0, 0
        dense = 3 * cfg.hidden * cfg.ffn
    return attn, dense, expert, router


def experts_touched(n_experts: int, k: int, tokens: int) -> float:
    """Expected number of distinct experts chosen by ``tokens`` tokens routing uniformly to ``k`` of ``n_experts``."""
    if n_experts == 0:
        return 0.0
    return n_experts * (1.0 - (1.0 - k / n_experts) ** tokens)


def estimate(cfg: ModelConfig, batch: int, ctx: int, gpus: int = 1, fmt: str = "mxfp8", mode: str = "ep", plat: Platform = Platform(),
             derate: float = 1.0, prefill_chunk: int = 16384) -> dict:
    """``mode`` "ep": experts sharded over the GPUs, attention replicated, the batch split by GPU (data-parallel attention);
    "tp": every projection sharded, batch replicated; "tp+ep": attention sharded by heads with the batch replicated, whole
    experts spread over the same GPUs (``parallel.tensor.TensorParallel(ep_experts=True)``): per layer one slot reduction
    after o_proj and one after the experts, no token exchange."""
    bw = _bytes_per_weight(fmt)
    attn, dense, expert, router = layer_params(cfg)
    n_layers = cfg.n_layers
    kv_tok = 2 * cfg.n_kv_heads * cfg.head_dim * 2                      # bytes per token per layer (bf16 K and V)
    head = cfg.vocab * cfg.hidden * 2                                   # LM head stays bf16
    hybrid = mode == "tp+ep"
    mode = "tp" if hybrid else mode
    local_batch = batch if mode == "tp" else -(-batch // gpus)
    # ---- decode: bytes one GPU reads per step
    touched = experts_touched(cfg.n_experts, cfg.n_experts_used, batch)
    if mode == "tp":
        # whole experts per GPU (hybrid) or every expert cut by columns (plain TP): the same bytes per GPU either way
        w_layer = (attn + dense + touched * expert) * bw / gpus + router * 2
        kv_layer = batch * ctx * kv_tok / min(gpus, cfg.n_kv_heads)
        comm_layer = 2 * batch * cfg.hidden * 4 * (gpus - 1) / gpus * (2 if gpus > 1 else 0)      # two all-reduces of fp32 rows
    else:
        w_layer = (attn + dense) * bw + touched * expert * bw / gpus + router * 2
        kv_layer = local_batch * ctx * kv_tok
        # all-gather of the token rows (bf16) in, fp32 partial rows back to the tokens' home GPUs
        comm_layer = (batch - local_batch) * cfg.hidden * 2 + local_batch * cfg.hidden * 4 * (gpus - 1) if gpus > 1 else 0
    mem_s = n_layers * (w_layer + kv_layer) / (plat.hbm_gbs * 1e9) + head / (1 if mode == "ep" else gpus) / (plat.hbm_gbs * 1e9)
    comm_s = n_layers * comm_layer / (plat.nvlink_gbs * 1e9)
    launch_s = n_layers * plat.kernels_per_layer * plat.launch_us * 1e-6
    step_s = (max(mem_s, comm_s) + launch_s) / derate
    # ---- prefill: FLOPs of one chunk
    tokens = min(prefill_chunk, batch * ctx)
    act = (attn + dense + cfg.n_experts_used * expert + router) * 2.0 * tokens
    attn_flops = 4.0 * tokens * cfg.n_heads * cfg.head_dim * (ctx / 2)
    peak = plat.tensor_tflops * 1e12 * (plat.fp8_speedup if fmt == "mxfp8" else 1.0)
    chunk_s = n_layers * (act / peak + attn_flops / (plat.tensor_tflops * 1e12)) / gpus / derate
    # ---- fit
    w_total = n_layers * ((attn + dense) * bw * (1 if mode == "ep" else 1 / gpus) + cfg.n_experts * expert * bw / gpus) + 2 * head
    kv_total = n_layers * (local_batch if mode == "ep" else batch / min(gpus, cfg.n_kv_heads)) * ctx * kv_tok
    return {
        "decode_ms_per_step": step_s * 1e3, "decode_tokens_per_s": batch / step_s,
        "decode_memory_ms": mem_s * 1e3, "decode_comm_ms": comm_s * 1e3, "decode_launch_ms": launch_s * 1e3,
        "decode_bound": "memory" if mem_s >= comm_s else "communication",
        "experts_touched_per_layer": touched,
        "prefill_tokens_per_s": tokens / chunk_s,
        "weights_gib_per_gpu": w_total / 2 ** 30, "kv_gib_per_gpu": kv_total / 2 ** 30,
        "fits": (w_total + kv_total) / 2 ** 30 < plat.hbm_gib * 0.95,
    }


def context_parallel_decode(cfg: ModelConfig, batch: int, ctx: int, cp: int, plat: Platform = Platform(), hop_us: float = 5.0) -> dict:
    """Cost model of context-parallel decode attention (KV positions sharded block-cyclically over ``cp`` GPUs, every GPU computes
    flash partials on its shard, the partials are merged).  Per layer and step a GPU reads 1/cp of the KV and owns a partial of
    ``n_heads * (head_dim + 1)`` f32 per sequence (O normalised + log-sum-exp; 16 640 bytes for 32 heads of 128 plus the maximum,
    the figure of the reference's ring-attention study).  Two ways to merge: the all-gather by peer stores that
    ``parallel/context.py`` uses (one exchange: a launch-and-flag latency plus (cp-1) partials over the link), and a ring relay of
    the running (m, l, o) state (cp-1 dependent hops, each a latency plus one partial): a64fx/utofu-tests/ring_attn_bench.c,
    summary.md:71-118.  ``hop_us`` is the one-way latency of a peer store becoming visible (flag round included)."""
    partial = batch * cfg.n_heads * (cfg.head_dim + 1) * 4
    kv_layer = batch * ctx * 2 * cfg.n_kv_heads * cfg.head_dim * 2
    link = plat.nvlink_gbs * 1e9
    attn_us = kv_layer / cp / (plat.hbm_gbs * 1e9) * 1e6
    gather_us = hop_us + (cp - 1) * partial / link * 1e6 if cp > 1 else 0.0
    ring_us = (cp - 1) * (hop_us + partial / link * 1e6) if cp > 1 else 0.0
    tree_us = 0.0
    n = 1
    while n < cp:                       # recursive doubling: log2(cp) exchanges of one partial
        tree_us += hop_us + partial / link * 1e6
        n *= 2
    return {"kv_read_us_per_layer": attn_us, "partial_bytes": partial, "merge_allgather_us": gather_us, "merge_ring_us": ring_us,
            "merge_tree_us": tree_us, "kv_gib_per_gpu": cfg.n_layers * kv_layer / cp / 2 ** 30,
            "attention_us_per_layer": attn_us + min(gather_us, ring_us, tree_us) if cp > 1 else attn_us}


def speculative_speedup(accept: float, gamma: int, verify_cost: float) -> dict:
    """Throughput of speculative decoding relative to plain decoding when every draft token is accepted independently with
    probability ``accept``: a verify step over ``1 + gamma`` positions yields ``(1 - accept^(gamma+1)) / (1 - accept)`` tokens in
    expectation and costs ``verify_cost`` decode steps (measured on the Qwen3-30B-A3B shape, 64 x 2048, MXFP8: 1.15, 1.26 and
    1.38 for gamma = 1, 2 and 4).  The drafter's own time is not included (prompt lookup is free; a draft model adds its steps)."""
    tokens = float(gamma + 1) if accept >= 1.0 else (1.0 - accept ** (gamma + 1)) / (1.0 - accept)
    return {"tokens_per_step": tokens, "speedup": tokens / verify_cost, "break_even_tokens_per_step": verify_cost}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="qwen3-30b-a3b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--gpus", default="1", help="comma separated GPU counts")
    ap.add_argument("--format", default="mxfp8", choices=["bf16", "mxfp8"])
    ap.add_argument("--mode", default="ep", choices=["ep", "tp", "tp+ep"])
    ap.add_argument("--derate", type=float, default=1.0)
    ap.add_argument("--hbm-gbs", type=float, default=Platform.hbm_gbs)
    ap.add_argument("--nvlink-gbs", type=float, default=Platform.nvlink_gbs)
    ap.add_argument("--cp", default="", help="comma separated context-parallel degrees: print the long-context decode attention cost model instead")
    ap.add_argument("--spec", default="", metavar="ACCEPT,GAMMA,COST",
                    help="speculative decoding: acceptance probability, draft depth, cost of a verify step in decode steps")
    args = ap.parse_args(argv)
    if args.spec:
        a, g, c = args.spec.split(",")
        print(json.dumps({k: round(v, 3) for k, v in speculative_speedup(float(a), int(g), float(c)).items()}))
        return
    cfg = get_config(args.model)
    plat = Platform(hbm_gbs=args.hbm_gbs, nvlink_gbs=args.nvlink_gbs)
    if args.cp:
        for c in [int(x) for x in args.cp.split(",")]:
            r = context_parallel_decode(cfg, args.batch, args.ctx, c, plat)
            print(json.dumps({"cp": c, **{k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()}}))
        return
    for g in [int(x) for x in args.gpus.split(",")]:
        r = estimate(cfg, args.batch, args.ctx, g, args.format, args.mode, plat, args.derate)
        print(json.dumps({"gpus": g, **{k: (round(v, 3) if isinstance(v, float) else v) for k, v in r.items()}}))


if __name__ == "__main__":
    main()
