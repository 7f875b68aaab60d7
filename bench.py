#!/usr/bin/env python
"""Headline benchmark: Qwen3-30B-A3B-shaped MoE, MXFP8, decode tokens/s (plus prefill tokens/s, TTFT, TPOT).

    python bench.py --gpus N --steps K --warmup W            # N = 1; torchrun launches N > 1
    python bench.py --impl reference ...                      # the reference arm (prints why it is unavailable)

Workload (the MoE expert-parallel benchmark configuration): 48 layers, hidden 2048, 32 Q / 4 KV heads of 128, 128 experts top-8 with
expert FFN 768, vocab 151936; random-init N(0, 0.02) weights quantised to MXFP8 (1x32 E8M0 scales), MXFP8
activations, bf16 outputs; 64 prompts of 2048 uniform-random token ids are prefilled, then decoded greedily.
With N GPUs the 64 sequences are split N ways for attention (data parallel) and the 128 experts N ways
(expert parallel), so the total work is fixed: strong scaling.

A timed *step* is one decode step of the whole 64-sequence batch at context >= 2048: it streams every expert's
weights (~29 GB over the job) and the KV cache (~13 GB) from HBM, far more than the 126 MB L2, so no L2 flush
is needed between steps.  ``value`` = decoded tokens per second over the whole job, timed on the device with
CUDA events, max over ranks.  The ``e2e`` figure drives the same steps through the public ``Engine`` API with
the step's input token ids copied from pinned host memory and the sampled ids read back to the host each step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "baseline"],
                    help="ours = this framework; reference = the unmodified reference code; baseline = plain PyTorch + NCCL (baseline/torch_nccl.py)")
    ap.add_argument("--model", default="qwen3-30b-a3b")
    ap.add_argument("--fmt", default="mxfp8", choices=["mxfp8", "bf16", "q4_k", "q8_0"],
                    help="weight format; q4_k / q8_0 keep ggml blocks in HBM (fused dequant-GEMV / GEMM)")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=0, help="debug only: run fewer layers (the JSON line then says so and is not a valid bench number)")
    ap.add_argument("--kv", default="bf16", choices=["bf16", "int8"], help="KV cache pages: bf16, or int8 + scales read directly by the decode "
                    "attention kernel (a reduced-precision mode: the JSON line is then marked as not the headline configuration)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--baseline-eager", action="store_true", help="--impl baseline: run the decode step without a CUDA graph")
    ap.add_argument("--parallel", default="auto", choices=["auto", "ep", "tp", "tp+ep"],
                    help="multi-GPU layout: ep = experts sharded, attention data-parallel (MoE models); tp = every projection sharded, "
                         "batch replicated (dense models); tp+ep = attention sharded by heads and experts spread over the same ranks, "
                         "batch replicated (the layout of the largest MoE models, e.g. --model qwen3-235b-a22b); auto picks by model")
    ap.add_argument("--moe-path", default="fused", choices=["fused", "nccl"], help="multi-GPU expert exchange: fused peer-memory kernels or the NCCL baseline")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks, power and throttle reasons of one GPU while the timed region runs (read-only NVML queries from a
    thread, every 50 ms; ``nvidia-smi -lms`` as the fallback when the NVML binding is missing)."""
    FIELDS = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index: int, uuid: str = ""):
        self.gpu, self.uuid = gpu_index, uuid
        self.proc = None
        self.lines = []
        self.samples = []          # (sm_mhz, max_mhz, power_w, set(reasons))
        self.stop_flag = False
        self.thread = None
        self.mode = None
        self.t_mark = None         # set by mark(): the timed region starts here
        self.max_query_ms = 0.0

    def _nvml_loop(self, nv, h):
        bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
        while not self.stop_flag:
            t_q = time.perf_counter()
            try:
                sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                pw = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                if self.t_mark is not None:          # queries before mark() only warm the NVML paths up
                    self.samples.append((float(sm), float(mx), pw, {n for n, b in bits.items() if r & b}))
            except Exception:
                pass
            self.max_query_ms = max(self.max_query_ms, (time.perf_counter() - t_q) * 1e3)     # slowest round of queries (diagnostic)
            time.sleep(0.05)

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByUUID(self.uuid) if self.uuid else nv.nvmlDeviceGetHandleByIndex(self.gpu)
            self.mode = "nvml"
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, h), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.mode = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.gpu)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.mode = "smi"
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def mark(self):
        """The timed region starts now; everything sampled before (first-call costs of the NVML queries included) is dropped."""
        self.t_mark = time.perf_counter()
        self.lines = []

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.mode is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML binding and no nvidia-smi"], "samples": 0}
        if self.mode == "nvml":
            self.stop_flag = True
            self.thread.join(timeout=1)
        else:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass
            for ln in self.lines:
                parts = [p.strip() for p in ln.split(",")]
                if len(parts) < 8:
                    continue
                try:
                    self.samples.append((float(parts[1]), float(parts[2]), float(parts[3]),
                                         {nm for nm, v in zip(self.NAMES, parts[4:8]) if v.lower().startswith("active")}))
                except ValueError:
                    continue
        sm = [x[0] for x in self.samples]
        power = [x[2] for x in self.samples]
        reasons = set().union(*[x[3] for x in self.samples]) if self.samples else set()
        busy = [c for c, p in zip(sm, power) if p > 300] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(x[1] for x in self.samples) if self.samples else None,
                "reasons": sorted(reasons), "samples": len(sm), "power_w_max": max(power) if power else None, "source": self.mode,
                "max_query_ms": round(self.max_query_ms, 1)}


def reference_arm(args):
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a C source tree without setup.py/pyproject.toml (pip: 'not installable'); its CUDA runner is "
                      "single-GPU, batch 1 and does not load the qwen3moe architecture, so this metric/config has no reference code path"}))
    return 0


def baseline_table():
    """Measured decode tokens/s of the plain PyTorch + NCCL baseline (``bench.py --impl baseline``), keyed by
    ``model|batch|prompt_len|n_gpus``; the file is written from runs on the same kind of box and sits beside the baseline code."""
    try:
        with open(os.path.join(ROOT, "baseline", "measured.json")) as f:
            return json.load(f)
    except Exception:
        return {}


def baseline_arm(args):
    """The same metric and config through baseline/torch_nccl.py: torch.matmul / bmm, SDPA, NCCL collectives, a CUDA graph for
    the decode step.  bf16 weights (PyTorch has no block-scaled fp8 grouped GEMM to call)."""
    import torch
    import torch.distributed as dist
    from baseline.torch_nccl import BaselineModel
    from gemm_b200.models.config import get_config
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    cfg = get_config(args.model)
    layout = "single"
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        layout = args.parallel if args.parallel != "auto" else ("ep" if cfg.n_experts > 0 else "tp")
        layout = "ep" if layout == "tp+ep" else layout             # the baseline has no hybrid layout: experts sharded, attention data-parallel
    n_layers = args.layers if args.layers > 0 else cfg.n_layers
    tp = layout == "tp"
    b_local = args.batch if (tp or world == 1) else args.batch // world
    model = BaselineModel(cfg, device, seed=0, n_layers=n_layers, group=dist.group.WORLD if world > 1 else None, layout=layout)
    total_new = args.warmup + 2 * args.steps + 8             # device-timed steps + the end-to-end steps + slack
    model.alloc_kv(b_local, args.prompt_len + total_new)
    g = torch.Generator().manual_seed(0)
    all_prompts = torch.randint(0, cfg.vocab, (args.batch, args.prompt_len), generator=g, dtype=torch.int32)
    prompts = all_prompts[(0 if (tp or world == 1) else rank * b_local): (0 if (tp or world == 1) else rank * b_local) + b_local]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def note(msg):
        if rank == 0:
            print(f"[bench baseline] {msg}", file=sys.stderr, flush=True)

    note("weights built")
    model.prefill(prompts[:1, :256])                      # lazy initialisation outside the timed region
    barrier()
    note("first prefill done")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    first = model.prefill(prompts).argmax(-1)
    e1.record()
    barrier()
    prefill_ms = max_over_ranks(e0.elapsed_time(e1))
    note(f"prefill {prefill_ms:.0f} ms")
    model.begin_decode(first, use_graph=not args.baseline_eager)
    note("decode graph captured" if not args.baseline_eager else "decode runs eagerly")
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        model.decode_step()
    barrier()
    sampler.mark()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        model.decode_step()
    b.record()
    barrier()
    total_ms = max_over_ranks(a.elapsed_time(b))
    clocks = sampler.stop()
    # end to end: the step's ids come from pinned host memory, the result goes back to the host
    ids_host = torch.empty(b_local, dtype=model._ids.dtype).pin_memory()
    out_host = torch.empty(b_local, dtype=model._ids.dtype).pin_memory()
    ids_host.copy_(model._ids.cpu())
    barrier()
    w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0.record()
    for _ in range(args.steps):
        model._ids.copy_(ids_host, non_blocking=True)
        out_host.copy_(model.decode_step(), non_blocking=True)
        torch.cuda.synchronize()
        ids_host.copy_(out_host)
    w1.record()
    barrier()
    e2e_ms = max_over_ranks(w0.elapsed_time(w1))
    if rank == 0:
        esz = ids_host.element_size()
        line = {"impl": "baseline", "metric": "decode_tokens_per_s", "value": args.batch * args.steps / (total_ms / 1e3), "unit": "tokens/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "bf16 (torch.matmul / bmm, SDPA, NCCL)",
                "data": "synthetic (uniform random token ids, random-init N(0,0.02) weights)",
                "config": {"model": args.model, "global_batch": args.batch, "seq_len": args.prompt_len, "parallelism": f"{layout}{world}" if world > 1 else "single",
                           "layers": n_layers, "l2": "no flush: every step streams all weights and the KV cache, far more than the 126 MB L2"},
                "prefill_tokens_per_s": args.batch * args.prompt_len / (prefill_ms / 1e3), "ttft_ms_whole_batch": prefill_ms, "clocks": clocks,
                "e2e": {"value": args.batch * args.steps / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": b_local * esz * world,
                        "d2h_bytes_per_step": b_local * esz * world, "ms_per_step": e2e_ms / args.steps},
                "gpu_launches": 0}
        if n_layers != cfg.n_layers:
            line["invalid"] = f"debug run with {n_layers} of {cfg.n_layers} layers"
        print(json.dumps(line))
    if world > 1:
        # The decode graph holds captured NCCL work: tearing the process group down under it did not return (the ranks sat in
        # destroy_process_group until the launcher's limit).  Drop the graph, meet once more, and leave without the teardown.
        torch.cuda.synchronize()
        model._graph = None
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.impl == "baseline":
        return baseline_arm(args)

    import torch
    import torch.distributed as dist
    from gemm_b200 import _native
    from gemm_b200.models.config import get_config
    from gemm_b200.models.weights import synthetic_weights
    from gemm_b200.serve.engine import Engine, SamplingParams

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    par = None
    cfg0 = get_config(args.model)
    layout = args.parallel if args.parallel != "auto" else ("ep" if cfg0.n_experts > 0 else "tp")
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        if layout == "ep":
            from gemm_b200.parallel.expert import ExpertParallel
            par = ExpertParallel(dist.group.WORLD, device, fused=(args.moe_path == "fused"))
        else:
            from gemm_b200.parallel.tensor import TensorParallel
            par = TensorParallel(dist.group.WORLD, device, fused=(args.moe_path == "fused"), ep_experts=(layout == "tp+ep"))
    if args.gpus != world and rank == 0:
        print(f"[bench] note: --gpus {args.gpus} but WORLD_SIZE {world}; using {world}", file=sys.stderr)
    n_gpus = world

    cfg = get_config(args.model)
    n_layers = args.layers if args.layers > 0 else cfg.n_layers
    tp = layout in ("tp", "tp+ep") and n_gpus > 1
    hybrid = layout == "tp+ep" and n_gpus > 1
    assert tp or args.batch % n_gpus == 0
    b_local = args.batch if tp else args.batch // n_gpus          # tensor parallelism replicates the batch on every rank
    t0 = time.time()
    if tp:
        weights = synthetic_weights(cfg, args.fmt, device=device, seed=0, tp_rank=rank, tp_size=n_gpus, n_layers=n_layers,
                                    ep_rank=rank if hybrid else 0, ep_size=n_gpus if hybrid else 1)
    else:
        weights = synthetic_weights(cfg, args.fmt, device=device, seed=0, ep_rank=rank, ep_size=n_gpus, n_layers=n_layers)
    torch.cuda.synchronize()
    if rank == 0:
        print(f"[bench] weights {weights.nbytes() / 2**30:.1f} GiB on rank 0 in {time.time() - t0:.1f}s", file=sys.stderr)
    total_new = args.warmup + args.steps * (2 if args.no_e2e else 3) + 16        # room for one re-measured timed region
    max_len = args.prompt_len + total_new + 8
    pages_per_seq = (max_len + 127) // 128
    # one spare page per sequence at N > 1: the fused-vs-NCCL check below writes its scratch tokens there
    engine = Engine(weights, max_batch=b_local, max_seq_len=max_len, page_size=128, par=par, max_prefill_tokens=16384,
                    num_pages=b_local * pages_per_seq + (b_local if n_gpus > 1 else 0), kv_dtype=args.kv)
    if par is not None:
        par.attach(engine, cfg, max_tokens=16384)

    # synthetic prompts: uniform token ids from seed 0 (the same global batch whatever N is)
    g = torch.Generator().manual_seed(0)
    all_prompts = torch.randint(0, cfg.vocab, (args.batch, args.prompt_len), generator=g, dtype=torch.int32)
    prompts = [all_prompts[(0 if tp else rank * b_local) + i] for i in range(b_local)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---------------------------------------------------------------- prefill (TTFT, prefill tok/s)
    # warm-up pass on a short prompt so that lazy initialisation is not timed
    engine.prefill([prompts[0][:256]])
    engine.reset()
    engine.prefill(prompts[: min(8, b_local)])        # one full-size chunk: the prefill-sized kernel variants are loaded too
    engine.reset()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    logits = engine.prefill(prompts, reserve=total_new)
    first = engine._sample(logits, SamplingParams(), 0)
    e1.record()
    barrier()
    prefill_ms = max_over_ranks(e0.elapsed_time(e1))
    prefill_tok_s = args.batch * args.prompt_len / (prefill_ms / 1e3)

    # ---------------------------------------------------------------- decode (device-timed steps)
    engine.begin_decode(first, SamplingParams(), max_new_tokens=total_new, use_graph=True)
    launches_before = _native.launch_count()
    engine._decode_body_count = None
    # The clock sampler starts BEFORE the warm-up steps: the first NVML queries of a process can take seconds and were seen to
    # stall the GPU's work submission for about 2 s once per process; they now land in the warm-up, not in the timed region.
    try:
        _uuid = "GPU-" + str(torch.cuda.get_device_properties(local_rank).uuid)
    except Exception:
        _uuid = ""
    sampler = ClockSampler(local_rank, _uuid)
    sampler.start()
    time.sleep(0.3)
    for _ in range(args.warmup):
        engine.decode_step()
    barrier()
    sampler.mark()
    _native.read_status()                     # clear: the status below belongs to the timed region only

    def timed_region():
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        evs[0].record()
        t_host0 = time.perf_counter()
        for i in range(args.steps):
            engine.decode_step()
            evs[i + 1].record()
        host_ms = (time.perf_counter() - t_host0) * 1e3 / args.steps      # host time to enqueue one step (diagnostic)
        barrier()
        tot = max_over_ranks(evs[0].elapsed_time(evs[-1]))
        return tot, [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)], host_ms, _native.read_status()

    total_ms, per_step, host_enqueue_ms, st = timed_region()
    rejected = None
    # A kernel whose bounded wait gave up (status != ok) on any rank returned without doing its work: that region measures nothing
    # valid.  It is reported and the K steps are timed once more.
    bad = max_over_ranks(float(st["code"] != 0))
    if bad > 0:
        rejected = {"ms_per_step": total_ms / args.steps, "kernel_status_detail": {k: (list(v) if isinstance(v, tuple) else v) for k, v in st.items()}}
        total_ms, per_step, host_enqueue_ms, st = timed_region()
    clocks = sampler.stop()
    tpot_p50 = max_over_ranks(statistics.median(per_step))
    decode_tok_s = args.batch * args.steps / (total_ms / 1e3)
    kernels_per_step = engine.kernels_per_step

    # ---------------------------------------------------------------- end to end through the public API
    e2e = None
    if not args.no_e2e:
        ids_host = torch.empty(b_local, dtype=torch.int32).pin_memory()
        out_host = torch.empty(b_local, dtype=torch.int32).pin_memory()
        ids_host.copy_(engine._static["tokens"].cpu())
        for _ in range(3):
            engine.set_next_tokens(ids_host); out_host.copy_(engine.decode_step(), non_blocking=True); torch.cuda.synchronize(); ids_host.copy_(out_host)
        barrier()
        w0 = torch.cuda.Event(enable_timing=True); w1 = torch.cuda.Event(enable_timing=True)
        w0.record()
        for _ in range(args.steps):
            engine.set_next_tokens(ids_host)                       # H2D: this step's input ids from pinned memory
            toks = engine.decode_step()
            out_host.copy_(toks, non_blocking=True)                # D2H: the step's result
            torch.cuda.synchronize()
            ids_host.copy_(out_host)                               # the host owns the token stream
        w1.record()
        barrier()
        e2e_ms = max_over_ranks(w0.elapsed_time(w1))
        e2e = {"value": args.batch * args.steps / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": b_local * 4 * n_gpus,
               "d2h_bytes_per_step": b_local * 4 * n_gpus, "ms_per_step": e2e_ms / args.steps}

    # ---------------------------------------------------------------- multi-GPU correctness: fused peer-memory path against the NCCL path
    check = None
    if world > 1 and par is not None and len(engine.pages.free) >= b_local:
        from gemm_b200.models.transformer import ForwardBatch
        n_tok = 4
        scratch = engine.pages.alloc(b_local)                          # one fresh page per sequence, given back below
        bt = torch.tensor([[p] for p in scratch], dtype=torch.int32)
        gchk = torch.Generator().manual_seed(1234 + (0 if tp else rank))
        ids = torch.randint(0, cfg.vocab, (b_local * n_tok,), generator=gchk, dtype=torch.int32)
        fbc = ForwardBatch.build([n_tok] * b_local, [0] * b_local, ids, bt, engine.page_size, engine.hq_local, engine.hkv_local, device,
                                 stage=engine.kv.quantized)
        outs = []
        outs, hid1 = [], []
        for fused_flag in (True, False):                               # same weights, same state, the two exchange implementations
            par.fused = fused_flag and (args.moe_path == "fused")
            x1 = engine.model.forward_hidden(fbc, 0, 1)                # the residual stream after one layer (one attention + one FFN / MoE block)
            hid1.append(x1.float() + engine.model._last_delta.float())
            outs.append(engine.model.forward(fbc).float())
        par.fused = args.moe_path == "fused"
        torch.cuda.synchronize()
        engine.pages.release(scratch)
        rel_of = lambda a, b: ((a - b).norm() / (b.norm() + 1e-12)).item()
        same = float((outs[0].argmax(-1) == outs[1].argmax(-1)).float().mean().item())
        st_chk = _native.read_status()
        check = {"tokens_equal": bool(-max_over_ranks(-same) >= 1.0), "token_agreement_min": -max_over_ranks(-same),
                 "rel_l2_after_layer_1_max": max_over_ranks(rel_of(hid1[0], hid1[1])), "rel_l2_logits_max": max_over_ranks(rel_of(outs[0], outs[1])),
                 "kernel_status": st_chk["what"],
                 "compared": "fused peer-memory exchange vs torch.distributed (NCCL) exchange on the same weights and cache: one forward of "
                             f"{n_tok} fresh tokens per sequence on every rank.  The two paths round the partial sums differently (fp32 slots vs "
                             "bf16 rows); with random-init routers near-tied experts swap under that rounding, which is what moves the "
                             "logits of the deep model while one layer agrees closely"}

    if rank == 0:
        # the comparison number: the plain PyTorch + NCCL implementation of the same config on the same number of GPUs
        base_val = baseline_table().get(f"{args.model}|{args.batch}|{args.prompt_len}|{n_gpus}")
        vs_base = (decode_tok_s / base_val) if (base_val and n_layers == cfg.n_layers) else None
        line = {
            "metric": "decode_tokens_per_s", "value": decode_tok_s, "unit": "tokens/s", "n_gpus": n_gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": vs_base, "baseline_tokens_per_s": base_val, "dtype": {"mxfp8": "mxfp8 weights+activations, bf16 outputs, fp32 accumulate", "bf16": "bf16",
                                          "q4_k": "ggml Q4_K weights (kept quantised), bf16 activations / int8 in the GEMV, fp32 accumulate",
                                          "q8_0": "ggml Q8_0 weights (kept quantised), bf16 activations / int8 in the GEMV, fp32 accumulate"}[args.fmt],
            "data": "synthetic (uniform random token ids, random-init N(0,0.02) weights)",
            "config": {"model": args.model, "global_batch": args.batch, "seq_len": args.prompt_len, "decode_context": args.prompt_len + args.warmup,
                       "parallelism": (f"tp{n_gpus}-attention+ep{n_gpus}" if hybrid else f"tp{n_gpus}" if tp else f"dp{n_gpus}-attention+ep{n_gpus}") if n_gpus > 1 else "single", "layers": n_layers,
                       "l2": f"no flush: each step streams the {weights.nbytes() / 2**30:.1f} GiB of weights of a rank plus its KV cache, far more than the 126 MB L2",
                       "moe_path": args.moe_path if n_gpus > 1 else "local"},
            "prefill_tokens_per_s": prefill_tok_s, "ttft_ms_whole_batch": prefill_ms, "tpot_ms_p50": tpot_p50,
            "clocks": clocks, "e2e": e2e, "check": check, "gpu_launches": kernels_per_step * args.steps,
            "kernels_per_step": kernels_per_step, "kernel_status": st["what"], "kernel_status_detail": {k: (list(v) if isinstance(v, tuple) else v) for k, v in st.items()},
            "rejected_region": rejected, "host_enqueue_ms_per_step": round(host_enqueue_ms, 3),
            "step_ms_min_max": [round(min(per_step), 3), round(max(per_step), 3)], "native_libs": _native.loaded_libraries(),
        }
        if n_layers != cfg.n_layers:
            line["invalid"] = f"debug run with {n_layers} of {cfg.n_layers} layers"
        if args.kv != "bf16":
            line["invalid"] = (line.get("invalid", "") + "; " if line.get("invalid") else "") + f"KV cache kept as {args.kv}: reduced precision, not the headline configuration"
            line["config"]["kv_cache"] = args.kv
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        if par is not None:
            par.close()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
