"""Kernel micro-benchmarks: ``python -m gemm_b200.utils.microbench --case <name> [--iters N]``.

Every case times one op of the library on shapes of the Qwen3-30B-A3B benchmark configuration with CUDA events on the
launching stream, after warm-up, with the L2 flushed (a 256 MiB buffer is rewritten) before every timed launch, and
prints one JSON line per measurement: achieved TFLOP/s and GB/s of the bytes that must come from HBM.  ``--once`` runs
each op a single time without timing (the form to put under a profiler).

Cases
  gemm         dense projections: decode (64 tokens) and prefill (16384 tokens), bf16 and MXFP8
  moe_decode   grouped expert GEMMs (gate/up with SwiGLU + re-quantisation, down) for 64 tokens x top-8 of 128 experts, as two
               launches and as the one persistent launch
  moe_prefill  the same for 16384 tokens
  attn_decode  paged flash-decode, 64 sequences x 2048 cached tokens, 32 query / 4 KV heads
  attn_prefill causal prefill, 8 sequences x 2048 tokens
  lm_head      64 x 151936 x 2048 with the arg-max epilogue
  quant        ggml-quantised projections of the Qwen3-32B shape (Q4_K and Q8_0 blocks kept in HBM): fused dequant-GEMV for
               1 and 4 tokens, fused dequant-GEMM for 8, 64 and 4096 tokens
  small        the kernels around them: RMSNorm + residual + MXFP8 copy, QK-norm + RoPE + cache write (64 and 16384 tokens), the
               one-launch MoE front end, sampler and arg-max over 64 x 151936 logits, the Delta-Net recurrence (decode, prefill)
  spec_verify  whole-model step over 1, 2, 3 and 5 positions per sequence (speculative verification against plain decode);
               builds the full Qwen3-30B-A3B shape, not part of ``all``

Counterpart in the reference: cuda/gemm/bench_log.md and cuda/fa2/bench_log.md are produced by stand-alone bench
programs of the same kind.
"""
from __future__ import annotations

import argparse
import json

import torch

from .. import _native
from ..ops import attention as att
from ..ops import elementwise as ew
from ..ops import gemm, moe, mxfp8

_flush = None


def _timeit(fn, iters: int, warm: int = 3) -> float:
    """Median milliseconds of ``fn`` (L2 flushed before each timed call)."""
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(iters):
        _flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def _emit(name: str, ms: float, flops: float, hbm_bytes: float, **kw) -> None:
    print(json.dumps(dict(case=name, ms=round(ms, 5), tflops=round(flops / ms / 1e9, 1), hbm_gbs=round(hbm_bytes / ms / 1e6, 1), **kw)),
          flush=True)


def _run(name, fn, flops, hbm_bytes, args, **kw):
    if args.once:
        fn()
        torch.cuda.synchronize()
        print(json.dumps(dict(case=name, ran="once")), flush=True)
        return
    _emit(name, _timeit(fn, args.iters), flops, hbm_bytes, **kw)


def case_gemm(args):
    for (m, n, k) in [(64, 5120, 2048), (64, 2048, 4096), (16384, 5120, 2048), (16384, 2048, 4096), (8192, 8192, 8192)]:
        x = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
        w = (torch.randn(n, k, device="cuda") * 0.05).bfloat16()
        wt = mxfp8.tile_weight(w)
        _run(f"gemm_bf16_{m}x{n}x{k}", lambda: gemm.linear(x, wt, w_tiled=True), 2.0 * m * n * k, n * k * 2 + m * k * 2 + m * n * 2, args)
        if not args.once:
            _emit(f"torch_matmul_{m}x{n}x{k}", _timeit(lambda: torch.matmul(x, w.t()), args.iters), 2.0 * m * n * k, n * k * 2 + m * k * 2 + m * n * 2)
        xq = mxfp8.quantize(x.float(), sf_layout=32 if m <= 32 else 128)
        wq = mxfp8.quantize(w.float())
        wq = mxfp8.MxTensor(mxfp8.tile_weight(wq.data), wq.sf, wq.rows, wq.k, 128, tiled=True)
        _run(f"gemm_mxfp8_{m}x{n}x{k}", lambda: gemm.linear_mx(xq, wq), 2.0 * m * n * k, n * k + m * k + m * n * 2, args)


def _moe(args, t: int, name: str):
    e, kk, h, inter = 128, 8, 2048, 768
    tn = 32 if (t * kk) // e <= 24 else 128
    ids, _ = moe.route(torch.randn(t, e, device="cuda"), kk)
    pl = moe.plan(ids, e, tn)
    x = torch.randn(t, h, device="cuda").bfloat16()
    xq = ew.mx_quantize(x, pl.row_token, sf_layout=tn)
    w1 = mxfp8.quantize(torch.randn(e * 2 * inter, h, device="cuda") * 0.05)
    w2 = mxfp8.quantize(torch.randn(e * h, inter, device="cuda") * 0.05)
    d1, d2 = mxfp8.tile_weight(w1.data), mxfp8.tile_weight(w2.data)
    hq = torch.empty(pl.capacity, inter, dtype=torch.uint8, device="cuda")
    hsf = ew.sf_alloc(pl.capacity, inter, "cuda", tn, init=False)

    gu = torch.empty(pl.capacity, 2 * inter, dtype=torch.bfloat16, device="cuda") if tn == 128 else None

    def gate_up():
        if tn == 32:        # decode: SiLU(gate) * up and the re-quantisation run in the GEMM epilogue
            gemm.grouped_linear(xq.data, d1.view(e, 2 * inter, h), pl.seg_start, pl.seg_count, tn, out=hq, dual=True, sfa=w1.sf, sfb=xq.sf,
                                quant_out=True, out_sf=hsf, w_tiled=True)
        else:               # prefill: plain GEMM over the stacked rows (256-token tiles) + one fused activation / quantise pass
            gemm.grouped_linear(xq.data, d1.view(e, 2 * inter, h), pl.seg_start, pl.seg_count, tn, out=gu, sfa=w1.sf, sfb=xq.sf, w_tiled=True)
            ew.silu_mul_quant(gu, hq, hsf, pl.row_token, sf_layout=tn)

    def down():
        gemm.grouped_linear(hq, d2.view(e, h, inter), pl.seg_start, pl.seg_count, tn, sfa=w2.sf, sfb=hsf, w_tiled=True, pair_rows=(tn == 32))

    gate_up()
    touched = int((pl.seg_count > 0).sum())
    fl = 2.0 * t * kk * h * inter
    _run(f"{name}_gate_up", gate_up, 2 * fl, touched * 2 * h * inter + t * kk * h, args, tn=tn, experts_touched=touched)
    _run(f"{name}_down", down, fl, touched * h * inter + t * kk * inter + t * kk * h * 2, args, tn=tn, experts_touched=touched)
    if tn == 32:
        # the same two projections as one persistent launch
        from ..models.weights import LinearWeight
        lw1 = LinearWeight("mxfp8", 2 * inter, h, mx=mxfp8.MxTensor(d1, w1.sf, e * 2 * inter, h, 128, tiled=True), groups=e, rows_per_group=2 * inter)
        lw2 = LinearWeight("mxfp8", h, inter, mx=mxfp8.MxTensor(d2, w2.sf, e * h, inter, 128, tiled=True), groups=e, rows_per_group=h)
        if moe.can_fuse_ffn(xq, lw1, lw2, e, pl.capacity):
            _run(f"{name}_ffn_fused", lambda: moe.expert_ffn_fused(xq, lw1, lw2, e, pl), 3 * fl,
                 touched * 3 * h * inter + t * kk * h + t * kk * h * 2, args, tn=tn, experts_touched=touched)


def case_moe_decode(args):
    _moe(args, 64, "moe_decode")
    # what ONE rank of an 8-way expert-parallel group runs per layer: all 64 gathered tokens against its 16 local experts
    from ..models.weights import LinearWeight
    e_all, e_loc, kk, h, inter = 128, 16, 8, 2048, 768
    x = torch.randn(64, h, device="cuda").bfloat16()
    router = (torch.randn(e_all, h, device="cuda") * 0.05).bfloat16()
    w1 = mxfp8.quantize(torch.randn(e_loc * 2 * inter, h, device="cuda") * 0.05)
    w2 = mxfp8.quantize(torch.randn(e_loc * h, inter, device="cuda") * 0.05)
    lw1 = LinearWeight("mxfp8", 2 * inter, h, mx=mxfp8.MxTensor(mxfp8.tile_weight(w1.data), w1.sf, e_loc * 2 * inter, h, 128, tiled=True),
                       groups=e_loc, rows_per_group=2 * inter)
    lw2 = LinearWeight("mxfp8", h, inter, mx=mxfp8.MxTensor(mxfp8.tile_weight(w2.data), w2.sf, e_loc * h, inter, 128, tiled=True),
                       groups=e_loc, rows_per_group=h)
    if moe.can_prep(x, router, kk):
        ids, wts, pl, xq = moe.prep_hidden(x, router, kk, e_loc, 32, local_range=(32, e_loc))
        touched = int((pl.seg_count > 0).sum())
        pairs = int(pl.seg_count.sum())
        _run("moe_prep_ep8_rank", lambda: moe.prep_hidden(x, router, kk, e_loc, 32, local_range=(32, e_loc)), 0.0, e_all * h * 2 + 64 * h * 2, args,
             local_pairs=pairs)
        if moe.can_fuse_ffn(xq, lw1, lw2, e_loc, pl.capacity):
            _run("moe_ffn_fused_ep8_rank", lambda: moe.expert_ffn_fused(xq, lw1, lw2, e_loc, pl), 6.0 * pairs * h * inter,
                 touched * 3 * h * inter + pairs * h * 3, args, experts_touched=touched, local_pairs=pairs)


def case_moe_prefill(args):
    _moe(args, 16384, "moe_prefill")


def _attn(args, b: int, q_len: int, ctx: int, name: str):
    hq, hkv, d, page = args.hq, args.hkv, 128, args.page
    b = args.batch if args.batch > 0 else b
    ctx = args.ctx if args.ctx >= 0 else ctx
    pages_per = (ctx + q_len + page - 1) // page
    n_pages = b * pages_per + 1
    k = (torch.randn(n_pages * page, hkv, d, device="cuda") * 0.5).bfloat16()
    v = (torch.randn(n_pages * page, hkv, d, device="cuda") * 0.5).bfloat16()
    bt = (torch.arange(b * pages_per, device="cuda", dtype=torch.int32) + 1).reshape(b, pages_per)
    q = (torch.randn(b * q_len, hq, d, device="cuda") * 0.5 * ew.softmax_scale_log2(d)).bfloat16()
    q_lens = [q_len] * b
    cu = torch.tensor([i * q_len for i in range(b + 1)], device="cuda", dtype=torch.int32)
    kv_len = torch.full((b,), ctx + q_len, device="cuda", dtype=torch.int32)
    splits = att.pick_splits(b, hkv, ctx + q_len) if q_len == 1 else 1
    if args.splits > 0:
        splits = args.splits
    work = att.build_work(q_lens, hq, hkv, splits).to("cuda")

    def run():
        att.attention(q, k, v, cu, kv_len, bt, page, work, num_splits=splits, causal=True, decode=(q_len == 1))

    kv_bytes = b * (ctx + q_len) * hkv * d * 2 * 2
    if q_len == 1:
        flops = 4.0 * b * hq * (ctx + 1) * d
    else:
        flops = 4.0 * b * hq * d * (q_len * ctx + q_len * (q_len + 1) / 2)
    _run(name, run, flops, kv_bytes + b * q_len * hq * d * 4, args, splits=splits, batch=b, ctx=ctx, hq=hq, hkv=hkv, page=page)
    if q_len == 1:
        # the same pages as int8 + one scale per slot and head, read directly by the INT8 decode attention kernel
        kq, vq = torch.empty(k.shape, dtype=torch.int8, device="cuda"), torch.empty(v.shape, dtype=torch.int8, device="cuda")
        ks, vs = torch.empty(k.shape[:2], device="cuda"), torch.empty(v.shape[:2], device="cuda")
        att.kv_store_q8(k, v, None, torch.arange(k.shape[0], dtype=torch.int32, device="cuda"), kq, vq, ks, vs)
        sp8 = args.splits if args.splits > 0 else max(1, min(8, (148 * 4) // max(1, b * hkv)))
        _run(name + "_int8_kv", lambda: att.attention_decode_q8(q, kq, vq, ks, vs, kv_len, bt, page, num_splits=sp8), flops,
             kv_bytes // 2 + b * (ctx + 1) * hkv * 8 + b * hq * d * 4, args, splits=sp8, batch=b, ctx=ctx, hq=hq, hkv=hkv, page=page)


def case_attn_decode(args):
    _attn(args, 64, 1, 2048, "attn_decode")


def case_attn_prefill(args):
    _attn(args, 8, 2048, 0, "attn_prefill")


def case_lm_head(args):
    m, n, k = 64, 151936, 2048
    x = (torch.randn(m, k, device="cuda") * 0.5).bfloat16()
    w = mxfp8.tile_weight((torch.randn(n, k, device="cuda") * 0.05).bfloat16())
    _run("lm_head_argmax", lambda: gemm.linear_argmax(x, w, w_tiled=True), 2.0 * m * n * k, n * k * 2, args)


def case_spec_verify(args):
    """Cost of a speculative-decoding verify step (1 + gamma query positions per sequence through the chunked-prefill path)
    against a plain decode step, on the benchmark model: 64 sequences x 2048 cached tokens, MXFP8."""
    from ..models.config import get_config
    from ..models.transformer import ForwardBatch
    from ..models.weights import synthetic_weights
    from ..serve.engine import Engine
    name, b, ctx = "qwen3-30b-a3b", (args.batch or 64), (args.ctx if args.ctx >= 0 else 2048)
    cfg = get_config(name)
    dev = torch.device("cuda", torch.cuda.current_device())
    w = synthetic_weights(cfg, "mxfp8", device=dev, seed=0)
    eng = Engine(w, max_batch=b, max_seq_len=ctx + 16, page_size=128, max_prefill_tokens=16384)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab, (b, ctx), generator=g, dtype=torch.int32)
    eng.prefill([prompts[i] for i in range(b)], reserve=8)
    bt = eng._block_table(range(b))
    variants = {}
    for q in (1, 2, 3, 5):
        ids = torch.randint(0, cfg.vocab, (b * q,), generator=g, dtype=torch.int32)
        splits = att.pick_splits(b, eng.hkv_local, ctx + 8) if q == 1 else 1
        variants[q] = ForwardBatch.build([q] * b, [ctx] * b, ids, bt, 128, eng.hq_local, eng.hkv_local, dev, num_splits=splits, all_logits=True)

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(max(3, args.iters // 2)):
            a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(e))
        ts.sort()
        return ts[len(ts) // 2]

    with torch.no_grad():
        base = None
        for q, fb in variants.items():
            ms = timed(lambda: eng.model.forward_greedy(fb))
            base = base or ms
            print(json.dumps(dict(case="spec_verify_eager", positions_per_seq=q, tokens=b * q, ms=round(ms, 3), vs_one=round(ms / base, 3))), flush=True)
        base = None
        for q, fb in variants.items():             # the same steps replayed from a CUDA graph (no host time between launches)
            try:
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    eng.model.forward_greedy(fb)
                ms = timed(gr.replay)
            except Exception as exc:               # a host read inside the step cannot be captured: the eager figure stands
                print(json.dumps(dict(case="spec_verify_graph", positions_per_seq=q, error=str(exc)[:120])), flush=True)
                break
            base = base or ms
            print(json.dumps(dict(case="spec_verify_graph", positions_per_seq=q, tokens=b * q, ms=round(ms, 3), vs_one=round(ms / base, 3))), flush=True)


def case_quant(args):
    from ..ops import ggml_torch as gt
    from ..ops import qlinear
    shapes = [("qkv", 10240, 5120), ("gate_up", 51200, 5120), ("down", 5120, 25600)]
    if args.once:
        shapes = shapes[1:2]
    for tname, t in (("q4_k", gt.Q4_K), ("q8_0", gt.Q8_0)):
        blk, nb = gt.BLOCK[t]
        for (pname, n, k) in shapes:
            w = qlinear.QTensor.from_float(torch.randn(n, k, device="cuda") * 0.02, t)
            wbytes = n * (k // blk) * nb
            for m in ((1,) if args.once else (1, 4)):
                x = torch.randn(m, k, device="cuda").bfloat16()
                sp = qlinear.pick_splits(n, k, m, t)
                out = torch.empty(sp, m, n, dtype=torch.float32, device="cuda")
                _run(f"qgemv_{tname}_{pname}_{m}x{n}x{k}", lambda: qlinear.gemv_partials(x, w, splits=sp, out=out), 2.0 * m * n * k, wbytes, args, splits=sp)
            for m in ((64,) if args.once else (8, 64, 4096)):
                if m == 4096 and pname != "qkv":
                    continue
                x = torch.randn(m, k, device="cuda").bfloat16()
                out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
                sp = qlinear.pick_gemm_splits(n, k, m)
                if sp > 1:      # few row tiles: K is cut and the consumer adds the slabs (here: a sum, which the model folds into its next kernel)
                    _run(f"qgemm_{tname}_{pname}_{m}x{n}x{k}", lambda: qlinear.gemm_partials(x, w, sp), 2.0 * m * n * k,
                         wbytes + m * k * 2 + sp * m * n * 4, args, splits=sp)
                else:
                    _run(f"qgemm_{tname}_{pname}_{m}x{n}x{k}", lambda: qlinear.gemm(x, w, out=out), 2.0 * m * n * k, wbytes + m * k * 2 + m * n * 2, args)
            del w


def case_small(args):
    """The kernels around the GEMMs and attention at the benchmark's shapes: RMSNorm (+ residual + MXFP8 copy), QK-norm + RoPE +
    cache write, the one-launch MoE front end, the sampler, the Delta-Net recurrence; decode size (64 tokens) and, for the
    bandwidth-bound ones, a prefill chunk (16384 tokens, more than L2)."""
    from ..ops import deltanet as dn, sampling
    h, hq, hkv, d = 2048, 32, 4, 128
    nw = torch.ones(h, device="cuda", dtype=torch.bfloat16)
    for t in (64, 16384):
        x = torch.randn(t, h, device="cuda").bfloat16()
        res = torch.randn(t, h, device="cuda").bfloat16()
        _run(f"rmsnorm_add_quant_{t}x{h}", lambda: ew.rmsnorm(x, nw, 1e-6, residual=res, quantize=True, sf_layout=128), 0.0,
             t * h * (2 + 2 + 2 + 2 + 1), args)
        qkv = torch.randn(t, (hq + 2 * hkv) * d, device="cuda").bfloat16()
        pos = torch.arange(t, device="cuda", dtype=torch.int32) % 4096
        slots = torch.randperm(t, device="cuda").to(torch.int32)
        kc = torch.empty(t, hkv, d, device="cuda", dtype=torch.bfloat16)
        vc = torch.empty_like(kc)
        qw = torch.ones(d, device="cuda", dtype=torch.bfloat16)
        tab = ew.rope_table(4096, d, 1e6, "cuda")
        _run(f"qk_norm_rope_{t}", lambda: ew.qk_norm_rope(qkv, pos, slots, qw, qw, kc, vc, hq, hkv, d, 1e6, 1e-6, 1.0, table=tab), 0.0,
             2 * t * (hq + 2 * hkv) * d * 2, args)
    x = torch.randn(64, h, device="cuda").bfloat16()
    router = (torch.randn(128, h, device="cuda") * 0.05).bfloat16()
    if moe.can_prep(x, router, 8):
        _run("moe_prep_64x2048_top8of128", lambda: moe.prep_hidden(x, router, 8, 128, 32), 2.0 * 64 * 128 * h, 128 * h * 2 + 64 * h * 2 + 512 * h, args)
    logits = torch.randn(64, 151936, device="cuda")
    _run("sampler_top_p_64x151936", lambda: sampling.sample(logits, 0.8, 40, 0.95, seed=1, step=3), 0.0, logits.numel() * 4, args)
    _run("argmax_64x151936", lambda: sampling.argmax(logits), 0.0, logits.numel() * 4, args)
    # Delta-Net layer of the Qwen3.5 shape: 16 key / 32 value heads of 128, one state matrix per value head and sequence
    ng, hv, ds = 16, 32, 128
    for name, lens in (("decode_64", [1] * 64), ("prefill_8x512", [512] * 8)):
        t = sum(lens)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
        sl = torch.arange(len(lens), dtype=torch.int32, device="cuda")
        qkv = (torch.randn(t, (2 * ng + hv) * ds, device="cuda") * 0.5).bfloat16()
        z = torch.randn(t, hv * ds, device="cuda").bfloat16()
        ab = torch.randn(t, 2 * hv, device="cuda")
        a = -(torch.rand(hv, device="cuda") * 2 + 0.1)
        bias = torch.randn(hv, device="cuda") * 0.5
        nwd = torch.rand(ds, device="cuda") + 0.5
        st = torch.randn(len(lens), hv, ds, ds, device="cuda") * 0.1
        _run(f"deltanet_{name}", lambda: dn.deltanet(qkv, z, ab, a, bias, nwd, st, cu, sl, ng, hv, ds, 1e-6), 4.0 * t * hv * ds * ds,
             2 * st.numel() * 4 + qkv.numel() * 2 + 2 * z.numel() * 2, args)


MODEL_CASES = {"spec_verify": case_spec_verify}      # build the whole benchmark model: not part of --case all
CASES = {"gemm": case_gemm, "moe_decode": case_moe_decode, "moe_prefill": case_moe_prefill, "attn_decode": case_attn_decode,
         "attn_prefill": case_attn_prefill, "lm_head": case_lm_head, "quant": case_quant, "small": case_small}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--case", default="all", choices=["all"] + sorted(CASES) + sorted(MODEL_CASES))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--splits", type=int, default=0, help="attention cases: force the number of KV splits")
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=4)
    ap.add_argument("--page", type=int, default=128, help="attention cases: KV page size")
    ap.add_argument("--batch", type=int, default=0, help="attention cases: number of sequences (0 = the case's default)")
    ap.add_argument("--ctx", type=int, default=-1, help="attention cases: cached tokens per sequence (-1 = the case's default)")
    ap.add_argument("--once", action="store_true", help="run each op once, untimed (for use under a profiler)")
    args = ap.parse_args(argv)
    torch.manual_seed(0)
    for name in (sorted(CASES) if args.case == "all" else [args.case]):
        (CASES.get(name) or MODEL_CASES[name])(args)
    print(json.dumps(dict(kernel_status=_native.read_status()["what"])), flush=True)


if __name__ == "__main__":
    main()
