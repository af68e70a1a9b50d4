"""Kernel micro-benchmarks with roofline fractions.

    python -m omni_npu_b200.ops.bench_kernels gemm            # GEMM shapes of the serving configs
    python -m omni_npu_b200.ops.bench_kernels gemm --m 128 --n 4096 --k 4096 --bn 128 --splits 4
    python -m omni_npu_b200.ops.bench_kernels attn | norm | sample | indexer | quant | all

Timing: CUDA events on the launching stream, 3 warm-up launches, L2 flushed
(a 256 MB buffer is rewritten) before every timed launch, median of the timed
launches.  Fractions are of the measured peaks in MEASURED_PEAKS.json at the
repository root when present (copy bandwidth and cuBLAS bf16 throughput), else
of 6.65 TB/s / 1.59 PFLOP/s.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

from omni_npu_b200 import ops


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    except Exception:
        return 6.65e12, 1.59e15, "fallback"


_flush = None


def time_fn(fn, iters=10, warmup=3, flush=True):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        if flush:
            _flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times)


SERVING_GEMMS = [
    # (label, M, N, K)
    ("llama8b qkv prefill", 8192, 6144, 4096), ("llama8b o prefill", 8192, 4096, 4096),
    ("llama8b gate_up prefill", 8192, 28672, 4096), ("llama8b down prefill", 8192, 4096, 14336),
    ("llama8b qkv decode", 128, 6144, 4096), ("llama8b o decode", 128, 4096, 4096),
    ("llama8b gate_up decode", 128, 28672, 4096), ("llama8b down decode", 128, 4096, 14336),
    ("llama8b lm_head decode", 128, 128256, 4096),
    ("square 8192", 8192, 8192, 8192),
]


def time_graph(make_fns, iters=5):
    """Capture the given launches (each reading different buffers, together larger
    than L2) in one CUDA graph and return the mean device time per launch in ms.
    This is how launch-bound decode kernels run in production: back to back from a
    graph, with cold operands but no host gaps."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for f in make_fns:
            f()
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in make_fns:
            f()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.median(times) / len(make_fns)


def bench_gemm_graph(args):
    hbm, flops_peak, src = peaks()
    shapes = [s for s in SERVING_GEMMS if s[1] <= 512] if args.m is None else [("custom", args.m, args.n, args.k)]
    print(f"# GEMM bf16 inside a CUDA graph over rotating weights (> L2 in total); fractions of {src} peaks")
    print(f"{'shape':28s} {'M':>6s} {'N':>7s} {'K':>6s} {'bn':>4s} {'sp':>3s} {'ours_us':>9s} {'cublas_us':>9s} "
          f"{'GB/s':>7s} {'frac':>5s} {'vs_cublas':>9s}")
    for label, m, n, k in shapes:
        nbuf = max(4, min(64, (300 << 20) // (n * k * 2) + 1))
        a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        ws = [torch.randn(n, k, device="cuda", dtype=torch.bfloat16) * 0.05 for _ in range(nbuf)]
        bn, sp = args.bn, args.splits
        plan = torch.ops.omni_b200.gemm_plan(m, n, k, 2, False, bn, sp)
        t = time_graph([(lambda w=w: ops.gemm(a, w, bn=bn, splits=sp)) for w in ws])
        tc = time_graph([(lambda w=w: torch.matmul(a, w.t())) for w in ws])
        by = 2.0 * (m * k + n * k + m * n)
        fl = 2.0 * m * n * k
        frac = max(fl / flops_peak, by / hbm) / (t / 1e3)
        print(f"{label:28s} {m:6d} {n:7d} {k:6d} {plan[0]:4d} {plan[1]:3d} {t*1e3:9.1f} {tc*1e3:9.1f} "
              f"{by/t/1e6:7.0f} {frac:5.2f} {tc/t:9.2f}")
    ops.check_status()


def bench_gemm(args):
    if args.graph:
        return bench_gemm_graph(args)
    hbm, flops_peak, src = peaks()
    shapes = SERVING_GEMMS if args.m is None else [("custom", args.m, args.n, args.k)]
    print(f"# GEMM bf16, fractions of {src} peaks: {hbm/1e12:.2f} TB/s, {flops_peak/1e12:.0f} TFLOP/s")
    print(f"{'shape':28s} {'M':>6s} {'N':>7s} {'K':>6s} {'bn':>4s} {'sp':>3s} {'ours_us':>9s} {'cublas_us':>9s} "
          f"{'TFLOP/s':>8s} {'GB/s':>7s} {'frac':>5s} {'vs_cublas':>9s}")
    for label, m, n, k in shapes:
        a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(n, k, device="cuda", dtype=torch.bfloat16) * 0.05
        bn, sp = args.bn, args.splits
        plan = torch.ops.omni_b200.gemm_plan(m, n, k, 2, False, bn, sp)
        if args.pair and m >= 256:
            t = time_fn(lambda: ops.gemm(a, w, bn=bn, pair=True), iters=args.iters)
            plan = (bn or 256, 1)
            label = label + " [pair]"
        else:
            t = time_fn(lambda: ops.gemm(a, w, bn=bn, splits=sp), iters=args.iters)
        tc = time_fn(lambda: torch.matmul(a, w.t()), iters=args.iters)
        fl = 2.0 * m * n * k
        by = 2.0 * (m * k + n * k + m * n)
        tf, gb = fl / t / 1e9, by / t / 1e6
        frac = max(fl / flops_peak, by / hbm) / (t / 1e3)
        print(f"{label:28s} {m:6d} {n:7d} {k:6d} {plan[0]:4d} {plan[1]:3d} {t*1e3:9.1f} {tc*1e3:9.1f} "
              f"{tf:8.1f} {gb:7.0f} {frac:5.2f} {tc/t:9.2f}")
    ops.check_status()


def bench_attn(args):
    hbm, flops_peak, src = peaks()
    print(f"# paged GQA attention, fractions of {src} peaks")
    hq, hk, d, bs = args.hq, args.hk, 128, args.block_size       # 32 / 8: Llama-3-8B on one GPU; 16 / 4, 8 / 2, 4 / 1: TP 2, 4, 8
    decode_cases = ((128, 1152), (128, 4096), (16, 8192), (1, 32768))
    prefill_cases = ((8, 1024), (2, 4096), (1, 8192))
    if args.b is not None:
        decode_cases = ((args.b, args.ctx),) if args.phase != "prefill" else ()
        prefill_cases = ((args.b, args.ctx),) if args.phase != "decode" else ()
    for b, ctx in decode_cases:
        nblk = b * ((ctx + bs - 1) // bs) + 1
        kc = torch.randn(nblk, hk, bs, d, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn_like(kc)
        q = torch.randn(b, hq * d, device="cuda", dtype=torch.bfloat16)
        bt = torch.arange(1, nblk, device="cuda", dtype=torch.int32).view(b, -1)
        sl = torch.full((b,), ctx, device="cuda", dtype=torch.int32)
        if args.ctx_spread > 0:      # lengths spread evenly over [ctx - spread, ctx]
            sl = (ctx - torch.arange(b, device="cuda") * args.ctx_spread // max(1, b - 1)).to(torch.int32)
            by_scale = float(sl.sum()) / (b * ctx)
        else:
            by_scale = 1.0
        for splits in ((0,) if args.splits == 0 else (args.splits,)):
            by = 2.0 * b * ctx * hk * d * 2 * by_scale
            for persistent in (2, 1, 0):
                used = 1 if persistent == 2 else (
                    splits or (ops.decode_splits_persistent if persistent else ops.decode_splits)(b, hk, ctx))
                t = time_fn(lambda: ops.gqa_decode(q, kc, vc, bt, sl, b, hq, d ** -0.5, splits=splits,
                                                   max_seq_len=ctx, persistent=persistent), iters=args.iters)
                kind = ("one CTA per item", "persistent CTAs", "balanced persistent CTAs")[persistent]
                print(f"decode  B={b:4d} ctx={ctx:6d} splits={used:2d} {kind}: {t*1e3:8.1f} us  "
                      f"{by/t/1e6:7.0f} GB/s frac {by/hbm/(t/1e3):.2f}")
    if prefill_cases:
        import ctypes
        lib = ctypes.CDLL(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_C.so"))
        print(f"# tcgen05 prefill kernel: {lib.b200_gqa_prefill_tc_ctas_per_sm(0)} CTAs per SM "
              f"(by shared memory size: " + ", ".join(f"{k} KiB -> {lib.b200_gqa_prefill_tc_ctas_per_sm(k << 10)}"
                                                       for k in (96, 104, 108, 110, 111, 112, 113)) + ")")
        res = (ctypes.c_int * 8)()
        lib.b200_gqa_prefill_tc_resources(res)
        print("# registers/thread, static smem, max dyn smem, smem/SM, regs/SM, reserved smem/block, max blocks/SM, "
              "local bytes:", list(res))
    for b, s in prefill_cases:
        nblk = b * (s // bs) + 1
        kc = torch.randn(nblk, hk, bs, d, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn_like(kc)
        q = torch.randn(b * s, hq * d, device="cuda", dtype=torch.bfloat16)
        bt = torch.arange(1, nblk, device="cuda", dtype=torch.int32).view(b, -1)
        sl = torch.full((b,), s, device="cuda", dtype=torch.int32)
        cu = torch.arange(0, (b + 1) * s, s, device="cuda", dtype=torch.int32)
        fl = 4.0 * b * hq * s * s * d / 2
        for tc in (True, False):
            t = time_fn(lambda: ops.gqa_prefill(q, kc, vc, bt, cu, sl, b, s, hq, d ** -0.5, tcgen05=tc),
                        iters=args.iters)
            kind = "tcgen05 + TMEM" if tc else "mma.sync      "
            print(f"prefill B={b:3d} S={s:6d} {kind}: {t*1e3:9.1f} us  {fl/t/1e9:7.1f} TFLOP/s  "
                  f"frac {fl/flops_peak/(t/1e3):.2f}")
    ops.check_status()


def bench_norm(args):
    hbm, _, src = peaks()
    print(f"# row kernels, fractions of {src} copy bandwidth")
    for t_, h in ((8192, 4096), (128, 4096), (8192, 7168), (65536, 4096)):
        x = torch.randn(t_, h, device="cuda", dtype=torch.bfloat16)
        r = torch.randn_like(x)
        w = torch.ones(h, device="cuda", dtype=torch.bfloat16)
        t = time_fn(lambda: ops.rms_norm(x, w, 1e-6), iters=args.iters)
        by = 2.0 * t_ * h * 2
        print(f"rms_norm      [{t_},{h}]: {t*1e3:8.1f} us {by/t/1e6:7.0f} GB/s frac {by/hbm/(t/1e3):.2f}")
        t = time_fn(lambda: ops.fused_add_rms_norm(x, r, w, 1e-6), iters=args.iters)
        by = 2.0 * t_ * h * 4
        print(f"add_rms_norm  [{t_},{h}]: {t*1e3:8.1f} us {by/t/1e6:7.0f} GB/s frac {by/hbm/(t/1e3):.2f}")
    x = torch.randn(8192, 2 * 14336, device="cuda", dtype=torch.bfloat16)
    t = time_fn(lambda: ops.silu_and_mul(x), iters=args.iters)
    by = 2.0 * 8192 * 14336 * 3
    print(f"silu_and_mul  [8192,28672]: {t*1e3:8.1f} us {by/t/1e6:7.0f} GB/s frac {by/hbm/(t/1e3):.2f}")


def bench_sample(args):
    hbm, _, src = peaks()
    for b, v in ((128, 128256), (1, 128256), (128, 151936)):
        logits = torch.randn(b, v, device="cuda", dtype=torch.float32)
        temp = torch.full((b,), 0.8, device="cuda")
        tk = torch.full((b,), 50, dtype=torch.int32, device="cuda")
        tp = torch.full((b,), 0.9, device="cuda")
        seeds = torch.arange(b, device="cuda")
        step = torch.zeros(1, dtype=torch.int64, device="cuda")
        t0 = time_fn(lambda: ops.argmax(logits), iters=args.iters)
        t1 = time_fn(lambda: ops.sample(logits, temp, tk, tp, seeds, step), iters=args.iters)
        print(f"B={b:4d} V={v}: argmax {t0*1e3:7.1f} us ({4.0*b*v/t0/1e6:6.0f} GB/s), "
              f"top-k/top-p sample {t1*1e3:7.1f} us")


def bench_quant(args):
    """Quantised GEMMs at a prefill and a decode shape: per-token x per-channel scaled e4m3 / int8
    (one accumulation, scales in the epilogue) and 128 x 128 block-scaled e4m3 (per-slab promotion)."""
    from omni_npu_b200.layers.quant_fp8 import quantize_weight_block
    _, flops, src = peaks()
    print(f"# quantised GEMMs, TFLOP/s and fraction of the {src} bf16 peak (fp8 / int8 nominal peak is 2x bf16)")
    shapes = ((8192, 4096, 4096), (8192, 7168, 2048), (128, 4096, 7168))
    if args.m and args.n and args.k:
        shapes = ((args.m, args.n, args.k),)
    for m, n, k in shapes:
        x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(n, k, device="cuda", dtype=torch.float32) * 0.05
        fl = 2.0 * m * n * k
        t = time_fn(lambda: ops.gemm(x, w.bfloat16()), iters=args.iters)
        print(f"bf16            [{m},{n},{k}]: {t*1e3:8.1f} us {fl/t/1e9:7.1f} TFLOP/s frac {fl/flops/(t/1e3):.2f}")
        wq, ws = quantize_weight_block(w)
        xq, xs = ops.quant_fp8_1x128(x)
        t = time_fn(lambda: ops.gemm_fp8_block(xq, xs, wq, ws), iters=args.iters)
        print(f"e4m3 128x128    [{m},{n},{k}]: {t*1e3:8.1f} us {fl/t/1e9:7.1f} TFLOP/s frac {fl/flops/(t/1e3):.2f}")
        wr = (w / w.abs().amax(1, keepdim=True) * 448).to(torch.float8_e4m3fn)
        wsr = (w.abs().amax(1) / 448).float()
        xr = (x.float() / x.float().abs().amax(1, keepdim=True) * 448).to(torch.float8_e4m3fn)
        xsr = (x.float().abs().amax(1) / 448).float()
        t = time_fn(lambda: ops.gemm_scaled(xr, wr, xsr, wsr), iters=args.iters)
        print(f"e4m3 row x col  [{m},{n},{k}]: {t*1e3:8.1f} us {fl/t/1e9:7.1f} TFLOP/s frac {fl/flops/(t/1e3):.2f}")
        xi, xsi = ops.quant_int8_per_token(x)
        wi = torch.round(w / w.abs().amax(1, keepdim=True) * 127).to(torch.int8)
        wsi = (w.abs().amax(1) / 127).float()
        t = time_fn(lambda: ops.gemm_scaled(xi, wi, xsi, wsi), iters=args.iters)
        print(f"int8 row x col  [{m},{n},{k}]: {t*1e3:8.1f} us {fl/t/1e9:7.1f} TFLOP/s frac {fl/flops/(t/1e3):.2f}")


def bench_indexer(args):
    """Sparse-attention indexer (64 heads x 128 dims, page 16, top-2048): decode batches and one
    prefill chunk.  Bytes = the index keys read once; FLOPs = 2 * heads * 128 per (token, key)."""
    hbm, flops, src = peaks()
    print(f"# dsa indexer: scores (tcgen05) + radix select, fractions of {src} peaks")
    h, bs, topk = 64, 16, 2048
    cases = [("decode", 128, 1, 4096), ("decode", 128, 1, 16384), ("decode", 32, 2, 32768), ("prefill", 2, 4096, 4096)]
    if args.b:
        cases = [(args.phase if args.phase != "both" else "decode", args.b, 1, args.ctx)]
    for mode, b, ql, ctx in cases:
        max_blocks = (ctx + bs - 1) // bs
        cache = torch.randn(b * max_blocks, bs, 128, device="cuda", dtype=torch.bfloat16)
        bt = torch.arange(b * max_blocks, device="cuda", dtype=torch.int32).view(b, max_blocks)
        t = b * ql
        q = torch.randn(t, h, 128, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(t, h, device="cuda") * 0.1
        pos = (torch.arange(ctx - ql, ctx, dtype=torch.int32).repeat(b)).cuda()
        cu = torch.arange(0, t + 1, ql, dtype=torch.int32, device="cuda")
        kw = dict(cu_q=cu if mode == "prefill" else None, q_len=ql, max_ctx=ctx, max_q=ql)
        ms = time_fn(lambda: ops.dsa_indexer_topk(q, w, cache, bt, pos, b, topk, **kw), iters=args.iters)
        pairs = b * (ql * (ctx - ql) + ql * (ql + 1) / 2)
        fl = 2.0 * h * 128 * pairs
        by = b * ctx * 256.0
        print(f"{mode:8s} B={b:4d} q={ql:5d} ctx={ctx:6d}: {ms*1e3:8.1f} us  {fl/ms/1e9:7.1f} TFLOP/s "
              f"(frac {fl/flops/(ms/1e3):.2f})  keys {by/ms/1e6:6.0f} GB/s (frac {by/hbm/(ms/1e3):.2f})")


def bench_moe(args):
    """Grouped (per-expert) GEMMs of the MoE layers at decode and prefill row counts, uniform routing."""
    hbm, flops_peak, src = peaks()
    print(f"# grouped expert GEMMs bf16, fractions of {src} peaks")
    print(f"{'shape':34s} {'rows':>6s} {'E':>4s} {'N':>6s} {'K':>6s} {'us':>9s} {'GB/s':>7s} {'TFLOP/s':>8s} {'frac':>5s}")
    cases = (("v2-lite w13 decode", 128 * 6, 64, 2 * 1408, 2048, True), ("v2-lite w2 decode", 128 * 6, 64, 2048, 1408, False),
             ("qwen3-30b w13 decode", 128 * 8, 128, 2 * 768, 2048, True), ("qwen3-30b w2 decode", 128 * 8, 128, 2048, 768, False),
             ("v2-lite w13 prefill", 8192 * 6, 64, 2 * 1408, 2048, True), ("qwen3-30b w13 prefill", 8192 * 8, 128, 2 * 768, 2048, True))
    for label, rows, e, n, k, swiglu in cases:
        torch.manual_seed(0)
        ids = torch.randint(0, e, (rows,), device="cuda")
        counts = torch.bincount(ids, minlength=e)
        offs = torch.zeros(e + 1, dtype=torch.int32, device="cuda")
        offs[1:] = torch.cumsum(counts, 0)
        a = torch.randn(rows, k, device="cuda", dtype=torch.bfloat16)
        w = torch.randn(e, n, k, device="cuda", dtype=torch.bfloat16) * 0.05
        t = time_fn(lambda: ops.grouped_gemm(a, w, offs, swiglu=swiglu), iters=args.iters)
        by = 2.0 * (e * n * k + rows * k + rows * (n // 2 if swiglu else n))
        fl = 2.0 * rows * n * k
        frac = max(fl / flops_peak, by / hbm) / (t / 1e3)
        print(f"{label:34s} {rows:6d} {e:4d} {n:6d} {k:6d} {t*1e3:9.1f} {by/t/1e6:7.0f} {fl/t/1e9:8.1f} {frac:5.2f}")
    ops.check_status()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attn", "norm", "sample", "indexer", "quant", "moe", "all"])
    ap.add_argument("--m", type=int)
    ap.add_argument("--n", type=int)
    ap.add_argument("--k", type=int)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--pair", action="store_true", help="gemm: run M >= 256 shapes on the CTA-pair kernel")
    ap.add_argument("--graph", action="store_true",
                    help="gemm: time decode-shaped GEMMs back to back inside a CUDA graph")
    ap.add_argument("--hq", type=int, default=32, help="attn: query heads")
    ap.add_argument("--hk", type=int, default=8, help="attn: KV heads")
    ap.add_argument("--b", type=int, help="attn: batch size of a single case")
    ap.add_argument("--ctx", type=int, default=1024, help="attn: context length of a single case")
    ap.add_argument("--ctx-spread", type=int, default=0, help="attn decode: lengths spread over [ctx - spread, ctx]")
    ap.add_argument("--block-size", type=int, default=16, help="attn: tokens per cache block")
    ap.add_argument("--phase", default="both", choices=["both", "decode", "prefill"])
    args = ap.parse_args()
    ops.load_extension(required=True)
    if args.what in ("gemm", "all"):
        bench_gemm(args)
    if args.what in ("attn", "all"):
        bench_attn(args)
    if args.what in ("norm", "all"):
        bench_norm(args)
    if args.what in ("sample", "all"):
        bench_sample(args)
    if args.what in ("indexer", "all"):
        bench_indexer(args)
    if args.what in ("quant", "all"):
        bench_quant(args)
    if args.what in ("moe", "all"):
        bench_moe(args)


if __name__ == "__main__":
    main()
