"""Headline benchmark: output tokens/s of offline serving.

Workload (the dense-GQA serving config): Llama-3-8B architecture, bf16, random
init (normal, std 0.02), 256 requests of 1024 uniform-random input tokens and
256 output tokens each (ignore_eos), at most 128 running sequences, paged KV
with 16-token blocks, tensor parallel over N GPUs of one node.

One benchmark "step" is one complete pass of that workload through the public
``LLM.generate`` API: continuous batching, prefill and decode, and in every
engine step a host-to-device copy of the step's inputs from pinned memory and
a device-to-host read of the sampled tokens.

Two numbers come out of the same K timed passes:
  * ``e2e.value``  output tokens / wall time of the passes (barrier +
                   synchronize on both sides, max over ranks);
  * ``value``      output tokens / device time, the sum over engine steps of
                   CUDA-event intervals around each step's kernels (forward,
                   LM head, sampling), i.e. without host gaps and copies.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--num-requests", type=int, default=None)
    ap.add_argument("--input-len", type=int, default=None)
    ap.add_argument("--output-len", type=int, default=None)
    ap.add_argument("--max-num-seqs", type=int, default=128)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--no-fused-collectives", action="store_true")
    ap.add_argument("--mixed-batches", action="store_true",
                    help="decoding requests ride along in prefill steps (default: prompts first)")
    ap.add_argument("--profile", default=None,
                    help="write a per-kernel time table (torch profiler, one extra untimed pass) to this file")
    args = ap.parse_args()
    n, i, o = WORKLOADS.get(args.model, WORKLOADS["llama-3-8b"])
    args.num_requests = args.num_requests or n
    args.input_len = args.input_len or i
    args.output_len = args.output_len or o
    return args


# requests, input tokens, output tokens of the named serving configurations
WORKLOADS = {"llama-3-8b": (256, 1024, 256), "deepseek-v2-lite": (512, 2048, 512),
             "qwen3-30b-a3b": (1024, 4096, 256), "deepseek-v3.2": (256, 8192, 1024)}


# ------------------------------------------------------------------ reference
def run_reference(args) -> None:
    """The reference arm must run the unmodified reference package from
    baseline/_ref through its own entry point.  That package is an Ascend
    plugin: its platform probe imports torch_npu, which does not exist for
    CUDA, so on this hardware it declines to activate."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    rank = int(os.environ.get("RANK", "0"))
    why = None
    if not os.path.isdir(os.path.join(ref_dir, "omni_npu")):
        why = "reference package not installed under baseline/_ref"
    else:
        sys.path.insert(0, ref_dir)
        try:
            from omni_npu.vllm_plugin import plugin  # type: ignore
            target = plugin()
            if target is None:
                why = ("reference platform plugin returns None: it needs torch_npu / Ascend CANN "
                       "devices and has no CUDA code path")
            else:  # pragma: no cover - cannot happen without torch_npu
                import importlib
                mod, cls = target.rsplit(".", 1)
                getattr(importlib.import_module(mod), cls)
                why = "reference platform imported but no Ascend device is present"
        except Exception as e:  # pragma: no cover
            why = f"reference import failed: {type(e).__name__}: {e}"
    if rank == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))


# --------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.path = f"/tmp/omni_b200_clocks_{os.getpid()}.csv"

    def start(self) -> None:
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "200"], stdout=self.f,
                stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


# ----------------------------------------------------------------------- ours
def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from omni_npu_b200 import SamplingParams, ops
    from omni_npu_b200.config import PRESETS
    from omni_npu_b200.engine.llm import LLM, build_engine_config

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
        args.gpus = world
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local_rank)

    mc = PRESETS[args.model]()
    max_len = args.input_len + args.output_len + 16
    moe = getattr(mc, "num_experts", 0) > 0
    cfg = build_engine_config(
        mc, tensor_parallel_size=args.gpus, enable_expert_parallel=moe and args.gpus > 1,
        max_num_seqs=args.max_num_seqs,
        max_num_batched_tokens=args.max_num_batched_tokens, max_model_len=max_len,
        block_size=args.block_size, device="cuda", seed=0, enable_mixed_batches=args.mixed_batches,
        additional_config={"fused_collectives": not args.no_fused_collectives})
    llm = LLM(cfg)
    runner = llm.engine.worker.model_runner
    runner.enable_step_events = True

    g = torch.Generator().manual_seed(1234)
    prompts = torch.randint(0, mc.vocab_size, (args.num_requests, args.input_len), generator=g).tolist()
    sp = SamplingParams(max_tokens=args.output_len, temperature=0.0, ignore_eos=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    ttfts, tpots = [], []

    def one_pass():
        outs = llm.generate(prompts, sp)
        ttfts.extend(o.ttft for o in outs if o.ttft is not None)
        tpots.extend(o.tpot for o in outs if o.tpot is not None)
        return sum(len(o.output_token_ids) for o in outs)

    for _ in range(args.warmup):
        one_pass()
        runner.drain_step_events()

    if args.profile and rank == 0:
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            one_pass()
            torch.cuda.synchronize()
        runner.drain_step_events()
        with open(args.profile, "w") as f:
            f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=40,
                                              max_name_column_width=90))
    elif args.profile:
        one_pass()
        runner.drain_step_events()

    runner.step_ms_by_kind.clear()
    runner.step_count_by_kind.clear()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    st0 = dict(llm.engine.stats)
    launches0 = ops.launch_count()
    ttfts.clear()
    tpots.clear()
    barrier()
    t0 = time.perf_counter()
    tokens = 0
    device_ms = 0.0
    for _ in range(args.steps):
        tokens += one_pass()
        device_ms += runner.drain_step_events()
    barrier()
    wall = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    launches = ops.launch_count() - launches0
    st1 = llm.engine.stats
    engine_steps = st1["steps"] - st0["steps"]

    # max over ranks of both times
    t = torch.tensor([wall, device_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    wall, device_ms = float(t[0]), float(t[1])
    ops.check_status()

    if rank == 0:
        value = tokens / (device_ms / 1e3)
        e2e = tokens / wall
        out = {
            "metric": "output tok/s (whole box, max over ranks)",
            "value": round(value, 1),
            "unit": "tok/s",
            "n_gpus": args.gpus,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(device_ms / args.steps, 2),
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": _vs_stock(args, e2e),
            "baseline": _stock_entry(args),
            "ttft_p50_ms": round(statistics.median(ttfts) * 1e3, 2) if ttfts else None,
            "tpot_p50_ms": round(statistics.median(tpots) * 1e3, 3) if tpots else None,
            "dtype": "bf16",
            "data": "synthetic uniform-random token ids; random-init weights (normal, std 0.02)",
            "impl": "ours",
            "config": {
                "model": "Llama-3-8B architecture (32 layers, hidden 4096, 32 q / 8 kv heads, "
                         "head_dim 128, FFN 14336, vocab 128256)" if args.model == "llama-3-8b" else args.model,
                "requests": args.num_requests, "input_len": args.input_len,
                "output_len": args.output_len, "global_batch": args.max_num_seqs,
                "seq_len": args.input_len + args.output_len, "kv_block": args.block_size,
                "parallelism": (f"ep{args.gpus}+tp{args.gpus}" if moe and args.gpus > 1 else f"tp{args.gpus}"),
                "step_definition": "one pass of the full workload through LLM.generate",
                "l2_policy": "inputs larger than L2: every engine step streams the weights "
                             "(16 GB / N) and the KV cache, far above the 126 MB L2",
                "engine_steps_per_pass": engine_steps // max(1, args.steps),
                # which kernels ran the plain decode-sized projections (qkv, o, down): "library" = cuBLAS
                # (not counted in gpu_launches), "own" = gemm_tcgen05_kernel; everything else is own code
                "small_m_gemm": ops.SMALL_M_GEMM, "mixed_batches": bool(args.mixed_batches),
            },
            "device_ms_by_step_kind": {k: round(v / args.steps, 1) for k, v in runner.step_ms_by_kind.items()},
            "steps_by_kind": {k: v // args.steps for k, v in runner.step_count_by_kind.items()},
            "e2e": {
                "value": round(e2e, 1), "unit": "tok/s",
                "wall_ms_per_step": round(wall * 1e3 / args.steps, 2),
                "h2d_bytes_per_step": (st1["h2d_bytes"] - st0["h2d_bytes"]) // max(1, args.steps),
                "d2h_bytes_per_step": (st1["d2h_bytes"] - st0["d2h_bytes"]) // max(1, args.steps),
            },
            "gpu_launches": launches,
            "clocks": clocks,
        }
        print(json.dumps(out), flush=True)
    _shutdown(llm, world)


def _stock_entry(args):
    """The measured stock-vLLM number for this model and GPU count (written by
    baseline/run_stock_vllm.py on the same kind of box), or None."""
    path = os.path.join(ROOT, "baseline", "stock_vllm_results.json")
    try:
        with open(path) as f:
            table = json.load(f)
    except Exception:
        return None
    same = (args.num_requests, args.input_len, args.output_len) == WORKLOADS.get(args.model) and \
        args.max_num_seqs == 128
    return table.get(args.model, {}).get(str(args.gpus)) if same else None


def _vs_stock(args, e2e_tok_s: float):
    """Ours / stock vLLM, both end to end (wall clock around generate), same N."""
    ent = _stock_entry(args)
    if not ent or not ent.get("value"):
        return None
    return round(e2e_tok_s / float(ent["value"]), 3)


def _shutdown(llm, world: int) -> None:
    """Orderly teardown, then a normal interpreter exit (exit hooks run).  A
    watchdog ends the process only if a library's finaliser blocks for 30 s, and
    says so."""
    import threading

    import torch.distributed as dist

    def _deadline():
        print("shutdown watchdog fired after 30 s: forcing exit", file=sys.stderr)
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)

    timer = threading.Timer(30.0, _deadline)
    timer.daemon = True
    timer.start()
    t0 = time.perf_counter()
    stage = "start"

    def mark(name):
        nonlocal stage
        stage = name
        if os.environ.get("OMNI_B200_BENCH_SHUTDOWN_TRACE"):
            print(f"shutdown[{os.environ.get('RANK', '0')}] {time.perf_counter() - t0:6.2f}s {name}", file=sys.stderr,
                  flush=True)
    try:
        import gc

        import torch
        if world > 1:
            dist.barrier()
        mark("barrier done")
        from omni_npu_b200.parallel import state as pstate
        runner = llm.engine.worker.model_runner
        llm.engine.shutdown()
        # captured graphs hold the communicators' buffers and streams: let them go before the
        # communicators are destroyed
        if getattr(runner, "graphs", None):
            runner.graphs.clear()
        gc.collect()
        torch.cuda.synchronize()
        mark("engine down, graphs released")
        pstate.destroy_model_parallel()
        mark("groups destroyed")
        if world > 1 and dist.is_initialized():
            dist.destroy_process_group()
        mark("process group destroyed")
    except Exception as e:  # pragma: no cover - best effort
        print(f"shutdown after '{stage}': {type(e).__name__}: {e}", file=sys.stderr)
    sys.stdout.flush()
    sys.stderr.flush()
    # the watchdog stays armed through interpreter shutdown (daemon timer): a clean exit beats it


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
