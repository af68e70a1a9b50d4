"""Stock vLLM on the same workload as ``bench.py``: the comparison baseline.

The Ascend reference cannot run on CUDA, so the yardstick for this framework is
the vLLM that is installed in the image, on its own CUDA platform, with its own
kernels and NCCL, and with this repository's platform plugin switched off
(``OMNI_B200_PLUGIN=0``).  The workload is the one ``bench.py`` times:
random-init weights of the named architecture, uniform-random prompt token ids,
``ignore_eos``, greedy sampling, at most ``--max-num-seqs`` running sequences,
paged KV blocks of ``--block-size`` tokens, tensor parallel over ``--gpus``.

One "step" is one pass of the whole workload through ``LLM.generate``.  Every
pass uses fresh random prompts and prefix caching is off, so no pass can reuse
the KV cache of an earlier one.  vLLM spawns its own worker processes for more
than one GPU, so this script is started as plain ``python`` for every N.

    python baseline/run_stock_vllm.py --gpus 1 --steps 2 --warmup 1 [--out FILE]

Prints one JSON line: output tok/s (tokens / wall time of the timed passes),
p50 TTFT and p50 TPOT in ms (vLLM's own per-request timestamps: queued to first
token; first to last token over n - 1), and the vLLM version.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WITH_PLUGIN = "--with-plugin" in sys.argv
if WITH_PLUGIN:
    # the same vLLM entry point, but with this repository's platform plugin active: vLLM's engine
    # core and scheduler drive this package's worker, model runner and kernels
    sys.path.insert(0, ROOT)
    from omni_npu_b200.plugin import write_entry_point_metadata
    _meta = tempfile.mkdtemp(prefix="omni_b200_meta_")
    write_entry_point_metadata(_meta)
    sys.path.insert(0, _meta)
    os.environ["PYTHONPATH"] = os.pathsep.join([ROOT, _meta, os.environ.get("PYTHONPATH", "")])
    os.environ["OMNI_B200_PLUGIN"] = "1"
else:
    os.environ["OMNI_B200_PLUGIN"] = "0"
os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
os.environ.setdefault("VLLM_HOST_IP", "127.0.0.1")

ARCHS = {
    "llama-3-8b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 4096,
        "intermediate_size": 14336, "num_hidden_layers": 32, "num_attention_heads": 32,
        "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 128256, "rms_norm_eps": 1e-5,
        "rope_theta": 500000.0, "max_position_embeddings": 8192, "hidden_act": "silu",
        "tie_word_embeddings": False, "torch_dtype": "bfloat16", "bos_token_id": 128000,
        "eos_token_id": 128001, "attention_bias": False, "mlp_bias": False,
    },
    "qwen3-30b-a3b": {
        "architectures": ["Qwen3MoeForCausalLM"], "model_type": "qwen3_moe", "hidden_size": 2048,
        "intermediate_size": 6144, "moe_intermediate_size": 768, "num_hidden_layers": 48,
        "num_attention_heads": 32, "num_key_value_heads": 4, "head_dim": 128, "vocab_size": 151936,
        "num_experts": 128, "num_experts_per_tok": 8, "norm_topk_prob": True, "decoder_sparse_step": 1,
        "mlp_only_layers": [], "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
        "max_position_embeddings": 40960, "hidden_act": "silu", "tie_word_embeddings": False,
        "torch_dtype": "bfloat16", "attention_bias": False, "bos_token_id": 151643, "eos_token_id": 151645,
    },
    "deepseek-v2-lite": {
        "architectures": ["DeepseekV2ForCausalLM"], "model_type": "deepseek_v2", "hidden_size": 2048,
        "intermediate_size": 10944, "moe_intermediate_size": 1408, "num_hidden_layers": 27,
        "num_attention_heads": 16, "num_key_value_heads": 16, "kv_lora_rank": 512, "q_lora_rank": None,
        "qk_nope_head_dim": 128, "qk_rope_head_dim": 64, "v_head_dim": 128, "n_routed_experts": 64,
        "n_shared_experts": 2, "num_experts_per_tok": 6, "first_k_dense_replace": 1, "moe_layer_freq": 1,
        "n_group": 1, "topk_group": 1, "topk_method": "greedy", "scoring_func": "softmax",
        "norm_topk_prob": False, "routed_scaling_factor": 1.0, "vocab_size": 102400, "rms_norm_eps": 1e-6,
        "rope_theta": 10000.0, "max_position_embeddings": 163840, "hidden_act": "silu",
        "tie_word_embeddings": False, "torch_dtype": "bfloat16", "bos_token_id": 100000,
        "eos_token_id": 100001, "attention_bias": False,
        "rope_scaling": {"type": "yarn", "factor": 40, "original_max_position_embeddings": 4096,
                         "beta_fast": 32, "beta_slow": 1, "mscale": 0.707, "mscale_all_dim": 0.707},
    },
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--model", default="llama-3-8b", choices=sorted(ARCHS))
    ap.add_argument("--num-requests", type=int, default=None)
    ap.add_argument("--input-len", type=int, default=None)
    ap.add_argument("--output-len", type=int, default=None)
    ap.add_argument("--max-num-seqs", type=int, default=128)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--expert-parallel", action="store_true")
    ap.add_argument("--with-plugin", action="store_true",
                    help="activate this repository's vLLM platform plugin instead of vLLM's CUDA platform")
    ap.add_argument("--out", default=None, help="also write the JSON line to this file")
    args = ap.parse_args()
    n, i, o = WORKLOADS[args.model]
    args.num_requests = args.num_requests or n
    args.input_len = args.input_len or i
    args.output_len = args.output_len or o
    return args


# requests, input tokens, output tokens of the named serving configurations
WORKLOADS = {"llama-3-8b": (256, 1024, 256), "deepseek-v2-lite": (512, 2048, 512),
             "qwen3-30b-a3b": (1024, 4096, 256)}


def main() -> None:
    args = parse_args()
    import torch
    import vllm
    from vllm import LLM, SamplingParams

    cfg = dict(ARCHS[args.model])
    model_dir = tempfile.mkdtemp(prefix="stock_vllm_model_")
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f)

    max_len = args.input_len + args.output_len + 16
    kw = dict(model=model_dir, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16",
              tensor_parallel_size=args.gpus, max_num_seqs=args.max_num_seqs, max_model_len=max_len,
              enable_prefix_caching=False, seed=0, disable_log_stats=False,
              enable_expert_parallel=args.expert_parallel)
    note = ""
    try:
        llm = LLM(block_size=args.block_size, **kw)
    except Exception as e:   # a backend that refuses this block size: fall back to vLLM's own choice
        note = f"block_size={args.block_size} refused ({type(e).__name__}); vLLM default block size used"
        llm = LLM(**kw)

    sp = SamplingParams(max_tokens=args.output_len, temperature=0.0, ignore_eos=True, detokenize=False)
    g = torch.Generator().manual_seed(1234)

    def one_pass():
        ids = torch.randint(0, cfg["vocab_size"], (args.num_requests, args.input_len), generator=g).tolist()
        prompts = [{"prompt_token_ids": p} for p in ids]
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp, use_tqdm=False)
        dt = time.perf_counter() - t0
        toks = sum(len(o.outputs[0].token_ids) for o in outs)
        ttft, tpot = [], []
        for o in outs:
            m = o.metrics
            if m is None or not m.first_token_ts:
                continue
            ttft.append(m.first_token_ts - m.queued_ts)
            n = len(o.outputs[0].token_ids)
            if n > 1 and m.last_token_ts:
                tpot.append((m.last_token_ts - m.first_token_ts) / (n - 1))
        return toks, dt, ttft, tpot

    for _ in range(args.warmup):
        one_pass()
    tokens, wall, ttfts, tpots = 0, 0.0, [], []
    for _ in range(args.steps):
        t, dt, a, b = one_pass()
        tokens += t
        wall += dt
        ttfts += a
        tpots += b

    out = {
        "impl": "vllm+omni_npu_b200-plugin" if WITH_PLUGIN else "stock-vllm", "vllm_version": vllm.__version__, "torch": torch.__version__,
        "metric": "output tok/s (whole box)", "value": round(tokens / wall, 1), "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(wall * 1e3 / args.steps, 2),
        "ttft_p50_ms": round(statistics.median(ttfts) * 1e3, 2) if ttfts else None,
        "tpot_p50_ms": round(statistics.median(tpots) * 1e3, 3) if tpots else None,
        "timing": "wall clock around LLM.generate (vLLM has no device-side step timer)",
        "config": {"model": args.model, "requests": args.num_requests, "input_len": args.input_len,
                   "output_len": args.output_len, "max_num_seqs": args.max_num_seqs,
                   "kv_block": args.block_size, "parallelism": f"tp{args.gpus}"
                   + ("+ep" if args.expert_parallel else ""), "note": note},
    }
    if WITH_PLUGIN:
        from vllm.platforms import current_platform
        out["platform"] = type(current_platform).__name__
        out["worker_cls"] = llm.llm_engine.vllm_config.parallel_config.worker_cls
    line = json.dumps(out)
    print(line, flush=True)
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            f.write(line + "\n")
    del llm
    sys.stdout.flush()


if __name__ == "__main__":
    main()
