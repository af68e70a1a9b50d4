"""Child process of the vLLM-engine tests: runs a vLLM ``LLM`` whose platform, worker and
model runner come from this package's plugin, and the package's standalone engine on the same
weights, and prints both token lists as one JSON line.

    python tests/vllm_engine_child.py cpu|cuda [tp] [max_num_seqs] [max_num_batched_tokens]
"""
import json
import os
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main() -> None:
    mode = sys.argv[1]
    tp = int(sys.argv[2]) if len(sys.argv) > 2 else 1
    seqs = int(sys.argv[3]) if len(sys.argv) > 3 else 1
    budget = int(sys.argv[4]) if len(sys.argv) > 4 else 64
    spec = sys.argv[5] if len(sys.argv) > 5 else ""          # "ngram": vLLM-driven n-gram speculative decoding
    os.environ["OMNI_B200_PLUGIN"] = "cpu" if mode == "cpu" else "1"
    if tp == 1:
        os.environ["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"
    os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")
    os.environ.setdefault("VLLM_HOST_IP", "127.0.0.1")
    from omni_npu_b200.plugin import write_entry_point_metadata
    meta = tempfile.mkdtemp(prefix="omni_b200_meta_")
    write_entry_point_metadata(meta)
    sys.path.insert(0, meta)
    os.environ["PYTHONPATH"] = os.pathsep.join([ROOT, meta, os.environ.get("PYTHONPATH", "")])

    import torch
    fp32 = mode == "cpu"
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama",
           "hidden_size": 256 if fp32 else 1024, "intermediate_size": 512 if fp32 else 2816,
           "num_hidden_layers": 2, "num_attention_heads": 4 if fp32 else 8, "num_key_value_heads": 2,
           "head_dim": 64 if fp32 else 128, "vocab_size": 1024 if fp32 else 4096, "rms_norm_eps": 1e-5,
           "rope_theta": 10000.0, "max_position_embeddings": 2048, "hidden_act": "silu",
           "tie_word_embeddings": False, "torch_dtype": "float32" if fp32 else "bfloat16",
           "bos_token_id": 1, "eos_token_id": 2}
    if spec == "mtp":
        # a small DeepSeek-V3 shaped model (latent attention, routed + shared experts) with one
        # multi-token-prediction layer: vLLM schedules the drafts that the runner's MTP head makes
        cfg = {"architectures": ["DeepseekV3ForCausalLM"], "model_type": "deepseek_v3", "hidden_size": 128,
               "intermediate_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 4,
               "vocab_size": 512, "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 512,
               "hidden_act": "silu", "tie_word_embeddings": False, "torch_dtype": "float32" if fp32 else "bfloat16",
               "bos_token_id": 1, "eos_token_id": 2, "n_routed_experts": 8, "num_experts_per_tok": 2,
               "moe_intermediate_size": 64, "n_shared_experts": 1, "first_k_dense_replace": 1, "moe_layer_freq": 1,
               "scoring_func": "sigmoid", "norm_topk_prob": True, "routed_scaling_factor": 1.0, "n_group": 1,
               "topk_group": 1, "topk_method": "noaux_tc", "kv_lora_rank": 512, "q_lora_rank": None,
               "qk_nope_head_dim": 32, "qk_rope_head_dim": 64, "v_head_dim": 32, "num_nextn_predict_layers": 1,
               "attention_bias": False, "rope_scaling": None}
        if not fp32:
            # the sizes of the GPU end-to-end tests (head sizes 128 + 64 / 128 that the kernels take)
            cfg.update({"hidden_size": 512, "intermediate_size": 1024, "num_hidden_layers": 3,
                        "num_attention_heads": 16, "num_key_value_heads": 16, "vocab_size": 2048,
                        "n_routed_experts": 16, "num_experts_per_tok": 4, "moe_intermediate_size": 256,
                        "n_group": 4, "topk_group": 2, "routed_scaling_factor": 2.5, "q_lora_rank": 256,
                        "qk_nope_head_dim": 128, "v_head_dim": 128, "max_position_embeddings": 2048})
    d = os.environ.get("OMNI_B200_TEST_MODEL_DIR")     # a checkpoint directory (config + safetensors)
    load_format = "auto" if d else "dummy"
    if not d:
        d = tempfile.mkdtemp(prefix="omni_b200_model_")
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg["vocab_size"], (32,), generator=g).tolist() for _ in range(4)]
    n_out = 16
    extra = {}
    if spec == "ngram":
        # prompts that repeat themselves, so that the look-up finds drafts, and enough new tokens
        # for a tiny random model to fall into a loop of its own
        prompts = [(p[:8] * 4) for p in prompts]
        n_out = 40
        extra["speculative_config"] = {"method": "ngram", "num_speculative_tokens": 3,
                                       "prompt_lookup_max": 3, "prompt_lookup_min": 2}
    want_logprobs = 2 if spec == "logprobs" else None
    if spec == "mtp":
        n_out = 24
        extra["speculative_config"] = {"method": "mtp", "num_speculative_tokens": 2}

    from vllm import LLM, SamplingParams
    from vllm.platforms import current_platform
    # one sequence at a time: both engines then run the same kernels on the same shapes in the
    # same order (whole prompt, then one token per step), so greedy tokens must agree exactly
    llm = LLM(model=d, load_format=load_format, skip_tokenizer_init=True, dtype=cfg["torch_dtype"],
              max_model_len=256, max_num_seqs=seqs, max_num_batched_tokens=budget, block_size=16,
              enforce_eager=fp32, seed=0, enable_prefix_caching=False, tensor_parallel_size=tp,
              gpu_memory_utilization=0.3, **extra, **({} if fp32 else {"kv_cache_memory_bytes": 1 << 30}))
    vcfg = llm.llm_engine.vllm_config
    outs = llm.generate([{"prompt_token_ids": p} for p in prompts],
                        SamplingParams(max_tokens=n_out, temperature=0.0, ignore_eos=True, detokenize=False,
                                       logprobs=want_logprobs),
                        use_tqdm=False)
    via_vllm = [list(o.outputs[0].token_ids) for o in outs]
    lp_info = None
    if want_logprobs:
        # per request: for every output token (its log-probability, its rank, ids of the alternatives)
        lp_info = [[(d[t].logprob, d[t].rank, sorted(d, key=lambda k: d[k].rank)[:want_logprobs])
                    for t, d in zip(o.outputs[0].token_ids, o.outputs[0].logprobs)] for o in outs]
    info = {"platform": type(current_platform).__name__, "worker_cls": vcfg.parallel_config.worker_cls,
            "async_scheduling": bool(vcfg.scheduler_config.async_scheduling)}
    if tp == 1:
        worker = llm.llm_engine.engine_core.engine_core.model_executor.driver_worker.worker
        info["worker"] = type(worker).__name__
        info["runner"] = type(worker.model_runner).__module__ + "." + type(worker.model_runner).__name__
        info["steps"] = dict(worker.steps)
        info["num_vllm_steps"] = sum(v for k, v in worker.steps.items() if k in ("prefill", "decode", "spec_decode"))
        info["graphs"] = len(worker.model_runner.graphs)
        if mode != "cpu":
            from omni_npu_b200 import ops
            info["launches"] = ops.launch_count()
        state = {k: v.detach().clone() for k, v in worker.get_model().state_dict().items()}
        del llm
        from omni_npu_b200 import SamplingParams as SP
        from omni_npu_b200.config import ModelConfig
        from omni_npu_b200.engine.llm import LLM as OwnLLM
        own = OwnLLM(model=ModelConfig.from_hf_dict(cfg), device="cpu" if fp32 else "cuda", max_num_seqs=1,
                     max_num_batched_tokens=64, max_model_len=256, block_size=16, num_gpu_blocks=64, seed=0,
                     enforce_eager=fp32)
        # the comparison engine decodes plainly: it has no draft head to load
        own.engine.worker.get_model().load_state_dict({k: v for k, v in state.items() if not k.startswith("mtp.")})
        res = own.generate(prompts, SP(max_tokens=n_out, temperature=0.0, ignore_eos=True))
        info["standalone"] = [o.output_token_ids for o in res]
    info["via_vllm"] = via_vllm
    info["logprobs"] = lp_info
    print("RESULT " + json.dumps(info), flush=True)


if __name__ == "__main__":
    main()
