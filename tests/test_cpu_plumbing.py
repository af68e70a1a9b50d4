"""End-to-end plumbing on CPU: tiny Llama (2 layers, hidden 256, 4 heads / 2 KV
heads, FFN 512, vocab 1024, fp32), 4 prompts of 32 tokens, 16 greedy tokens,
compared token for token against a plain PyTorch implementation."""
import os
import tempfile

import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import tiny_llama
from omni_npu_b200.engine.llm import LLM, build_engine_config

import reference_llama as refm


def _save(weights, cfg, d):
    import json
    from safetensors.torch import save_file
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump({"architectures": ["LlamaForCausalLM"], "model_type": "llama",
                   "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_layers,
                   "num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_kv_heads,
                   "head_dim": cfg.head_dim, "intermediate_size": cfg.intermediate_size,
                   "vocab_size": cfg.vocab_size, "rms_norm_eps": cfg.rms_norm_eps,
                   "rope_theta": cfg.rope_theta, "max_position_embeddings": 2048,
                   "torch_dtype": "float32"}, f)


def test_tiny_llama_greedy_matches_plain_pytorch():
    cfg = tiny_llama()
    weights = refm.make_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (32,), generator=g).tolist() for _ in range(4)]
    with tempfile.TemporaryDirectory() as d:
        _save(weights, cfg, d)
        llm = LLM(model=d, device="cpu", max_num_seqs=4, max_num_batched_tokens=64,
                  max_model_len=256, block_size=16, dtype="float32")
        outs = llm.generate(prompts, SamplingParams(max_tokens=16, temperature=0.0, ignore_eos=True))
    for p, o in zip(prompts, outs):
        want = refm.greedy_generate(weights, cfg, p, 16)
        assert o.output_token_ids == want
        assert o.finished and o.finish_reason == "length"


def test_chunked_prefill_and_preemption_keep_tokens_identical():
    cfg = tiny_llama()
    weights = refm.make_weights(cfg, seed=1)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (40, 7, 33, 19, 64)]
    with tempfile.TemporaryDirectory() as d:
        _save(weights, cfg, d)
        # 24-token budget forces chunked prefill; 14 blocks of 16 force preemption
        llm = LLM(model=d, device="cpu", max_num_seqs=3, max_num_batched_tokens=24,
                  max_model_len=128, block_size=16, num_gpu_blocks=14, dtype="float32")
        outs = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.output_token_ids == refm.greedy_generate(weights, cfg, p, 12)
