"""Qwen3-MoE from an HF-style checkpoint on CPU: one process, tensor parallel with the
token-sharded residual stream, the same with the head <-> sequence all-to-all after
attention, and two pipeline stages must all generate the same tokens."""
import json
import os
import tempfile

import torch

from dist_utils import run_ranks
from omni_npu_b200 import SamplingParams
from omni_npu_b200.engine.llm import LLM

HF = {"architectures": ["Qwen3MoeForCausalLM"], "model_type": "qwen3_moe", "hidden_size": 64,
      "num_hidden_layers": 3, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
      "intermediate_size": 128, "vocab_size": 256, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
      "max_position_embeddings": 1024, "torch_dtype": "float32", "num_experts": 4, "num_experts_per_tok": 2,
      "moe_intermediate_size": 32, "norm_topk_prob": True}


def _checkpoint(d: str, seed: int = 0, hf: dict = None) -> None:
    """A random HF-style Qwen3-MoE checkpoint of the shape ``hf`` (default: the small CPU shape)."""
    from safetensors.torch import save_file
    HF = hf or globals()["HF"]
    g = torch.Generator().manual_seed(seed)

    def r(*shape, std=0.05):
        return torch.randn(*shape, generator=g) * std

    h, nh, nk, hd, v = HF["hidden_size"], HF["num_attention_heads"], HF["num_key_value_heads"], HF["head_dim"], \
        HF["vocab_size"]
    w = {"model.embed_tokens.weight": r(v, h, std=0.5), "model.norm.weight": torch.ones(h), "lm_head.weight": r(v, h)}
    for i in range(HF["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = 1 + r(h)
        w[p + "post_attention_layernorm.weight"] = 1 + r(h)
        w[p + "self_attn.q_proj.weight"] = r(nh * hd, h, std=0.2)
        w[p + "self_attn.k_proj.weight"] = r(nk * hd, h, std=0.2)
        w[p + "self_attn.v_proj.weight"] = r(nk * hd, h, std=0.2)
        w[p + "self_attn.o_proj.weight"] = r(h, nh * hd, std=0.2)
        w[p + "self_attn.q_norm.weight"] = 1 + r(hd)
        w[p + "self_attn.k_norm.weight"] = 1 + r(hd)
        w[p + "mlp.gate.weight"] = r(HF["num_experts"], h, std=0.5)
        for e in range(HF["num_experts"]):
            q = p + f"mlp.experts.{e}."
            w[q + "gate_proj.weight"] = r(HF["moe_intermediate_size"], h, std=0.2)
            w[q + "up_proj.weight"] = r(HF["moe_intermediate_size"], h, std=0.2)
            w[q + "down_proj.weight"] = r(h, HF["moe_intermediate_size"], std=0.2)
    dt = torch.bfloat16 if HF.get("torch_dtype") == "bfloat16" else torch.float32
    save_file({k: t.to(dt).contiguous() for k, t in w.items()}, os.path.join(d, "model.safetensors"))
    json.dump(HF, open(os.path.join(d, "config.json"), "w"))


def test_token_sharded_stream_and_head_to_sequence_exchange_match_one_process():
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 256, (n,), generator=g).tolist() for n in (20, 33, 9)]
    results = {}
    with tempfile.TemporaryDirectory() as d:
        os.makedirs(os.path.join(d, "model"))
        _checkpoint(os.path.join(d, "model"))
        json.dump(prompts, open(os.path.join(d, "prompts.json"), "w"))
        llm = LLM(model=os.path.join(d, "model"), device="cpu", dtype="float32", max_num_seqs=4,
                  max_num_batched_tokens=64, max_model_len=256, block_size=16, num_gpu_blocks=64)
        want = [o.output_token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))]
        assert len({tuple(t) for t in want}) == 3          # not a degenerate model
        open(os.path.join(d, "sequence_parallel"), "w").close()
        results["sp"] = run_ranks("tp_engine", 2, d)
        json.dump({"attn_output_all_to_all": True}, open(os.path.join(d, "additional_config.json"), "w"))
        results["a2a"] = run_ranks("tp_engine", 2, d)
        os.remove(os.path.join(d, "additional_config.json"))
        os.remove(os.path.join(d, "sequence_parallel"))
        open(os.path.join(d, "pipeline_parallel"), "w").write("2")
        results["pp"] = run_ranks("tp_engine", 2, d)
    assert "HeadToSequenceAttention" in results["a2a"][0]["attention_modules"]
    assert "HeadToSequenceAttention" not in results["sp"][0]["attention_modules"]
    assert "HeadToSequenceAttention" not in results["pp"][0]["attention_modules"]
    for kind, res in results.items():
        assert res[0]["tokens"] == want, kind
        assert res[1]["tokens"] == want, kind


def test_data_parallel_replicas_with_shared_experts_step_in_lock_step():
    """Two data-parallel replicas, experts sharded over both: the replica with less work keeps
    the expert exchanges alive with dummy batches and every request decodes as in one process."""
    g = torch.Generator().manual_seed(3)
    per_rank = [[torch.randint(0, 256, (n,), generator=g).tolist() for n in (20, 70, 9)],
                [torch.randint(0, 256, (5,), generator=g).tolist()]]
    with tempfile.TemporaryDirectory() as d:
        os.makedirs(os.path.join(d, "model"))
        _checkpoint(os.path.join(d, "model"), seed=4)
        json.dump(per_rank, open(os.path.join(d, "prompts.json"), "w"))
        llm = LLM(model=os.path.join(d, "model"), device="cpu", dtype="float32", max_num_seqs=4,
                  max_num_batched_tokens=64, max_model_len=256, block_size=16, num_gpu_blocks=64)
        sp = SamplingParams(max_tokens=10, ignore_eos=True)
        want = [[o.output_token_ids for o in llm.generate(p, sp)] for p in per_rank]
        res = run_ranks("dp_engine", 2, d)
    assert res[0]["tokens"] == want[0] and res[1]["tokens"] == want[1]
    assert res[0]["local_experts"] == HF["num_experts"] // 2
    assert res[0]["dummy_steps"] == 0 and res[1]["dummy_steps"] > 0
    assert res[0]["steps"] == res[1]["steps"]
