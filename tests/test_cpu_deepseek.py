"""DeepSeek-style models on CPU: the decode path (absorbed MLA over the latent
cache, routed experts) must continue a sequence exactly as repeated prefills of
the growing sequence (non-absorbed path) do."""
import pytest
import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import ModelConfig
from omni_npu_b200.engine.llm import LLM


def _cfg(**kw):
    base = dict(architecture="DeepseekV3ForCausalLM", model_type="deepseek_v3", hidden_size=128, num_layers=3,
                num_heads=4, num_kv_heads=4, head_dim=48, intermediate_size=256, vocab_size=512,
                rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512, rope_neox=False,
                num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, num_shared_experts=1,
                first_k_dense=1, use_mla=True, q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=32,
                qk_rope_head_dim=64, v_head_dim=32, dtype=torch.float32)
    base.update(kw)
    return ModelConfig(**base)


def _generate_by_prefill_only(llm, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        out = llm.generate([toks], SamplingParams(max_tokens=1, ignore_eos=True))[0]
        toks.append(out.output_token_ids[0])
    return toks[len(prompt):]


@pytest.mark.parametrize("variant", ["v2_lite", "v3", "v32_sparse"])
def test_decode_path_matches_prefill_path(variant):
    kw = {}
    if variant == "v3":
        kw = dict(q_lora_rank=48, scoring_func="sigmoid", n_group=4, topk_group=2, router_bias=True,
                  norm_topk_prob=True, routed_scaling_factor=2.5)
    if variant == "v32_sparse":
        kw = dict(architecture="DeepseekV32ForCausalLM", q_lora_rank=48, scoring_func="sigmoid",
                  norm_topk_prob=True, index_topk=12, index_n_heads=4, index_head_dim=128)
    cfg = _cfg(**kw)
    llm = LLM(model=cfg, device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128,
              block_size=16, num_gpu_blocks=64, seed=7)
    # make routing / sparse selection non-trivial: random (not constant) biases
    g = torch.Generator().manual_seed(0)
    for name, p in llm.engine.worker.get_model().named_parameters():
        if name.endswith("e_score_correction_bias"):
            p.data.copy_(torch.randn(p.shape, generator=g) * 0.1)
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (21, 34)]
    fast = llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
    for p, o in zip(prompts, fast):
        assert o.output_token_ids == _generate_by_prefill_only(llm, p, 6)
