"""openPangu Ultra MoE on CPU: sandwich-norm decoder layer against a hand-written
composition of its parts, and decode/prefill consistency of the whole model."""
import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import ModelConfig
from omni_npu_b200.engine.llm import LLM


def _cfg(sandwich=True):
    return ModelConfig(architecture="PanguUltraMoEForCausalLM", model_type="pangu_ultra_moe", hidden_size=128,
                       num_layers=3, num_heads=4, num_kv_heads=4, head_dim=48, intermediate_size=256, vocab_size=512,
                       rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512, rope_neox=False,
                       num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, num_shared_experts=1,
                       first_k_dense=1, use_mla=True, q_lora_rank=48, kv_lora_rank=512, qk_nope_head_dim=32,
                       qk_rope_head_dim=64, v_head_dim=32, dtype=torch.float32, norm_topk_prob=True,
                       routed_scaling_factor=2.5,
                       hf_config={"sandwich_norm": sandwich, "router_enable_expert_bias": True})


def test_pangu_ultra_routing_config_and_sandwich_layers():
    llm = LLM(model=_cfg(), device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128,
              block_size=16, num_gpu_blocks=64, seed=7)
    model = llm.engine.worker.get_model()
    assert model.config.scoring_func == "sigmoid" and model.config.n_group == 1 and model.config.router_bias
    layer = model.model.layers[1]
    assert layer.sandwich_norm and hasattr(layer, "pre_mlp_layernorm") and hasattr(layer, "post_mlp_layernorm")
    assert hasattr(layer.mlp, "e_score_correction_bias")
    # checkpoint names: both spellings of the router bias land on the same parameter
    b = torch.arange(8, dtype=torch.float32)
    loaded = model.load_weights([("model.layers.1.mlp.gate.bias", b),
                                 ("model.layers.2.mlp.gate.e_score_correction_bias", b + 1)])
    assert torch.equal(model.model.layers[1].mlp.e_score_correction_bias.data, b)
    assert torch.equal(model.model.layers[2].mlp.e_score_correction_bias.data, b + 1) and len(loaded) == 2


def test_pangu_ultra_decode_matches_prefill():
    for sandwich in (True, False):
        llm = LLM(model=_cfg(sandwich), device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128,
                  block_size=16, num_gpu_blocks=64, seed=9)
        g = torch.Generator().manual_seed(1)
        for name, p in llm.engine.worker.get_model().named_parameters():
            if name.endswith("e_score_correction_bias"):
                p.data.copy_(torch.randn(p.shape, generator=g) * 0.1)
            if "layernorm" in name:                      # make the extra norms matter
                p.data.copy_(1.0 + 0.3 * torch.randn(p.shape, generator=g))
        prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (19, 33)]
        fast = llm.generate(prompts, SamplingParams(max_tokens=5, ignore_eos=True))
        for p, o in zip(prompts, fast):
            toks = list(p)
            for _ in range(5):
                toks.append(llm.generate([toks], SamplingParams(max_tokens=1, ignore_eos=True))[0].output_token_ids[0])
            assert o.output_token_ids == toks[len(p):]


def test_sandwich_norm_changes_the_function():
    outs = []
    for sandwich in (True, False):
        llm = LLM(model=_cfg(sandwich), device="cpu", max_num_seqs=2, max_num_batched_tokens=64, max_model_len=128,
                  block_size=16, num_gpu_blocks=32, seed=9)
        outs.append(llm.generate([[5, 9, 200, 31, 7, 7, 100]], SamplingParams(max_tokens=8, ignore_eos=True))[0]
                    .output_token_ids)
    assert outs[0] != outs[1]
