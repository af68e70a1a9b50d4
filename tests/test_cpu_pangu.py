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


# ------------------------------------------------------------------ Pangu Pro MoE V2
def _pro_cfg(sink=16, window=None, v_dim=24):
    return ModelConfig(architecture="PanguProMoEV2ForCausalLM", model_type="pangu_pro_moe_v2", hidden_size=64,
                       num_layers=3, num_heads=4, num_kv_heads=2, head_dim=32, intermediate_size=128,
                       vocab_size=211, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512,
                       rope_neox=False, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
                       num_shared_experts=1, first_k_dense=1, dtype=torch.float32, norm_topk_prob=True,
                       hf_config={"param_sink_number": sink, "param_sink_with_value": True, "v_channels": v_dim,
                                  "qk_rope_dim": 16, "interleaved_sliding_window": window})


def _pro_llm(cfg, seed=4):
    llm = LLM(model=cfg, device="cpu", max_num_seqs=4, max_num_batched_tokens=32, max_model_len=128,
              block_size=8, num_gpu_blocks=64, seed=seed)
    g = torch.Generator().manual_seed(seed)
    for name, p in llm.engine.worker.get_model().named_parameters():
        if "param_sink" in name:
            p.data.copy_(torch.randn(p.shape, generator=g))
    return llm


def test_pangu_pro_sink_blocks_are_reserved_and_filled():
    llm = _pro_llm(_pro_cfg())
    model = llm.engine.worker.get_model()
    assert model.num_reserved_kv_blocks == 3                        # null block + 16 sink tokens / 8
    out = llm.generate([[1, 2, 3, 4, 5]], SamplingParams(max_tokens=3, ignore_eos=True))[0]
    assert len(out.output_token_ids) == 3
    k0, v0 = llm.engine.worker.model_runner.kv_caches[0]
    assert k0.shape[-1] == 32 and v0.shape[-1] == 24                # separate key / value head sizes
    assert float(k0[1:3].abs().sum()) > 0 and float(v0[1:3].abs().sum()) > 0
    attn = model.model.layers[0].self_attn
    # stored sink keys: normalised, rotary lanes de-interleaved
    want = attn.sink_key_layout(attn.k_layernorm(attn.param_sink_key.reshape(-1, 32)).view(16, 2, 32))
    assert torch.allclose(k0[1, :, 0], want[0], atol=1e-6) and torch.allclose(k0[2, :, 7], want[15], atol=1e-6)
    # no request block may collide with the reserved ones
    assert all(b >= 3 for r in llm.engine.scheduler.requests.values() for b in r.block_ids)


def test_pangu_pro_decode_matches_prefill_with_sinks_and_sliding_window():
    for window in (None, [0, 6]):
        llm = _pro_llm(_pro_cfg(window=window))
        g = torch.Generator().manual_seed(2)
        prompts = [torch.randint(0, 211, (n,), generator=g).tolist() for n in (13, 22)]
        fast = llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
        for p, o in zip(prompts, fast):
            toks = list(p)
            for _ in range(6):
                toks.append(llm.generate([toks], SamplingParams(max_tokens=1, ignore_eos=True))[0].output_token_ids[0])
            assert o.output_token_ids == toks[len(p):]


def test_sinks_and_window_change_the_function():
    prompt = [[7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17, 18]]
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    base = _pro_llm(_pro_cfg()).generate(prompt, sp)[0].output_token_ids
    assert _pro_llm(_pro_cfg(sink=0)).generate(prompt, sp)[0].output_token_ids != base
    assert _pro_llm(_pro_cfg(window=[3])).generate(prompt, sp)[0].output_token_ids != base


def test_sink_mask_reference():
    """Window 2 with 3 sink tokens: a query at position p sees keys {0,1,2} and {p-1, p}."""
    from omni_npu_b200.ops import ref
    torch.manual_seed(0)
    n, d = 10, 8
    kc = torch.randn(2, 1, 8, d)
    vc = torch.randn(2, 1, 8, d)
    q = torch.randn(n, d)
    bt = torch.tensor([[0, 1]], dtype=torch.int32)
    out = ref.paged_attention(q, kc, vc, bt, torch.tensor([0, n]), torch.tensor([n]), 1, 1.0, True, 2, False, 3)
    keys = kc.permute(0, 2, 1, 3).reshape(16, d)[:n]
    vals = vc.permute(0, 2, 1, 3).reshape(16, d)[:n]
    for p in (0, 4, 9):
        vis = sorted({0, 1, 2} & set(range(p + 1)) | {k for k in (p - 1, p) if k >= 0})
        w = torch.softmax(q[p] @ keys[vis].t(), -1)
        assert torch.allclose(out[p], w @ vals[vis], atol=1e-5)
