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


def test_redundant_experts_and_periodic_rebalancing_keep_tokens_identical():
    """Two spare expert slots per MoE layer, placement re-planned every 3 engine steps: the generated
    tokens equal those of the plain model (replicas hold the same weights; moves happen between steps)."""
    cfg = _cfg()
    common = dict(device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=16,
                  num_gpu_blocks=64, seed=7)
    plain = LLM(model=cfg, **common)
    red = LLM(model=cfg, num_redundant_experts=2, eplb_step_interval=3, **common)
    src = dict(plain.engine.worker.get_model().named_parameters())
    for name, p in red.engine.worker.get_model().named_parameters():
        if name.endswith((".w13", ".w2")):
            slots = red.engine.worker.get_model().get_submodule(name.rsplit(".", 1)[0]).eplb.placement()
            p.data.copy_(src[name].data[slots])          # physical slot s holds logical expert slots[s]
        else:
            p.data.copy_(src[name].data)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (19, 30)]
    want = [o.output_token_ids for o in plain.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
    got = [o.output_token_ids for o in red.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
    assert got == want
    assert red.engine.stats.get("eplb_moves", 0) >= 0 and red.engine.stats["steps"] >= 6
    moe = [m for m in red.engine.worker.get_model().modules() if getattr(m, "eplb", None) is not None]
    assert moe and all(m.w13.shape[0] == 10 for m in moe)


def test_fp8_checkpoint_experts_and_linears_load_with_their_block_scales(tmp_path):
    """A DeepSeek-style checkpoint in block-scaled e4m3 (weight + weight_scale_inv per projection and per
    expert) generates the tokens of the same model with the de-quantised weights."""
    import json
    from safetensors.torch import save_file
    from omni_npu_b200.layers.quant_fp8 import quantize_weight_block
    from omni_npu_b200.ops import ref
    cfg = _cfg(hidden_size=128, moe_intermediate_size=128, intermediate_size=256)
    base = LLM(model=cfg, device="cpu", max_num_seqs=2, max_num_batched_tokens=64, max_model_len=128,
               block_size=16, num_gpu_blocks=32, seed=5)
    model = base.engine.worker.get_model()
    state, deq = {}, {}
    for name, p in model.named_parameters():
        t = p.data
        if name.endswith((".w13", ".w2")):
            # FusedMoE keeps experts stacked (gate/up interleaved): write them per expert like a checkpoint
            prefix = name.rsplit(".", 1)[0]
            inter = t.shape[1] // 2 if name.endswith(".w13") else None
            for e in range(t.shape[0]):
                if inter is not None:
                    j = torch.arange(inter)
                    parts = {"gate_proj": t[e][(j // 8) * 16 + j % 8], "up_proj": t[e][(j // 8) * 16 + 8 + j % 8]}
                else:
                    parts = {"down_proj": t[e]}
                for proj, w in parts.items():
                    wq, ws = quantize_weight_block(w)
                    state[f"{prefix}.experts.{e}.{proj}.weight"] = wq
                    state[f"{prefix}.experts.{e}.{proj}.weight_scale_inv"] = ws
                    deq[f"{prefix}.experts.{e}.{proj}.weight"] = ref.dequant_fp8_block(wq, ws)
        else:
            state[name] = t.clone()
            deq[name] = t.clone()
    hf = {"architectures": ["DeepseekV3ForCausalLM"], "model_type": "deepseek_v3"}
    # reference: the same model with the de-quantised expert weights loaded back in
    want_model = LLM(model=cfg, device="cpu", max_num_seqs=2, max_num_batched_tokens=64, max_model_len=128,
                     block_size=16, num_gpu_blocks=32, seed=5)
    want_model.engine.worker.get_model().load_weights(deq.items())
    qcfg = _cfg(hidden_size=128, moe_intermediate_size=128, intermediate_size=256, quant_method="fp8")
    q = LLM(model=qcfg, device="cpu", max_num_seqs=2, max_num_batched_tokens=64, max_model_len=128,
            block_size=16, num_gpu_blocks=32, seed=5)
    qm = q.engine.worker.get_model()
    # the constructor already expanded the (randomly initialised) experts; give them back their
    # checkpoint storage, as a model that loads a real checkpoint has it before the post-load hooks run
    for m in qm.modules():
        if getattr(m, "quant", None) == "fp8-expanded":
            m.w13 = torch.nn.Parameter(torch.empty(m.w13.shape, dtype=torch.float8_e4m3fn), requires_grad=False)
            m.w2 = torch.nn.Parameter(torch.empty(m.w2.shape, dtype=torch.float8_e4m3fn), requires_grad=False)
            m.quant = "fp8"
    # dense projections of the fp8 model are block-scaled too: quantise the reference's dense weights for it
    qstate = {}
    for name, t in state.items():
        qstate[name] = t
    for name, p in qm.named_parameters():
        if name.endswith(".weight_scale_inv") and ".experts." not in name and name not in qstate:
            wname = name[: -len("_scale_inv")]
            src = dict(model.named_parameters())[wname].data
            wq, ws = quantize_weight_block(src)
            qstate[wname], qstate[name] = wq, ws
            deq[wname] = ref.dequant_fp8_block(wq, ws)
    want_model.engine.worker.get_model().load_weights(deq.items())
    qm.load_weights(qstate.items())
    for root in (qm, want_model.engine.worker.get_model()):      # derived tensors (absorbed MLA, expert expansion)
        for m in root.modules():
            hook = getattr(m, "process_weights_after_loading", None)
            if hook is not None and m is not root:
                hook()
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (17, 25)]
    want = [o.output_token_ids for o in want_model.generate(prompts, SamplingParams(max_tokens=5, ignore_eos=True))]
    got = [o.output_token_ids for o in q.generate(prompts, SamplingParams(max_tokens=5, ignore_eos=True))]
    assert got == want
