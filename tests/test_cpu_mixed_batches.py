"""Mixed batches: decoding requests take their next token inside the prefill steps of other
requests.  The tokens must be those of the engine that runs prefill and decode steps apart, fewer
steps must be needed, and a decoding request must never wait for a whole prompt."""
import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import CacheConfig, ModelConfig, SchedulerConfig
from omni_npu_b200.engine.llm import LLM
from omni_npu_b200.engine.request import Request
from omni_npu_b200.engine.scheduler import Scheduler


def _cfg():
    return ModelConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128,
                       vocab_size=97, rope_theta=10000.0, max_position_embeddings=512, dtype=torch.float32)


def _run(mixed, prompts, sps, async_on=False, **kw):
    args = dict(device="cpu", max_num_seqs=3, max_num_batched_tokens=24, max_model_len=128, block_size=4,
                num_gpu_blocks=96, seed=3, enable_mixed_batches=mixed,
                additional_config={"async_scheduling": async_on})
    args.update(kw)
    llm = LLM(model=_cfg(), **args)
    outs = llm.generate(prompts, sps)
    return llm, [(o.output_token_ids, o.finish_reason) for o in outs]


def _workload():
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(1, 97, (n,), generator=g).tolist() for n in (5, 40, 9, 30, 3, 21, 17)]
    sps = [SamplingParams(max_tokens=m, ignore_eos=True) for m in (6, 9, 12, 3, 10, 2, 8)]
    return prompts, sps


def test_tokens_equal_the_engine_with_separate_steps_and_fewer_steps_are_needed():
    prompts, sps = _workload()
    apart, want = _run(False, prompts, sps)
    mixed, got = _run(True, prompts, sps)
    assert got == want
    assert mixed.engine.stats["steps"] < apart.engine.stats["steps"]
    assert mixed.engine.scheduler.pool.num_free == apart.engine.scheduler.pool.num_free


def test_tokens_equal_with_asynchronous_scheduling_on():
    prompts, sps = _workload()
    _, want = _run(False, prompts, sps)
    llm, got = _run(True, prompts, sps, async_on=True)
    assert got == want
    assert llm.engine._inflight is None and not llm.engine.has_unfinished_requests()


def test_scheduler_puts_the_riders_first_and_charges_them_to_the_token_budget():
    sched = Scheduler(SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=16, max_model_len=64,
                                      enable_mixed_batches=True), CacheConfig(block_size=4), num_blocks=64)
    a = Request("a", list(range(1, 7)), SamplingParams(max_tokens=8, ignore_eos=True))
    sched.add_request(a)
    out = sched.schedule()
    assert out.kind == "prefill" and out.num_decode_seqs == 0
    sched.update_from_output(out, [11])
    b = Request("b", list(range(1, 31)), SamplingParams(max_tokens=4, ignore_eos=True))
    sched.add_request(b)
    out = sched.schedule()
    # one row for the decoding request, the other fifteen tokens of the budget for the new prompt
    assert out.kind == "prefill" and out.num_decode_seqs == 1
    assert [(s.request.request_id, s.num_new_tokens, s.samples) for s in out.seqs] == [("a", 1, True), ("b", 15, False)]
    assert out.num_tokens == 16
    sched.update_from_output(out, [12, 0])
    assert a.output_token_ids == [11, 12] and b.output_token_ids == []
    out = sched.schedule()
    assert [(s.request.request_id, s.num_new_tokens, s.samples) for s in out.seqs] == [("a", 1, True), ("b", 15, True)]
    sched.update_from_output(out, [13, 21])
    out = sched.schedule()
    assert out.kind == "decode" and out.num_decode_seqs == 0 and len(out.seqs) == 2


def test_latent_attention_model_riders_take_the_absorbed_decode_path():
    """Mixed batches of a small latent-attention (MLA) + MoE model: the riders' rows go through the
    latent-space decode path, the prompt rows through the non-absorbed prefill; tokens equal the
    engine with separate steps."""
    from omni_npu_b200.attention.mla import MLAAttention
    model = ModelConfig(architecture="DeepseekV2ForCausalLM", model_type="deepseek_v2", hidden_size=128, num_layers=3,
                        num_heads=4, num_kv_heads=4, head_dim=48, intermediate_size=256, vocab_size=512,
                        rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512, rope_neox=False,
                        num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, num_shared_experts=1,
                        first_k_dense=1, use_mla=True, q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=32,
                        qk_rope_head_dim=64, v_head_dim=32, dtype=torch.float32)
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(1, 512, (n,), generator=g).tolist() for n in (5, 40, 9, 30, 3, 21)]
    sps = [SamplingParams(max_tokens=m, ignore_eos=True) for m in (6, 9, 12, 3, 10, 2)]
    outs, calls = {}, {}
    for mixed in (False, True):
        llm = LLM(model=model, device="cpu", max_num_seqs=3, max_num_batched_tokens=24, max_model_len=128,
                  block_size=4, num_gpu_blocks=96, seed=3, enable_mixed_batches=mixed)
        seen = []
        real = MLAAttention._decode

        def spy(self, q, q_pe, cache, md, topk, _seen=seen, _real=real):
            _seen.append((md.is_prefill, q.shape[0]))
            return _real(self, q, q_pe, cache, md, topk)
        MLAAttention._decode = spy
        try:
            outs[mixed] = [o.output_token_ids for o in llm.generate(prompts, sps)]
        finally:
            MLAAttention._decode = real
        calls[mixed] = llm.engine.stats["steps"]
    assert outs[True] == outs[False]
    assert calls[True] < calls[False]
