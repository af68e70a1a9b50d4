"""Asynchronous decode scheduling: step n + 1 is launched before the tokens of step n are read.
The generated tokens must be exactly those of the synchronous engine, including requests that end on
an EOS token (one surplus step is computed and discarded), length caps, preemption and late arrivals."""
import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import ModelConfig
from omni_npu_b200.engine.llm import LLM


def _cfg():
    return ModelConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128,
                       vocab_size=97, rope_theta=10000.0, max_position_embeddings=512, dtype=torch.float32)


def _run(async_on, prompts, sps, eos=None, **kw):
    cfg = _cfg()
    cfg.eos_token_id = eos
    args = dict(device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=4,
                num_gpu_blocks=64, seed=3, additional_config={"async_scheduling": async_on})
    args.update(kw)
    llm = LLM(model=cfg, **args)
    outs = llm.generate(prompts, sps)
    return llm, [(o.output_token_ids, o.finish_reason) for o in outs]


def test_tokens_equal_the_synchronous_engine_with_mixed_lengths():
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(1, 97, (n,), generator=g).tolist() for n in (5, 17, 9, 30, 3, 12)]   # 6 requests, 4 slots
    sps = [SamplingParams(max_tokens=m, ignore_eos=True) for m in (1, 7, 12, 3, 9, 2)]
    sync_llm, want = _run(False, prompts, sps)
    async_llm, got = _run(True, prompts, sps)
    assert got == want
    assert async_llm.engine._inflight is None and not async_llm.engine.has_unfinished_requests()
    assert async_llm.engine.stats["output_tokens"] >= sum(len(t) for t, _ in got) - len(prompts)
    assert async_llm.engine.scheduler.pool.num_free == 64            # every block came back


def test_requests_ending_on_eos_drop_the_surplus_step():
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(1, 97, (n,), generator=g).tolist() for n in (6, 11, 8)]
    sps = [SamplingParams(max_tokens=20) for _ in prompts]
    _, free_run = _run(False, prompts, [SamplingParams(max_tokens=20, ignore_eos=True)] * 3)
    eos = free_run[0][0][4]                                           # a token the first request emits at step 5
    _, want = _run(False, prompts, sps, eos=eos)
    _, got = _run(True, prompts, sps, eos=eos)
    assert got == want
    assert want[0][1] == "stop" and len(want[0][0]) <= 5 and want[0][0][-1] == eos


def test_preemption_while_a_step_is_in_flight():
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(1, 97, (n,), generator=g).tolist() for n in (14, 13, 15)]
    sps = [SamplingParams(max_tokens=14, ignore_eos=True) for _ in prompts]
    kw = dict(num_gpu_blocks=14)                                      # too few blocks for three growing sequences
    sync_llm, want = _run(False, prompts, sps, **kw)
    async_llm, got = _run(True, prompts, sps, **kw)
    assert got == want
    assert async_llm.engine.scheduler.num_preemptions > 0 and not async_llm.engine.scheduler.requests


def test_abort_while_a_step_is_in_flight_leaves_the_other_request_intact():
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(1, 97, (n,), generator=g).tolist() for n in (9, 13)]
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    _, want = _run(False, prompts, [sp, sp])
    cfg = _cfg()
    llm = LLM(model=cfg, device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=4,
              num_gpu_blocks=64, seed=3, additional_config={"async_scheduling": True})
    eng = llm.engine
    a = eng.add_request(prompts[0], sp)
    b = eng.add_request(prompts[1], sp)
    outs = []
    for _ in range(4):                                   # prefill, then a few decode steps: one is in flight now
        outs += eng.step()
    assert eng._inflight is not None
    eng.abort_request(a)
    while eng.has_unfinished_requests():
        outs += eng.step()
    done = {o.request_id: o for o in outs}
    assert done[b].output_token_ids == want[1][0] and done[b].finish_reason == "length"
    assert a not in done or done[a].finish_reason == "abort"
    assert eng.scheduler.pool.num_free == 64 and eng._inflight is None
