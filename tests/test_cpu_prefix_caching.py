"""Automatic prefix caching of the standalone engine: full KV blocks are findable by the hash of
their token prefix, shared between requests by reference count and kept after their last user until
the block is needed again."""
import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import CacheConfig, ModelConfig, SchedulerConfig
from omni_npu_b200.engine.block_manager import BlockPool, chain_block_hashes
from omni_npu_b200.engine.llm import LLM
from omni_npu_b200.engine.request import Request
from omni_npu_b200.engine.scheduler import Scheduler


def _cfg():
    return ModelConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128,
                       vocab_size=97, rope_theta=10000.0, max_position_embeddings=512, dtype=torch.float32)


def test_block_hashes_chain_over_prefixes_and_stop_at_placeholders():
    a = chain_block_hashes(list(range(10)), 4)
    b = chain_block_hashes(list(range(8)) + [50, 51, 52, 53], 4)
    assert len(a) == 2 and len(b) == 3 and a == b[:2]
    c = chain_block_hashes([9] + list(range(1, 8)), 4)
    assert c[0] != a[0] and c[1] != a[1]                     # a different first block changes every later hash
    d = chain_block_hashes([1, 2, 3, 4, 5, -1, 7, 8, 9, 10, 11, 12], 4)
    assert len(d) == 1                                       # a token that is not known yet ends the chain
    d2 = chain_block_hashes([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12], 4, prev=d)
    assert len(d2) == 3 and d2[0] == d[0]                    # ... and the chain resumes once it is


def test_pool_shares_blocks_by_reference_and_evicts_the_oldest_unused_content():
    pool = BlockPool(8, 4, prefix_caching=True)
    hs = chain_block_hashes(list(range(12)), 4)
    a = pool.allocate(3)
    for blk, h in zip(a, hs):
        pool.register(blk, h)
    pool.acquire(a[:2])                                       # a second user of the first two blocks
    pool.free(a)
    assert pool.num_free == 6 and pool.match_prefix(hs) == a  # the third block is unused but still findable
    pool.free(a[:2])
    assert pool.num_free == 8
    got = pool.allocate(6)                                    # five never-used blocks and the content freed first
    assert a[2] in got and a[0] not in got and a[1] not in got
    assert pool.match_prefix(hs) == a[:2]
    pool.free(got)
    assert pool.num_free == 8


def test_scheduler_reuses_a_finished_requests_blocks_for_a_shared_prefix():
    sched = Scheduler(SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=64),
                      CacheConfig(block_size=4, enable_prefix_caching=True), num_blocks=32)
    shared = list(range(1, 15))                               # 14 tokens: three full blocks and a bit
    a = Request("a", shared + [20, 21], SamplingParams(max_tokens=1, ignore_eos=True))
    sched.add_request(a)
    out = sched.schedule()
    assert out.seqs[0].start == 0 and out.seqs[0].num_new_tokens == 16
    blocks_a = list(a.block_ids)
    sched.update_from_output(out, [5])
    assert a.is_finished and sched.pool.num_free == 32
    b = Request("b", shared + [30, 31, 32], SamplingParams(max_tokens=2, ignore_eos=True))
    sched.add_request(b)
    out = sched.schedule()
    # the three full blocks of the shared prefix are taken over; the rest of the prompt is computed
    assert out.seqs[0].start == 12 and out.seqs[0].num_new_tokens == 5
    assert b.block_ids[:3] == blocks_a[:3]
    assert sched.prefix_stats["hit_tokens"] == 12
    sched.update_from_output(out, [6])
    # a request equal to a cached one still computes its last token
    c = Request("c", shared[:12], SamplingParams(max_tokens=1, ignore_eos=True))
    sched.add_request(c)
    out = sched.schedule()
    seq_c = [s for s in out.seqs if s.request is c][0]
    assert seq_c.start == 8 and seq_c.num_new_tokens == 4


def test_engine_tokens_are_unchanged_and_prefill_work_drops():
    g = torch.Generator().manual_seed(11)
    system = torch.randint(1, 97, (37,), generator=g).tolist()
    prompts = [system + torch.randint(1, 97, (n,), generator=g).tolist() for n in (5, 9, 3, 14, 1, 8)]
    sps = [SamplingParams(max_tokens=m, ignore_eos=True) for m in (6, 4, 9, 3, 7, 5)]
    res = {}
    for on in (False, True):
        llm = LLM(model=_cfg(), device="cpu", max_num_seqs=2, max_num_batched_tokens=64, max_model_len=128,
                  block_size=4, num_gpu_blocks=64, seed=3, enable_prefix_caching=on)
        outs = llm.generate(prompts, sps)
        res[on] = ([o.output_token_ids for o in outs], llm.engine.scheduler.prefix_stats["hit_tokens"],
                   llm.engine.scheduler.pool.num_free)
    assert res[True][0] == res[False][0]
    assert res[False][1] == 0 and res[True][1] >= 4 * 36      # later requests take over the 36 cached prompt tokens
    assert res[True][2] == 64


def test_engine_with_asynchronous_scheduling_and_preemption_keeps_tokens():
    g = torch.Generator().manual_seed(12)
    system = torch.randint(1, 97, (18,), generator=g).tolist()
    prompts = [system + torch.randint(1, 97, (n,), generator=g).tolist() for n in (6, 7, 5)]
    sps = [SamplingParams(max_tokens=14, ignore_eos=True) for _ in prompts]
    res = {}
    for on in (False, True):
        llm = LLM(model=_cfg(), device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128,
                  block_size=4, num_gpu_blocks=22, seed=3, enable_prefix_caching=on,
                  additional_config={"async_scheduling": True})
        outs = llm.generate(prompts, sps)
        res[on] = [o.output_token_ids for o in outs]
        assert llm.engine.scheduler.pool.num_free == 22
    assert res[True] == res[False]
