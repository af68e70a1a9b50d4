"""Scheduler and KV block pool: admission, chunked prefill, decode batching, preemption, draft
tokens, reserved blocks and delayed release (host-side logic, no model)."""
import pytest

from omni_npu_b200.config import CacheConfig, SchedulerConfig
from omni_npu_b200.engine.block_manager import BlockPool
from omni_npu_b200.engine.request import Request, RequestStatus, SamplingParams
from omni_npu_b200.engine.scheduler import Scheduler


def _sched(num_blocks=16, block=4, seqs=4, budget=16, chunked=True, max_len=64, reserved=0):
    return Scheduler(SchedulerConfig(max_num_seqs=seqs, max_num_batched_tokens=budget, max_model_len=max_len,
                                     enable_chunked_prefill=chunked), CacheConfig(block_size=block), num_blocks, reserved)


def _req(rid, n, max_tokens=4):
    return Request(rid, list(range(1, n + 1)), SamplingParams(max_tokens=max_tokens, ignore_eos=True))


def test_block_pool_lifo_reserved_and_parking():
    pool = BlockPool(8, 4, num_reserved=2)
    assert pool.num_free == 6 and pool.blocks_needed(9) == 3 and pool.blocks_needed(9, have=2) == 1
    a = pool.allocate(3)
    assert a == [2, 3, 4] and all(b >= 2 for b in a)              # reserved blocks 0, 1 are never handed out
    assert not pool.can_allocate(4) and pool.can_allocate(3)
    with pytest.raises(RuntimeError):
        pool.allocate(4)
    pool.park("r", a, delay_s=10.0, now=100.0)
    assert pool.num_parked == 1 and pool.num_free == 3
    assert pool.expire_parked(now=105.0) == [] and pool.num_free == 3
    assert pool.expire_parked(now=111.0) == ["r"] and pool.num_free == 6
    assert not pool.release_parked("r")
    assert pool.allocate(1) == [2]                                # most recently freed first
    assert 0.0 < pool.usage < 1.0
    with pytest.raises(ValueError):
        BlockPool(2, 4, num_reserved=2)


def test_prefill_is_chunked_to_the_token_budget_then_decodes():
    s = _sched(budget=8)
    s.add_request(_req("a", 13))
    o = s.schedule()
    assert o.kind == "prefill" and [(q.start, q.num_new_tokens, q.samples) for q in o.seqs] == [(0, 8, False)]
    s.update_from_output(o, [0])
    o = s.schedule()
    assert [(q.start, q.num_new_tokens, q.samples) for q in o.seqs] == [(8, 5, True)]
    s.update_from_output(o, [42])
    req = s.requests["a"]
    assert req.output_token_ids == [42] and len(req.block_ids) == 4
    o = s.schedule()
    assert o.kind == "decode" and o.num_tokens == 1 and o.seqs[0].start == 13
    for tok in (43, 44, 45):
        s.update_from_output(o, [tok])
        o = s.schedule()
    assert req.status == RequestStatus.FINISHED_LENGTH_CAPPED and not s.has_unfinished()
    assert s.pool.num_free == 16 and o.kind == "idle" and o.finished_req_ids == ["a"]


def test_without_chunking_a_prompt_waits_for_a_step_it_fits_in():
    s = _sched(budget=8, chunked=False)
    s.add_request(_req("a", 6))
    s.add_request(_req("b", 6))
    o = s.schedule()
    assert [q.request.request_id for q in o.seqs] == ["a"] and o.num_tokens == 6
    s.update_from_output(o, [9])
    o = s.schedule()
    assert o.kind == "prefill" and [q.request.request_id for q in o.seqs] == ["b"]


def test_admission_respects_max_num_seqs_and_batches_decodes():
    s = _sched(seqs=2, budget=32, num_blocks=32)
    for name in "abc":
        s.add_request(_req(name, 3))
    o = s.schedule()
    assert sorted(q.request.request_id for q in o.seqs) == ["a", "b"] and len(s.waiting) == 1
    s.update_from_output(o, [7, 7])
    o = s.schedule()
    assert o.kind == "decode" and len(o.seqs) == 2           # c waits for a free slot
    s.abort_request("a")
    assert s.requests.get("a") is None or s.requests["a"].status == RequestStatus.FINISHED_ABORTED
    o = s.schedule()
    assert o.kind == "prefill" and [q.request.request_id for q in o.seqs] == ["c"]


def test_decode_preempts_the_newest_request_when_blocks_run_out():
    s = _sched(num_blocks=4, block=4, budget=16)
    s.add_request(_req("old", 8, max_tokens=8))
    s.add_request(_req("new", 7, max_tokens=8))
    o = s.schedule()
    s.update_from_output(o, [1, 1])            # both prompts in: 2 + 2 blocks, pool empty
    assert s.pool.num_free == 0
    o = s.schedule()                           # "old" needs a 3rd block for token 9 -> "new" is preempted
    assert o.preempted == ["new"] and [q.request.request_id for q in o.seqs] == ["old"]
    new = s.requests["new"]
    assert new.status == RequestStatus.PREEMPTED or new in s.waiting
    assert new.num_computed_tokens == 0 and new.block_ids == [] and new.num_preemptions == 1


def test_draft_tokens_are_scheduled_for_verification_and_accounted():
    s = _sched(budget=32, num_blocks=32)
    s.add_request(_req("a", 5, max_tokens=10))
    o = s.schedule()
    s.update_from_output(o, [11], drafts=[[12, 13]])
    o = s.schedule()
    assert o.kind == "spec_decode" and o.seqs[0].spec_token_ids == [12, 13] and o.num_tokens == 3
    s.update_from_output(o, [[12, 99]])        # first draft accepted, second replaced by the target's token
    req = s.requests["a"]
    assert req.output_token_ids == [11, 12, 99] and s.spec_stats == {"drafted": 2, "accepted": 1}
    assert req.num_computed_tokens == 5 + 2    # prompt + [11, 12] have valid KV; 99 is fed next step


def test_reserved_blocks_stay_out_of_the_free_list():
    s = _sched(num_blocks=6, reserved=2)
    s.add_request(_req("a", 16, max_tokens=1))
    o = s.schedule()
    assert o.kind == "prefill" and all(b >= 2 for b in s.requests["a"].block_ids)


def test_half_computed_prompt_is_never_sampled_when_blocks_run_out():
    """A chunked prompt whose next chunk finds no free blocks must not fall through to the decode
    branch: no step may sample for it before its whole prompt is in the cache."""
    s = Scheduler(SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256,
                                  enable_chunked_prefill=True), CacheConfig(block_size=16), 10)
    b = _req("B", 64, max_tokens=64)
    s.add_request(b)
    o = s.schedule()
    s.update_from_output(o, [7])                     # B: 4 blocks, decoding
    a = _req("A", 128, max_tokens=8)
    s.add_request(a)
    sampled_early = []
    for _ in range(600):
        o = s.schedule()
        if o.kind == "idle":
            break
        for q in o.seqs:
            r = q.request
            if q.samples and q.start + q.num_new_tokens < r.num_tokens:
                sampled_early.append((r.request_id, q.start, q.num_new_tokens))
            if o.kind == "decode":
                assert r.num_tokens - r.num_computed_tokens == 1, (r.request_id, q.start)
        s.update_from_output(o, [5] * len(o.seqs))
        if not s.has_unfinished():
            break
    assert not sampled_early
    assert a.is_finished and b.is_finished and not s.requests       # finished requests leave the scheduler's table
    assert len(a.output_token_ids) == 8 and len(b.output_token_ids) == 64
    assert s.pool.num_free == 10


def test_priority_policy_orders_admission_and_picks_the_least_urgent_victim():
    from omni_npu_b200.config import CacheConfig, SchedulerConfig
    from omni_npu_b200.engine.request import Request, SamplingParams
    from omni_npu_b200.engine.scheduler import Scheduler
    sched = Scheduler(SchedulerConfig(max_num_seqs=2, max_num_batched_tokens=64, max_model_len=64, policy="priority"),
                      CacheConfig(block_size=4), num_blocks=64)
    for rid, prio, t in (("late-urgent", 0, 3.0), ("early-relaxed", 5, 1.0), ("early-urgent", 0, 2.0), ("mid", 2, 2.5)):
        sched.add_request(Request(rid, [1, 2, 3, 4, 5], SamplingParams(max_tokens=4, ignore_eos=True, priority=prio),
                                  arrival_time=t))
    assert [r.request_id for r in sched.waiting] == ["early-urgent", "late-urgent", "mid", "early-relaxed"]
    out = sched.schedule()                                       # two sequence slots: the two urgent ones
    assert [s.request.request_id for s in out.seqs] == ["early-urgent", "late-urgent"]
    sched.update_from_output(out, [7, 7])
    victim = sched._preempt_one(protect=None)
    assert victim.request_id == "late-urgent"                    # same priority: the later arrival goes
    # first come, first served ignores the field
    fcfs = Scheduler(SchedulerConfig(max_num_seqs=2, max_num_batched_tokens=64, max_model_len=64),
                     CacheConfig(block_size=4), num_blocks=64)
    for rid, prio in (("a", 9), ("b", 0)):
        fcfs.add_request(Request(rid, [1, 2, 3], SamplingParams(max_tokens=2, priority=prio)))
    assert [r.request_id for r in fcfs.waiting] == ["a", "b"]
