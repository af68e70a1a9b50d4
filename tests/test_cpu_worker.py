"""Worker-level behaviour on CPU: the token-threshold profiling window, profiler control without a
trace directory, KV-cache sizing and spec, dummy batches, and the memory budget formula with a
faked device."""
import pytest
import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import tiny_llama
from omni_npu_b200.engine.llm import LLM, build_engine_config
from omni_npu_b200.worker.worker import Worker


def _llm(**kw):
    base = dict(device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=16,
                num_gpu_blocks=32, seed=1)
    base.update(kw)
    cfg = tiny_llama()
    cfg.dtype = torch.float32
    return LLM(model=cfg, **base)


class _FakeProfiler:
    def __init__(self):
        self.events = []

    def start(self):
        self.events.append("start")

    def stop(self):
        self.events.append("stop")


def test_profiling_window_opens_on_the_token_threshold_and_closes_after_n_steps():
    llm = _llm()
    w = llm.engine.worker
    prof = _FakeProfiler()
    w.profiler, w._profile_threshold, w._profile_stop_step = prof, 4, 3
    # four sequences decoding together = 4 scheduled tokens per decode step -> window opens there
    prompts = [[1, 2, 3, 4, 5], [6, 7, 8], [9, 10, 11, 12], [13, 14]]
    llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    # the window re-arms whenever a later step hits the threshold again: strictly alternating events,
    # each window 3 steps long (8 decode steps -> two closed windows and one still open at the end)
    assert prof.events[:2] == ["start", "stop"]
    assert all(e == ("start", "stop")[i % 2] for i, e in enumerate(prof.events))
    assert prof.events.count("start") == 3 and prof.events.count("stop") == 2
    w2 = _llm(additional_config={"async_scheduling": False})
    prof2 = _FakeProfiler()
    w2.engine.worker.profiler, w2.engine.worker._profile_threshold, w2.engine.worker._profile_stop_step = prof2, 4, 3
    w2.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    assert prof2.events == prof.events                 # same windows with and without steps launched ahead
    steps = llm.engine.stats
    assert steps["decode_steps"] >= 7


def test_profile_control_needs_a_trace_directory(monkeypatch, tmp_path):
    monkeypatch.delenv("VLLM_TORCH_PROFILER_DIR", raising=False)
    llm = _llm()
    with pytest.raises(RuntimeError, match="VLLM_TORCH_PROFILER_DIR"):
        llm.start_profile()
    monkeypatch.setenv("VLLM_TORCH_PROFILER_DIR", str(tmp_path))
    llm2 = _llm()
    assert llm2.engine.worker.profiler is not None
    llm2.start_profile()
    llm2.generate([[1, 2, 3]], SamplingParams(max_tokens=2, ignore_eos=True))
    llm2.stop_profile()
    assert any(tmp_path.iterdir())                      # a trace file was written


def test_kv_cache_spec_and_block_count():
    llm = _llm(num_gpu_blocks=None)
    runner = llm.engine.worker.model_runner
    cfg = llm.config
    spec = runner.get_kv_cache_spec()
    mc = cfg.model
    assert spec.num_layers == mc.num_layers and spec.block_size == 16
    assert spec.bytes_per_block == mc.num_layers * 2 * 16 * mc.num_kv_heads * mc.head_dim * 4
    assert runner.num_blocks == max(64, 4 * cfg.scheduler.max_num_seqs)      # CPU default
    assert len(runner.kv_caches) == mc.num_layers
    k, v = runner.kv_caches[0]
    assert k.shape[0] == runner.num_blocks and k.shape == v.shape


def test_dummy_batch_leaves_requests_and_cache_rows_untouched():
    llm = _llm()
    runner = llm.engine.worker.model_runner
    before = [(k.clone(), v.clone()) for k, v in runner.kv_caches]
    llm.engine.worker.execute_dummy_batch()
    for (k0, v0), (k1, v1) in zip(before, runner.kv_caches):
        # padding rows carry slot -1: nothing may be written anywhere
        assert torch.equal(k0, k1) and torch.equal(v0, v1)
    out = llm.generate([[3, 4, 5]], SamplingParams(max_tokens=3, ignore_eos=True))[0]
    assert len(out.output_token_ids) == 3


def test_memory_budget_formula_with_a_faked_device(monkeypatch):
    """blocks = (total * utilisation - already used - activation peak) / bytes per block, capped by
    what max_num_seqs full-length sequences could use."""
    cfg = tiny_llama()
    cfg.dtype = torch.float32
    ec = build_engine_config(cfg, device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128,
                             block_size=16, gpu_memory_utilization=0.5)
    w = Worker(ec)
    w.init_device()
    w.load_model()
    runner = w.model_runner
    spec = runner.get_kv_cache_spec()
    total, free, peak = 1000 * spec.bytes_per_block, 900 * spec.bytes_per_block, 10 * spec.bytes_per_block

    class _Dev:
        type = "cuda"

    monkeypatch.setattr(runner, "device", _Dev())
    monkeypatch.setattr(runner, "profile_run", lambda: peak)
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda device=None: (free, total))
    # budget: 500 - 100 used - 10 peak = 390 blocks, but 4 sequences x 8 blocks + 64 spare = 96 is the cap
    assert runner.determine_num_blocks() == 96
    ec.scheduler.max_num_seqs = 64
    assert runner.determine_num_blocks() == 390
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda device=None: (110 * spec.bytes_per_block, total))
    with pytest.raises(RuntimeError, match="not enough memory"):
        runner.determine_num_blocks()


def test_sleep_and_wake_reach_the_pool_with_the_right_tags(monkeypatch):
    from omni_npu_b200.worker import mem_pool

    class _FakePool:
        def __init__(self):
            self.calls = []

        def sleep(self, offload_tags=None):
            self.calls.append(("sleep", tuple(offload_tags)))
            return 123

        def wake_up(self, tags=None):
            self.calls.append(("wake", tags))
            return 456

    fake = _FakePool()
    monkeypatch.setattr(mem_pool.B200MemAllocator, "get_instance", staticmethod(lambda: fake))
    w = _llm().engine.worker
    assert w.sleep(level=1) == 123 and w.sleep(level=2) == 123
    assert w.wake_up(["weights"]) == 456 and w.wake_up() == 456
    assert fake.calls == [("sleep", ("weights",)), ("sleep", ()), ("wake", ["weights"]), ("wake", None)]
