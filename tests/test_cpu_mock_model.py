"""Capture / replay / random modes of the mock model factory (CPU)."""
import time

import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import ModelConfig
from omni_npu_b200.engine.llm import LLM
from omni_npu_b200.models import mock as mock_mod


def _cfg():
    return ModelConfig(architecture="MockModel", hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2,
                       head_dim=16, intermediate_size=128, vocab_size=101, max_position_embeddings=256,
                       dtype=torch.float32)


def _llm():
    mock_mod._LazyMock._cls = None          # environment switches are read when the class is first built
    return LLM(model=_cfg(), device="cpu", max_num_seqs=4, max_num_batched_tokens=16, max_model_len=128,
               block_size=8, num_gpu_blocks=64, seed=5)


def _clear(monkeypatch):
    for k in ("RANDOM_MODE", "CAPTURE_MODE", "REPLAY_MODE", "KV_CACHE_MODE", "FORWARD_TIME",
              "SIMULATE_ELAPSED_TIME", "MOCK_COMPUTE_LOGITS", "PREFILL_PROCESS"):
        monkeypatch.delenv(k, raising=False)


def test_capture_then_replay_reproduces_tokens_without_running_the_network(tmp_path, monkeypatch):
    _clear(monkeypatch)
    monkeypatch.setenv("MOCK_CAPTURE_DIR", str(tmp_path))
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 101, (n,), generator=g).tolist() for n in (5, 21, 12)]     # 21 > chunk of 16
    sp = SamplingParams(max_tokens=7, ignore_eos=True)
    monkeypatch.setenv("CAPTURE_MODE", "1")
    cap = _llm()
    model = cap.engine.worker.get_model()
    assert isinstance(model, mock_mod.MockModel) and model.capture_mode
    want = [o.output_token_ids for o in cap.generate(prompts, sp)]
    assert model.base_forward_calls > 0 and (tmp_path / "mock_cache.json").exists()
    monkeypatch.delenv("CAPTURE_MODE")
    monkeypatch.setenv("REPLAY_MODE", "1")
    monkeypatch.setenv("KV_CACHE_MODE", "1")
    rep = _llm()
    rmodel = rep.engine.worker.get_model()
    got = [o.output_token_ids for o in rep.generate(prompts, sp)]
    assert got == want and rmodel.base_forward_calls == 0
    # the KV slots of the replayed steps were filled
    k0 = rep.engine.worker.model_runner.kv_caches[0][0]
    assert float(k0.abs().sum()) > 0


def test_random_mode_runs_and_simulated_time_sleeps(monkeypatch, tmp_path):
    _clear(monkeypatch)
    monkeypatch.setenv("MOCK_CAPTURE_DIR", str(tmp_path))
    monkeypatch.setenv("RANDOM_MODE", "1")
    monkeypatch.setenv("MOCK_COMPUTE_LOGITS", "1")
    monkeypatch.setenv("FORWARD_TIME", "20")
    llm = _llm()
    t0 = time.perf_counter()
    outs = llm.generate([[1, 2, 3]], SamplingParams(max_tokens=4, ignore_eos=True))
    dt = time.perf_counter() - t0
    assert len(outs[0].output_token_ids) == 4
    assert llm.engine.worker.get_model().base_forward_calls == 0
    assert dt >= 4 * 0.02          # one prefill + three decode steps, 20 ms each
    # deterministic
    again = _llm().generate([[1, 2, 3]], SamplingParams(max_tokens=4, ignore_eos=True))
    assert again[0].output_token_ids == outs[0].output_token_ids
