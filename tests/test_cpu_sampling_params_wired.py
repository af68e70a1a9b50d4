"""Sampling parameters that need the token history are honoured or refused, never ignored:
penalties and the thinking-token budget change the output of a tiny CPU engine exactly as a
plain re-implementation predicts; what cannot be honoured is refused; default seeds do not depend on the
process; a failed step does not end the server's engine loop."""
import subprocess
import sys

import pytest
import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import ModelConfig
from omni_npu_b200.engine.llm import LLM
from omni_npu_b200.sample.sampler import apply_penalties
from omni_npu_b200.worker.input_batch import default_seed


def _llm(**kw):
    cfg = ModelConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
                      intermediate_size=128, vocab_size=97, max_position_embeddings=256, dtype=torch.float32)
    return LLM(model=cfg, device="cpu", max_num_seqs=4, max_num_batched_tokens=32, max_model_len=128,
               block_size=8, num_gpu_blocks=64, seed=1, **kw)


def test_default_seed_is_the_same_in_every_process():
    here = default_seed("cmpl-abc123", 7)
    code = ("import sys; sys.path.insert(0, %r); from omni_npu_b200.worker.input_batch import default_seed; "
            "print(default_seed('cmpl-abc123', 7))" % str(__import__("pathlib").Path(__file__).resolve().parents[1]))
    other = [int(subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, check=True,
                                env={"PYTHONHASHSEED": str(s), "PATH": "/usr/bin:/bin"}).stdout) for s in (1, 2)]
    assert other == [here, here]
    assert default_seed("cmpl-abc123", 8) != here and default_seed("cmpl-abc124", 7) != here
    assert 0 <= here < 2 ** 63


def _greedy_with_penalties(llm, prompt, n, sp):
    """Plain re-computation: full forward of the model on CPU each step, penalties by the
    reference formula, argmax."""
    runner = llm.engine.worker.model_runner
    plain = LLM(model=llm.config.model, device="cpu", max_num_seqs=1, max_num_batched_tokens=128,
                max_model_len=128, block_size=8, num_gpu_blocks=32, seed=1)
    plain.engine.worker.model_runner.model.load_state_dict(runner.model.state_dict())
    V = llm.config.model.vocab_size
    outs = []
    for _ in range(n):
        # logits of the next token = those that produce the first token of a fresh request
        captured = {}
        pr = plain.engine.worker.model_runner
        pr._logits_fn_saved = None

        def grab(lg):
            captured["l"] = lg.float().clone()
            return lg
        real = pr._make_logits_fn
        pr._make_logits_fn = lambda seqs: grab
        plain.generate([prompt + outs], SamplingParams(max_tokens=1, ignore_eos=True))
        pr._make_logits_fn = real
        logits = captured["l"][:1]
        counts = torch.zeros(1, V)
        for t in outs:
            counts[0, t] += 1
        pmask = torch.zeros(1, V, dtype=torch.bool)
        pmask[0, prompt] = True
        logits = apply_penalties(logits, pmask, counts, torch.tensor([sp.presence_penalty]),
                                 torch.tensor([sp.frequency_penalty]), torch.tensor([sp.repetition_penalty]))
        outs.append(int(logits.argmax(-1)))
    return outs


def test_penalties_change_greedy_output_as_the_formula_says():
    llm = _llm()
    prompt = [5, 6, 7, 8, 9, 10]
    base = llm.generate([prompt], SamplingParams(max_tokens=12, ignore_eos=True))[0].output_token_ids
    sp = SamplingParams(max_tokens=12, ignore_eos=True, repetition_penalty=1.8, frequency_penalty=0.7,
                        presence_penalty=0.4)
    got = llm.generate([prompt], sp)[0].output_token_ids
    want = _greedy_with_penalties(llm, prompt, 12, sp)
    assert got == want
    assert got != base                      # a tiny random model repeats itself; the penalties break that
    # a batch mixing penalised and plain rows keeps the plain rows unchanged
    both = llm.generate([prompt, prompt], [SamplingParams(max_tokens=12, ignore_eos=True), sp])
    assert both[0].output_token_ids == base and both[1].output_token_ids == want


def test_thinking_budget_forces_the_end_marker():
    rc = {"think_start_token_ids": [90], "think_end_token_ids": [91, 92]}
    llm = _llm(additional_config={"reasoning_config": rc})
    prompt = [5, 6, 7, 90]                  # the prompt ends inside an open thinking span
    out = llm.generate([prompt], SamplingParams(max_tokens=10, ignore_eos=True, thinking_token_budget=3))[0]
    toks = out.output_token_ids
    assert toks[3:5] == [91, 92], toks       # three thinking tokens, then the forced two-token marker
    free = llm.generate([prompt], SamplingParams(max_tokens=10, ignore_eos=True))[0].output_token_ids
    assert free[:3] == toks[:3]
    with pytest.raises(ValueError):
        _llm().generate([prompt], SamplingParams(max_tokens=4, thinking_token_budget=3))


def test_what_the_sampler_cannot_honour_is_refused_not_ignored():
    llm = _llm()
    with pytest.raises(ValueError, match="logprobs"):
        llm.generate([[1, 2, 3]], SamplingParams(max_tokens=2, logprobs=50))          # more than 20 alternatives
    with pytest.raises(ValueError, match="tokenizer"):
        llm.generate([[1, 2, 3]], SamplingParams(max_tokens=2, structured={"choice": ["a"]}))
    out = llm.generate([[1, 2, 3]], SamplingParams(max_tokens=2, ignore_eos=True, logprobs=5))[0]
    assert len(out.logprobs) == 2 and len(out.logprobs[0][1]) == 5                    # ... and what it can is done


def test_server_answers_400_and_survives_a_failing_step():
    from starlette.testclient import TestClient

    from omni_npu_b200.serving.api_server import build_app
    llm = _llm()
    app = build_app(llm, None, "tiny")
    with TestClient(app) as c:
        r = c.post("/v1/completions", json={"prompt": [1, 2, 3], "max_tokens": 2, "logprobs": 30})
        assert r.status_code == 400 and "logprobs" in r.text
        r = c.post("/v1/completions", json={"prompt": [1, 2, 3], "max_tokens": 2, "guided_choice": ["a", "b"]})
        assert r.status_code == 400 and "tokenizer" in r.text                  # this server has no tokenizer
        r = c.post("/v1/completions", json={"prompt": [1, 2, 3], "max_tokens": 4, "ignore_eos": True,
                                            "repetition_penalty": 1.3})
        assert r.status_code == 200 and len(r.json()["choices"][0]["token_ids"]) == 4
        # one step raises: the request in flight ends as aborted, the loop thread lives on
        real = llm.engine.step
        state = {"n": 0}

        def flaky():
            state["n"] += 1
            if state["n"] == 2:
                raise RuntimeError("injected step failure")
            return real()
        llm.engine.step = flaky
        r = c.post("/v1/completions", json={"prompt": [4, 5, 6], "max_tokens": 8, "ignore_eos": True})
        assert r.status_code == 200 and r.json()["choices"][0]["finish_reason"] == "abort"
        llm.engine.step = real
        r = c.post("/v1/completions", json={"prompt": [4, 5, 6], "max_tokens": 3, "ignore_eos": True})
        assert r.status_code == 200 and len(r.json()["choices"][0]["token_ids"]) == 3
        assert app.state.engine_loop.counters["failed_steps"] == 1
    app.state.engine_loop.shutdown()
