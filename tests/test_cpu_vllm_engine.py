"""The plugin under a real vLLM engine, without a GPU: vLLM's ``LLM`` (its scheduler, KV block
manager and executor) drives this package's platform (CPU / gloo variant), worker and model
runner.  Runs in a child process because vLLM resolves its platform once per process."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from omni_npu_b200 import compat

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.skipif(not compat.vllm_available(), reason="vLLM is not installed")


def _child(*args: str, timeout: int = 900, model_dir: str = "", extra_env=None) -> dict:
    env = dict(os.environ)
    env.update(extra_env or {})
    env.pop("OMNI_B200_PLUGIN", None)
    env.pop("OMNI_B200_TEST_MODEL_DIR", None)
    if model_dir:
        env["OMNI_B200_TEST_MODEL_DIR"] = model_dir
    r = subprocess.run([sys.executable, str(ROOT / "tests" / "vllm_engine_child.py"), *args],
                       capture_output=True, text=True, timeout=timeout, env=env, cwd=str(ROOT))
    lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
    assert lines, f"child failed (rc={r.returncode}):\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
    return json.loads(lines[-1][7:])


def test_vllm_engine_runs_own_worker_and_runner_token_for_token():
    res = _child("cpu")
    assert res["platform"] == "B200CpuPlatform"
    assert res["worker_cls"] == "omni_npu_b200.worker.vllm_worker.B200Worker" and res["worker"] == "B200Worker"
    assert res["runner"] == "omni_npu_b200.worker.model_runner.ModelRunner"      # not vLLM's GPUModelRunner
    assert res["async_scheduling"] is True            # vLLM schedules ahead; decode steps are launched ahead
    assert res["steps"]["launched_ahead"] > 0
    assert res["steps"]["prefill"] == 4 and res["steps"]["decode"] == 4 * 15
    assert res["via_vllm"] == res["standalone"]
    assert all(len(t) == 16 for t in res["via_vllm"])


def test_vllm_engine_loads_a_safetensors_checkpoint_and_matches_plain_pytorch(tmp_path):
    """The CPU plumbing configuration: tiny Llama, fp32, 4 prompts of 32 tokens, 16 greedy tokens,
    through vLLM's engine and this package's platform / worker / runner, against a plain PyTorch
    model reading the same checkpoint."""
    sys.path.insert(0, str(ROOT / "tests"))
    import reference_llama as refm
    from safetensors.torch import save_file
    from omni_npu_b200.config import tiny_llama
    cfg = tiny_llama()
    weights = refm.make_weights(cfg, seed=0)
    save_file({k: v.contiguous() for k, v in weights.items()}, str(tmp_path / "model.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": cfg.hidden_size,
        "num_hidden_layers": cfg.num_layers, "num_attention_heads": cfg.num_heads,
        "num_key_value_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
        "intermediate_size": cfg.intermediate_size, "vocab_size": cfg.vocab_size, "rms_norm_eps": cfg.rms_norm_eps,
        "rope_theta": cfg.rope_theta, "max_position_embeddings": 2048, "torch_dtype": "float32",
        "hidden_act": "silu", "tie_word_embeddings": False, "bos_token_id": 1, "eos_token_id": 2}))
    res = _child("cpu", "1", "4", "64", model_dir=str(tmp_path))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (32,), generator=g).tolist() for _ in range(4)]
    want = [refm.greedy_generate(weights, cfg, p, 16) for p in prompts]
    assert res["via_vllm"] == want
    assert res["standalone"] == want


def test_vllm_chunked_prefill_mixed_with_decode_gives_the_same_tokens():
    # 4 running sequences and a 24-token budget: vLLM schedules prompt chunks together with
    # decoding sequences; such steps run as variable-length prefill steps in the runner
    # (a) as ONE pass: the decoding rows first, through the decode attention, one GEMM over all rows
    res = _child("cpu", "1", "4", "24")
    assert res["via_vllm"] == res["standalone"]
    assert res["steps"].get("mixed_one_pass", 0) > 0
    # (b) as plain variable-length prefill steps
    res = _child("cpu", "1", "4", "24", extra_env={"OMNI_B200_MIXED_ONE_PASS": "0"})
    assert res["via_vllm"] == res["standalone"]
    assert res["steps"]["prefill"] > 4 and res["steps"].get("mixed", 0) == 0
    # (c) split into a decode launch and a prefill launch
    res = _child("cpu", "1", "4", "24", extra_env={"OMNI_B200_MIXED_ONE_PASS": "0", "OMNI_B200_MIXED_SPLIT_MIN": "1"})
    assert res["via_vllm"] == res["standalone"]
    assert res["steps"].get("mixed", 0) > 0 and res["steps"].get("mixed_one_pass", 0) == 0


def test_vllm_driven_ngram_speculative_decoding_gives_greedy_tokens_in_fewer_steps():
    """vLLM's scheduler hands out the drafts that this worker's n-gram look-up proposed
    (``take_draft_token_ids``); the worker verifies 1 + k rows per request in one pass and returns
    the accepted tokens.  Forty greedy tokens per request arrive in fewer than 39 decode steps and
    equal plain greedy decoding of the standalone engine."""
    res = _child("cpu", "1", "4", "64", "ngram")
    assert res["via_vllm"] == res["standalone"]
    assert all(len(t) == 40 for t in res["via_vllm"])
    assert 0 < res["steps"]["spec_decode"] < 39 and res["steps"]["decode"] == 0
    assert res["async_scheduling"] is False           # vLLM turns it off for n-gram drafts


def test_vllm_driven_drafting_with_the_models_mtp_head_gives_greedy_tokens():
    """``speculative_config={"method": "mtp", "num_speculative_tokens": 2}`` under vLLM: the runner
    builds the MTP head of a small DeepSeek-V3 shaped model and drafts two tokens per step as a chain,
    vLLM schedules them, the worker verifies.  With random weights next to nothing is accepted; the
    tokens must be those of plain greedy decoding."""
    res = _child("cpu", "1", "4", "64", "mtp")
    assert res["via_vllm"] == res["standalone"]
    assert all(len(t) == 24 for t in res["via_vllm"])
    assert res["steps"]["spec_decode"] > 0 and res["steps"]["decode"] == 0


def test_vllm_gets_log_probabilities_from_the_worker():
    """``SamplingParams(logprobs=2)`` through vLLM: the worker fills vLLM's ``LogprobsLists`` (sampled
    token, its rank, the top alternatives) from the runner's own logits; tokens are unchanged."""
    res = _child("cpu", "1", "4", "64", "logprobs")
    assert res["via_vllm"] == res["standalone"]
    for toks, per_tok in zip(res["via_vllm"], res["logprobs"]):
        assert len(per_tok) == len(toks) == 16
        for t, (lp, rank, top_ids) in zip(toks, per_tok):
            assert lp <= 0.0 and rank == 1 and top_ids[0] == t          # greedy: the sampled token leads


def test_structured_output_request_is_constrained_by_vllms_grammar_bitmask():
    """A request with ``StructuredOutputsParams(choice=["red", "blue"])`` beside a free one: vLLM hands
    the grammar's bitmask to ``sample_tokens``, the worker runs the step there and masks the logits
    rows of the structured request, which therefore answers with one of the two words and stops."""
    env = dict(os.environ)
    env.pop("OMNI_B200_PLUGIN", None)
    r = subprocess.run([sys.executable, str(ROOT / "tests" / "vllm_structured_child.py")], capture_output=True,
                       text=True, timeout=900, env=env, cwd=str(ROOT))
    lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
    assert lines, f"child failed (rc={r.returncode}):\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
    res = json.loads(lines[-1][7:])
    assert res["texts"][0].strip() in ("red", "blue")
    assert res["ids"][0][-1] == 2 and len(res["ids"][0]) == 2          # the word, then end of sequence
    assert len(res["ids"][1]) == 4                                     # the free request ran to its length cap
    assert res["steps"]["structured"] >= 2
