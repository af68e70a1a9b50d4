"""The plugin under a real vLLM engine on a B200: vLLM's ``LLM`` drives this package's platform,
worker and model runner (tcgen05 GEMMs, own attention kernels, full-step decode graphs), and
the result equals the package's standalone engine on the same weights.  Child processes,
because vLLM resolves its platform once per process."""
import pytest

from omni_npu_b200 import compat
from test_cpu_vllm_engine import _child

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not compat.vllm_available(), reason="vLLM is not installed")]


def test_vllm_engine_on_gpu_runs_own_kernels_and_matches_standalone_engine():
    res = _child("cuda", timeout=1200)
    assert res["platform"] == "B200Platform"
    assert res["worker"] == "B200Worker"
    assert res["runner"] == "omni_npu_b200.worker.model_runner.ModelRunner"
    assert res["async_scheduling"] is True            # vLLM schedules ahead; decode steps are launched ahead
    assert res["steps"]["launched_ahead"] > 0
    assert res["graphs"] > 0                       # decode steps replay this package's CUDA graphs
    assert res["launches"] > 100                   # kernels of this package's extension were launched
    assert res["steps"]["prefill"] == 4 and res["steps"]["decode"] == 4 * 15
    # one sequence at a time: identical kernels on identical shapes in both engines
    assert res["via_vllm"] == res["standalone"]


def test_vllm_engine_on_gpu_batched_requests_finish():
    res = _child("cuda", "1", "4", "48", timeout=1200)
    assert all(len(t) == 16 for t in res["via_vllm"])
    # batched and chunked steps differ from the one-at-a-time run only by bf16 rounding of a
    # different batch composition: the first tokens of every request agree
    assert [t[0] for t in res["via_vllm"]] == [t[0] for t in res["standalone"]]


@pytest.mark.parametrize("method,n_out", [("ngram", 40), ("mtp", 24)])
def test_vllm_driven_speculative_decoding_on_gpu(method, n_out):
    """vLLM schedules the drafts that this worker makes (n-gram look-up, or the MTP head of a small
    DeepSeek-V3 shaped model) and the worker verifies them with its own kernels.  Verification rows
    and plain decode rows are rounded differently in bf16, so the tokens are compared as in the
    batched test: the same first tokens, most tokens equal."""
    res = _child("cuda", "1", "4", "64", method, timeout=1200)
    assert res["worker"] == "B200Worker" and res["launches"] > 100
    assert res["steps"].get("spec_decode", 0) > 0
    assert all(len(t) == n_out for t in res["via_vllm"])
    same = sum(x == y for a, b in zip(res["via_vllm"], res["standalone"]) for x, y in zip(a, b))
    assert [t[0] for t in res["via_vllm"]] == [t[0] for t in res["standalone"]]
    assert same >= 0.6 * n_out * len(res["via_vllm"])


@pytest.mark.multi_gpu
def test_vllm_engine_tensor_parallel_two_gpus():
    one = _child("cuda", timeout=1200)
    two = _child("cuda", "2", timeout=1500)
    assert two["worker_cls"] == "omni_npu_b200.worker.vllm_worker.B200Worker"
    assert all(len(t) == 16 for t in two["via_vllm"])
    assert [t[0] for t in two["via_vllm"]] == [t[0] for t in one["via_vllm"]]
