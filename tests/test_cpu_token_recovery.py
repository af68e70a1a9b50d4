"""Token recovery end to end on CPU: the failure is made on the host (the model step raises
an exception carrying a target error code); coordinator and worker endpoints talk over
127.0.0.1."""
import threading
import time

import pytest
import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import ModelConfig
from omni_npu_b200.engine.llm import LLM
from omni_npu_b200.ha import common as C
from omni_npu_b200.ha.monitor import HAWorkerAgent, matching_error_code, token_recover_wrapper
from omni_npu_b200.ha.server import HAServer, post_json


def _tiny():
    return ModelConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
                       intermediate_size=128, vocab_size=97, max_position_embeddings=512, dtype=torch.float32)


class FakeWorker:
    """Two of these stand for two ranks; rank 0's step fails once."""

    def __init__(self, agent, fail_msg=None):
        self.ha_agent = agent
        self.fail_msg = fail_msg
        self.calls = []
        self.failed = False

    def stop_device(self):
        self.calls.append("stop")

    def restart_device(self):
        self.calls.append("restart")

    def reinit_process_group(self):
        self.calls.append("reinit")

    @token_recover_wrapper
    def execute_model(self, out):
        if self.fail_msg and not self.failed:
            self.failed = True
            raise RuntimeError(self.fail_msg)
        return [1, 2, 3]


def test_error_code_matching():
    assert matching_error_code("NCCL error in: foo.cpp unhandled system error") == "NCCL error"
    assert matching_error_code("index out of range") is None


@pytest.mark.parametrize("msg,kind", [("[Rank 0] NCCL error: remote process exited", "recompute"),
                                      ("CUDA error: uncorrectable ECC error encountered", "abort")])
def test_two_workers_recover_together(msg, kind):
    server = HAServer("127.0.0.1", 0, wait_stop_s=5, wait_recovery_s=5, poll_s=0.01).start()
    env = C.HAEnv(True, "127.0.0.1", server.port)
    a0 = HAWorkerAgent(env, 0).start()
    a1 = HAWorkerAgent(env, 1).start()
    assert len(server.processor.worker_servers) == 2
    w0, w1 = FakeWorker(a0, msg), FakeWorker(a1)
    if kind == "abort":
        w0.find_bad_kv_blocks = lambda: [7, 9]
    res = {}

    def run(name, w):
        try:
            res[name] = w.execute_model(None)
        except Exception as e:
            res[name] = e

    # rank 1 is healthy: it gets poked by the coordinator and fails its next step on purpose
    t0 = threading.Thread(target=run, args=("w0", w0))
    t0.start()
    deadline = time.time() + 5
    while not a1.stop_requested.is_set() and time.time() < deadline:
        time.sleep(0.01)
    assert a1.stop_requested.is_set()
    t1 = threading.Thread(target=run, args=("w1", w1))
    t1.start()
    t0.join(10), t1.join(10)
    try:
        assert res["w0"] == {"opt": kind, "bad_blocks": [7, 9] if kind == "abort" else []}
        assert res["w1"]["opt"] == kind
        assert w0.calls == ["stop", "restart", "reinit"] and w1.calls == ["stop", "restart", "reinit"]
        deadline = time.time() + 2
        while not server.processor.history and time.time() < deadline:
            time.sleep(0.01)                      # the coordinator records the outcome after its last broadcast
        assert server.processor.history and server.processor.history[-1][1] == kind
        assert a0.recompute_pending == (kind == "recompute")
        # the next step works and clears the flag
        assert w0.execute_model(None) == [1, 2, 3] and not a0.recompute_pending
    finally:
        a0.stop(), a1.stop(), server.stop()


def test_unrecoverable_paths_re_raise():
    # no coordinator command arrives: the original exception propagates
    env = C.HAEnv(True, "127.0.0.1", 1)            # nothing listens on port 1
    agent = HAWorkerAgent(env, 0, post=lambda url, body: None)
    agent.http.start()
    w = FakeWorker(agent, "NCCL error: x")
    old = C.WORKER_WAITING_STOP_TIME
    C.WORKER_WAITING_STOP_TIME = 0.05
    try:
        with pytest.raises(RuntimeError, match="NCCL error"):
            w.execute_model(None)
        # errors without a target code are not touched
        w2 = FakeWorker(agent, "shape mismatch")
        with pytest.raises(RuntimeError, match="shape mismatch"):
            w2.execute_model(None)
        assert w2.calls == []
    finally:
        C.WORKER_WAITING_STOP_TIME = old
        agent.stop()


def test_processor_options_and_timeouts():
    server = HAServer("127.0.0.1", 0, wait_stop_s=0.2, wait_recovery_s=0.2, poll_s=0.01)
    p = server.processor
    p.worker_servers.append("127.0.0.1:9")
    p.post = lambda url, body: None
    assert p.process_fault_step(1) == "stop_timeout"
    st = C.WorkerStatus("127.0.0.1:9", 0, 0, C.WORKER_STATUS_DEVICE_FORCE_STOPPED, "NCCL error")
    server.worker_status["127.0.0.1:9"] = st
    assert p.keep_run_option() == (C.OPT_RECOMPUTE, [])
    st.err_code, st.bad_memory, st.bad_blocks = C.ERR_UNCORRECTABLE_MEMORY, True, [-1]
    assert p.keep_run_option()[0] == C.OPT_EXIT
    st.bad_blocks = [3]
    assert p.keep_run_option() == (C.OPT_ABORT, [3])
    st.err_code, st.bad_memory, st.bad_blocks = "CUDA error: unspecified launch failure", False, []
    assert p.keep_run_option()[0] == C.OPT_EXIT
    server.http.httpd.server_close()


def test_engine_recomputes_a_failed_step_and_finishes_all_requests(monkeypatch):
    """One decode step of a real (CPU) engine raises; after recovery every request still
    produces exactly the tokens of an undisturbed run."""
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 97, (n,), generator=g).tolist() for n in (7, 15, 11)]
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    kw = dict(device="cpu", max_num_seqs=4, max_num_batched_tokens=32, max_model_len=128,
              block_size=8, num_gpu_blocks=64, seed=3)
    want = [o.output_token_ids for o in LLM(model=_tiny(), **kw).generate(prompts, sp)]

    server = HAServer("127.0.0.1", 0, wait_stop_s=5, wait_recovery_s=5, poll_s=0.01).start()
    llm = LLM(model=_tiny(), **kw)
    worker = llm.engine.worker
    worker.enable_token_recovery(C.HAEnv(True, "127.0.0.1", server.port))
    runner = worker.model_runner
    real = runner.execute_model
    state = {"n": 0}

    def flaky(out):
        state["n"] += 1
        if state["n"] == 4:                       # a decode step in the middle of generation
            raise RuntimeError("NCCL error: peer rank exited")
        return real(out)

    monkeypatch.setattr(runner, "execute_model", flaky)
    try:
        got = [o.output_token_ids for o in llm.generate(prompts, sp)]
        assert got == want
        assert llm.engine.stats["recovered_steps"] == 1
        deadline = time.time() + 2
        while not server.processor.history and time.time() < deadline:
            time.sleep(0.01)
        assert server.processor.history[-1][1] == "recompute"
    finally:
        worker.ha_agent.stop()
        server.stop()
