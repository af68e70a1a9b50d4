"""The OpenAI-compatible server in front of a tiny CPU engine, driven through the ASGI app
(no sockets), and the benchmark client's statistics."""
import json

import pytest
import torch

from omni_npu_b200.config import ModelConfig
from omni_npu_b200.engine.llm import LLM
from omni_npu_b200.serving import bench_client
from omni_npu_b200.serving.api_server import build_app, make_parser, sampling_from_body


def _llm():
    cfg = ModelConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
                      intermediate_size=128, vocab_size=97, max_position_embeddings=256, dtype=torch.float32)
    return LLM(model=cfg, device="cpu", max_num_seqs=4, max_num_batched_tokens=32, max_model_len=128,
               block_size=8, num_gpu_blocks=64, seed=1)


@pytest.fixture(scope="module")
def client():
    from starlette.testclient import TestClient
    llm = _llm()
    want = llm.generate([[5, 6, 7, 8]], __import__("omni_npu_b200").SamplingParams(max_tokens=6, ignore_eos=True))
    app = build_app(llm, None, "tiny")
    with TestClient(app) as c:
        c.expected = want[0].output_token_ids
        yield c
    app.state.engine_loop.shutdown()


def test_completions_and_metrics(client):
    assert client.get("/health").json() == {"status": "ok"}
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny"
    r = client.post("/v1/completions", json={"prompt": [5, 6, 7, 8], "max_tokens": 6, "ignore_eos": True})
    assert r.status_code == 200
    body = r.json()
    assert body["choices"][0]["token_ids"] == client.expected
    assert body["usage"] == {"prompt_tokens": 4, "completion_tokens": 6, "total_tokens": 10}
    assert client.post("/v1/completions", json={"prompt": "text without tokenizer"}).status_code == 400
    m = client.get("/metrics").text
    assert "omni_b200_requests_finished_total" in m and "omni_b200_output_tokens_total" in m


def test_completions_and_chat_return_log_probabilities(client):
    r = client.post("/v1/completions", json={"prompt": [5, 6, 7, 8], "max_tokens": 6, "ignore_eos": True, "logprobs": 2})
    assert r.status_code == 200
    ch = r.json()["choices"][0]
    assert ch["token_ids"] == client.expected
    lp = ch["logprobs"]
    assert lp["token_ids"] == client.expected and len(lp["token_logprobs"]) == 6 and len(lp["top_logprobs"]) == 6
    assert all(v <= 0 for v in lp["token_logprobs"]) and all(len(t) == 2 for t in lp["top_logprobs"])
    # greedy: the sampled token is the first alternative
    assert all(str(t) in top and abs(top[str(t)] - v) < 1e-6
               for t, v, top in zip(lp["token_ids"], lp["token_logprobs"], lp["top_logprobs"]))
    r = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [5, 6, 7, 8]}],
                                                  "max_tokens": 3, "ignore_eos": True, "logprobs": True,
                                                  "top_logprobs": 3})
    assert r.status_code == 200
    content = r.json()["choices"][0]["logprobs"]["content"]
    assert len(content) == 3 and all(len(e["top_logprobs"]) == 3 and e["top_logprobs"][0]["token_id"] == e["token_id"]
                                     for e in content)
    # not asked for: the field is null
    r = client.post("/v1/completions", json={"prompt": [5, 6, 7, 8], "max_tokens": 2, "ignore_eos": True})
    assert r.json()["choices"][0]["logprobs"] is None


def test_streaming_yields_all_tokens(client):
    with client.stream("POST", "/v1/completions", json={"prompt": [5, 6, 7, 8], "max_tokens": 6, "ignore_eos": True,
                                                         "stream": True}) as r:
        toks, done, finish = [], False, None
        for line in r.iter_lines():
            if not line.startswith("data:"):
                continue
            data = line[5:].strip()
            if data == "[DONE]":
                done = True
                break
            ch = json.loads(data)["choices"][0]
            toks += ch["token_ids"]
            finish = ch["finish_reason"] or finish
    assert done and toks == client.expected and finish


def test_chat_streaming_yields_delta_chunks(client):
    body = {"messages": [{"role": "user", "content": [5, 6, 7, 8]}], "max_tokens": 6, "ignore_eos": True, "stream": True}
    with client.stream("POST", "/v1/chat/completions", json=body) as r:
        toks, roles, finish, done = [], [], None, False
        for line in r.iter_lines():
            if not line.startswith("data: "):
                continue
            if line == "data: [DONE]":
                done = True
                break
            ev = json.loads(line[6:])
            assert ev["object"] == "chat.completion.chunk"
            ch = ev["choices"][0]
            toks += ch["token_ids"]
            if "role" in ch["delta"]:
                roles.append(ch["delta"]["role"])
            finish = ch["finish_reason"] or finish
    assert done and toks == client.expected and roles == ["assistant"] and finish == "length"


def test_n_choices_are_independent_samples(client):
    body = {"prompt": [5, 6, 7, 8], "max_tokens": 6, "ignore_eos": True, "n": 3, "temperature": 1.0, "seed": 11}
    r = client.post("/v1/completions", json=body)
    assert r.status_code == 200
    out = r.json()
    assert [c["index"] for c in out["choices"]] == [0, 1, 2] and out["usage"]["completion_tokens"] == 18
    assert len({tuple(c["token_ids"]) for c in out["choices"]}) > 1            # seeds 11, 12, 13 draw differently
    # a seeded request draws the same tokens whenever it runs, whatever the engine did in between
    client.post("/v1/completions", json={"prompt": [9, 9, 9], "max_tokens": 3, "temperature": 1.0})
    again = client.post("/v1/completions", json=body).json()
    assert [c["token_ids"] for c in again["choices"]] == [c["token_ids"] for c in out["choices"]]
    alone = client.post("/v1/completions", json=dict(body, n=1, seed=12)).json()
    assert alone["choices"][0]["token_ids"] == out["choices"][1]["token_ids"]
    assert client.post("/v1/completions", json=dict(body, stream=True)).status_code == 400
    assert client.post("/v1/completions", json=dict(body, n=17)).status_code == 400


def test_request_fields_and_cli():
    sp = sampling_from_body({"max_tokens": 9, "temperature": 0.7, "top_k": 5, "top_p": 0.9, "thinking_token_budget": 64,
                             "stop_token_ids": [2], "repetition_penalty": 1.1})
    assert (sp.max_tokens, sp.top_k, sp.thinking_token_budget, tuple(sp.stop_token_ids)) == (9, 5, 64, (2,))
    a = make_parser().parse_args(["--model", "llama-3-8b", "--kv-transfer-config",
                                  '{"kv_connector": "LLMDataDistConnector", "kv_role": "kv_producer"}',
                                  "--reasoning-parser", "pangu", "--speculative-config",
                                  '{"method": "deepseek_mtp", "num_speculative_tokens": 1}'])
    assert a.kv_transfer_config["kv_role"] == "kv_producer" and a.speculative_config["method"] == "deepseek_mtp"
    assert a.enable_kv_rmsnorm_rope_cache


def test_bench_client_statistics():
    rs = [bench_client.RequestResult(True, 100, 11, ttft=0.1, latency=1.1, itl=[0.1] * 10),
          bench_client.RequestResult(True, 100, 21, ttft=0.2, latency=2.2, itl=[0.1] * 20),
          bench_client.RequestResult(False, 100, 0, error="boom")]
    s = bench_client.summarise(rs, wall=4.0)
    assert s["completed"] == 2 and s["failed"] == 1
    assert s["output_token_throughput"] == 8.0 and s["input_token_throughput"] == 50.0
    assert abs(s["mean_tpot_ms"] - 100.0) < 1e-6 and abs(s["median_ttft_ms"] - 100.0) < 1e-6 or s["median_ttft_ms"] == 200.0
    assert bench_client.percentile([1, 2, 3, 4, 5], 99) == 5
    a = bench_client.make_parser().parse_args(["--num-processes", "4", "--num-warmups", "8", "--profile"])
    assert a.num_processes == 4 and a.num_warmups == 8 and a.profile
