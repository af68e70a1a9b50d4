"""Structured outputs of the standalone engine: a request restricted to a choice of strings, a JSON
schema, a regular expression or a grammar only produces tokens its grammar allows, and ends when
the grammar is complete."""
import json

import pytest
import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import ModelConfig
from omni_npu_b200.engine.llm import LLM
from omni_npu_b200.sample.structured import StructuredOutputManager, structured_spec_from_body

pytest.importorskip("xgrammar")

WORDS = ["yes", "no", "maybe", "the", "a", "cat", "dog", "is", "red", "blue", "{", "}", ":", ",", '"', "1", "2", "3",
         "true", "false", "name", "age", "x", "q"]


@pytest.fixture(scope="module")
def tokenizer():
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    vocab = {"<unk>": 0, "<s>": 1, "</s>": 2}
    for w in WORDS + [f"w{i}" for i in range(97 - 3 - len(WORDS))]:
        vocab[w] = len(vocab)
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    return PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", bos_token="<s>", eos_token="</s>")


def _llm(tokenizer, **kw):
    cfg = ModelConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128,
                      vocab_size=97, rope_theta=10000.0, max_position_embeddings=512, dtype=torch.float32)
    cfg.eos_token_id = 2
    llm = LLM(model=cfg, device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=4,
              num_gpu_blocks=64, seed=3, **kw)
    if tokenizer is not None:
        llm.enable_structured_outputs(tokenizer)
    return llm


def test_choice_regex_and_free_requests_share_a_batch(tokenizer):
    llm = _llm(tokenizer)
    v = tokenizer.get_vocab()
    prompts = [[5, 6, 7], [9, 8, 7, 6], [4, 4, 4]]
    sps = [SamplingParams(max_tokens=8, structured={"choice": ["red", "blue"]}),
           SamplingParams(max_tokens=8, temperature=0.9, seed=5, structured={"regex": "(yes|no)(yes|no)"}),
           SamplingParams(max_tokens=5, ignore_eos=True)]
    outs = llm.generate(prompts, sps)
    # the word, then the end-of-sequence token (the only token a complete grammar allows)
    assert outs[0].output_token_ids in ([v["red"], 2], [v["blue"], 2]) and outs[0].finish_reason == "stop"
    two = outs[1].output_token_ids
    assert len(two) == 3 and two[2] == 2 and all(t in (v["yes"], v["no"]) for t in two[:2])
    assert len(outs[2].output_token_ids) == 5
    free = _llm(None).generate(prompts[2:], sps[2:])
    assert free[0].output_token_ids == outs[2].output_token_ids          # the free request is not disturbed
    assert not llm.engine.worker.model_runner.structured._matchers       # matchers of finished requests are gone


def test_a_grammar_the_vocabulary_cannot_continue_ends_the_request(tokenizer):
    """"q" is a token and a prefix of the only allowed word, but no token spells the rest: after
    "q" nothing is allowed, and the request ends instead of sampling from an empty row."""
    llm = _llm(tokenizer)
    v = tokenizer.get_vocab()
    out = llm.generate([[5, 6, 7]], SamplingParams(max_tokens=6, structured={"regex": "qzz"}))[0]
    assert out.output_token_ids == [v["q"], 2] and out.finish_reason == "stop"


def test_json_schema_output_parses(tokenizer):
    llm = _llm(tokenizer)
    schema = {"type": "object", "properties": {"x": {"type": "boolean"}}, "required": ["x"], "additionalProperties": False}
    out = llm.generate([[3, 4, 5]], SamplingParams(max_tokens=24, structured={"json_schema": schema}))[0]
    assert out.finish_reason == "stop"
    text = "".join(tokenizer.convert_ids_to_tokens(out.output_token_ids[:-1]))
    assert json.loads(text) in ({"x": True}, {"x": False})


def test_refusals_and_request_fields(tokenizer):
    with pytest.raises(ValueError):
        _llm(None).generate([[1, 2]], SamplingParams(max_tokens=2, structured={"choice": ["red"]}))
    llm = _llm(tokenizer)
    with pytest.raises(ValueError):
        llm.generate([[1, 2]], SamplingParams(max_tokens=2, structured={"grammar": "root ::= ("}))
    with pytest.raises(ValueError):
        StructuredOutputManager.check_spec({"choice": []})
    assert structured_spec_from_body({"guided_choice": ["a", "b"]}) == {"choice": ["a", "b"]}
    assert structured_spec_from_body({"structured_outputs": {"regex": "a+"}}) == {"regex": "a+"}
    assert structured_spec_from_body({"response_format": {"type": "json_object"}}) == {"json_object": True}
    assert structured_spec_from_body({"response_format": {"type": "json_schema", "json_schema": {"schema": {"type": "object"}}}}) \
        == {"json_schema": {"type": "object"}}
    assert structured_spec_from_body({"max_tokens": 3}) is None


def test_api_server_routes_take_structured_output_fields(tokenizer):
    from starlette.testclient import TestClient
    from omni_npu_b200.serving.api_server import build_app
    llm = _llm(tokenizer)
    app = build_app(llm, tokenizer, "tiny")
    with TestClient(app) as c:
        r = c.post("/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 8, "guided_choice": ["cat", "dog"]})
        assert r.status_code == 200 and r.json()["choices"][0]["text"].replace("</s>", "").strip() in ("cat", "dog")
        r = c.post("/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 8,
                                            "structured_outputs": {"grammar": "root ::= ("}})
        assert r.status_code == 400                       # a grammar that does not compile is refused up front
    app.state.engine_loop.shutdown()


def test_stop_strings_end_the_request_and_cut_the_text(tokenizer):
    """``stop`` of the OpenAI routes: the decoded output is watched for the strings; the request is
    aborted in the engine when one shows up and the answer's text ends before it."""
    from starlette.testclient import TestClient
    from omni_npu_b200.serving.api_server import build_app
    llm = _llm(tokenizer)
    app = build_app(llm, tokenizer, "tiny")
    with TestClient(app) as c:
        free = c.post("/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 8, "ignore_eos": True}).json()
        ids = free["choices"][0]["token_ids"]
        words = tokenizer.convert_ids_to_tokens(ids)
        stop_word = words[3]                                   # the fourth generated word ends the answer
        first = words.index(stop_word)
        r = c.post("/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 8, "ignore_eos": True,
                                            "stop": [stop_word, "never-there"]})
        ch = r.json()["choices"][0]
        assert r.status_code == 200 and ch["finish_reason"] == "stop"
        assert ch["token_ids"] == ids[:first]
        assert stop_word not in ch["text"].split() and ch["text"].strip() == tokenizer.decode(ids[:first]).strip()
        # the engine is free again and serves the next request in full
        again = c.post("/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 8, "ignore_eos": True}).json()
        assert again["choices"][0]["token_ids"] == ids
        assert llm.engine.scheduler.pool.num_free == 64
    app.state.engine_loop.shutdown()
    # a server without a tokenizer refuses stop strings instead of ignoring them
    app = build_app(_llm(None), None, "tiny")
    with TestClient(app) as c:
        assert c.post("/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 4, "stop": "x"}).status_code == 400
    app.state.engine_loop.shutdown()


def test_tokenize_detokenize_and_version_routes(tokenizer):
    from starlette.testclient import TestClient
    from omni_npu_b200.serving.api_server import build_app
    app = build_app(_llm(tokenizer), tokenizer, "tiny")
    with TestClient(app) as c:
        assert c.get("/ping").text == "pong" and "version" in c.get("/version").json()
        t = c.post("/tokenize", json={"prompt": "the cat is red"}).json()
        assert t["count"] == 4 and t["tokens"] == tokenizer.encode("the cat is red") and t["max_model_len"] == 128
        assert c.post("/detokenize", json={"tokens": t["tokens"]}).json()["prompt"].split() == ["the", "cat", "is", "red"]
    app.state.engine_loop.shutdown()
    app = build_app(_llm(None), None, "tiny")
    with TestClient(app) as c:
        assert c.post("/tokenize", json={"prompt": "x"}).status_code == 400
    app.state.engine_loop.shutdown()


def test_text_prompts_with_a_tokenizer_in_the_model_directory(tokenizer, tmp_path):
    """``LLM(model=<directory>)`` finds the tokenizer beside the weights: text prompts are encoded,
    outputs carry their text, structured outputs work without further set-up."""
    import reference_llama as refm
    from omni_npu_b200.config import tiny_llama
    from test_cpu_plumbing import _save
    cfg = tiny_llama()
    weights = refm.make_weights(cfg, seed=0)
    _save(weights, cfg, str(tmp_path))
    tokenizer.save_pretrained(str(tmp_path))
    llm = LLM(model=str(tmp_path), device="cpu", dtype="float32", max_num_seqs=4, max_num_batched_tokens=64,
              max_model_len=128, block_size=16, num_gpu_blocks=32)
    ids = tokenizer.encode("the cat is")
    a, b = llm.generate(["the cat is", ids], SamplingParams(max_tokens=5, ignore_eos=True))
    assert a.output_token_ids == b.output_token_ids == refm.greedy_generate(weights, cfg, ids, 5)
    assert a.text == tokenizer.decode(a.output_token_ids)
    c = llm.generate(["the cat is"], SamplingParams(max_tokens=4, structured={"choice": ["red", "blue"]}))[0]
    assert c.text.replace("</s>", "").strip() in ("red", "blue")
    with pytest.raises(ValueError):
        _llm(None).generate(["text without a tokenizer"], SamplingParams(max_tokens=2))
