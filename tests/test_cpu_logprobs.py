"""Log-probabilities of the sampled tokens: the engine returns, per output token, the
log-probability of the token under the model's own distribution and the most likely alternatives."""
import math

import pytest
import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import ModelConfig
from omni_npu_b200.engine.llm import LLM


def _cfg():
    return ModelConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128,
                       vocab_size=97, rope_theta=10000.0, max_position_embeddings=512, dtype=torch.float32)


def _llm(**kw):
    return LLM(model=_cfg(), device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=4,
               num_gpu_blocks=64, seed=3, **kw)


def test_greedy_tokens_are_the_most_likely_ones_and_unchanged_by_asking():
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(1, 97, (n,), generator=g).tolist() for n in (5, 17, 9)]
    plain = _llm().generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
    sps = [SamplingParams(max_tokens=6, ignore_eos=True, logprobs=k) for k in (3, 1, 5)]
    outs = _llm().generate(prompts, sps)
    for o, p, sp in zip(outs, plain, sps):
        assert o.output_token_ids == p.output_token_ids and p.logprobs is None
        assert len(o.logprobs) == 6
        for tok, (lp, top) in zip(o.output_token_ids, o.logprobs):
            assert len(top) == sp.logprobs and lp <= 0.0
            assert top[0][0] == tok and abs(top[0][1] - lp) < 1e-6          # greedy: the sampled token leads
            assert all(a[1] >= b[1] for a, b in zip(top, top[1:]))
            assert sum(math.exp(v) for _, v in top) <= 1.0 + 1e-5


def test_mixed_batch_of_requests_with_and_without_logprobs_and_sampling():
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(1, 97, (n,), generator=g).tolist() for n in (8, 12)]
    sps = [SamplingParams(max_tokens=5, ignore_eos=True),
           SamplingParams(max_tokens=5, ignore_eos=True, temperature=0.8, seed=7, logprobs=2)]
    outs = _llm().generate(prompts, sps)
    assert outs[0].logprobs is None and len(outs[1].logprobs) == 5
    for tok, (lp, top) in zip(outs[1].output_token_ids, outs[1].logprobs):
        # a sampled token need not be the most likely one, but its log-probability is that of the
        # model's distribution: never above the leader's
        assert lp <= top[0][1] + 1e-6
        if tok == top[0][0]:
            assert abs(lp - top[0][1]) < 1e-6


def test_logprobs_with_speculative_decoding_are_refused():
    llm = _llm(speculative_config={"method": "ngram", "num_speculative_tokens": 2})
    with pytest.raises(ValueError):
        llm.generate([[1, 2, 3]], SamplingParams(max_tokens=2, logprobs=1))


def test_logit_bias_and_min_tokens_shape_what_is_sampled():
    prompts = [[5, 6, 7, 8]]
    free = _llm().generate(prompts, SamplingParams(max_tokens=4, ignore_eos=True))[0].output_token_ids
    # a large bias makes a token win; a large negative one bans the token greedy decoding would pick
    forced = _llm().generate(prompts, SamplingParams(max_tokens=4, ignore_eos=True, logit_bias={42: 100.0}))[0]
    assert forced.output_token_ids == [42] * 4
    banned = _llm().generate(prompts, SamplingParams(max_tokens=4, ignore_eos=True, logit_bias={free[0]: -100.0}))[0]
    assert banned.output_token_ids[0] != free[0]
    # stop token = the first free token: without min_tokens the request ends at once, with it only later
    stops = SamplingParams(max_tokens=6, stop_token_ids=(free[0],))
    assert _llm().generate(prompts, stops)[0].output_token_ids == [free[0]]
    held = _llm().generate(prompts, SamplingParams(max_tokens=6, stop_token_ids=(free[0],), min_tokens=3))[0]
    assert len(held.output_token_ids) >= 3 and free[0] not in held.output_token_ids[:3]


def test_allowed_token_ids_and_min_p_restrict_the_candidates():
    prompts = [[5, 6, 7, 8]]
    only = _llm().generate(prompts, SamplingParams(max_tokens=5, ignore_eos=True, temperature=1.0, seed=1,
                                                    allowed_token_ids=[10, 11, 12]))[0]
    assert set(only.output_token_ids) <= {10, 11, 12}
    # min_p = 1: only the most likely token survives, so sampling at any temperature is greedy decoding
    greedy = _llm().generate(prompts, SamplingParams(max_tokens=5, ignore_eos=True))[0].output_token_ids
    hot = _llm().generate(prompts, SamplingParams(max_tokens=5, ignore_eos=True, temperature=5.0, seed=3, min_p=1.0))[0]
    assert hot.output_token_ids == greedy


def test_bad_words_ban_a_token_only_after_its_prefix():
    prompts = [[5, 6, 7, 8]]
    free = _llm().generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))[0].output_token_ids
    # a one-token word is banned everywhere
    one = _llm().generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True, bad_words_token_ids=[[free[0]]]))[0]
    assert free[0] not in one.output_token_ids
    # a two-token word: its first token may come, the second not right after it
    two = _llm().generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True,
                                                  bad_words_token_ids=[[free[1], free[2]]]))[0].output_token_ids
    assert two[:2] == free[:2] and two[2] != free[2]
    # a word whose prefix never appears changes nothing
    same = _llm().generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True,
                                                   bad_words_token_ids=[[96, free[0]]]))[0].output_token_ids
    assert same == free


def test_server_turns_bad_words_into_token_sequences():
    from omni_npu_b200.serving.api_server import bad_words_token_ids, sampling_from_body

    class Tok:
        def encode(self, text, add_special_tokens=False):
            return [100 + len(text)] if text.startswith(" ") else [len(text)]
    assert bad_words_token_ids(["abc", " de"], Tok()) == [[3], [104], [2], [103]]
    assert sampling_from_body({"bad_words": ["abc"]}, Tok()).bad_words_token_ids == [[3], [104]]
    assert sampling_from_body({}, None).bad_words_token_ids is None
    with pytest.raises(ValueError, match="tokenizer"):
        sampling_from_body({"bad_words": ["abc"]}, None)


def test_prompt_logprobs_match_a_plain_forward_pass_across_chunks():
    prompt = list(range(3, 3 + 23))
    # a token budget of 8 splits the prompt into three chunks
    llm = LLM(model=_cfg(), device="cpu", max_num_seqs=4, max_num_batched_tokens=8, max_model_len=128, block_size=4,
              num_gpu_blocks=64, seed=3, enable_prefix_caching=True)
    out = llm.generate([prompt, [7, 8, 9]], [SamplingParams(max_tokens=2, ignore_eos=True, prompt_logprobs=3),
                                             SamplingParams(max_tokens=2, ignore_eos=True)])
    plp = out[0].prompt_logprobs
    assert out[1].prompt_logprobs is None and len(plp) == len(prompt) and plp[0] is None
    model = llm.engine.worker.model_runner.model
    # the oracle: one unchunked pass of the same engine over the prompt, reading every row's logits
    one = LLM(model=_cfg(), device="cpu", max_num_seqs=1, max_num_batched_tokens=64, max_model_len=128, block_size=4,
              num_gpu_blocks=64, seed=3)
    one.engine.worker.model_runner.model.load_state_dict(model.state_dict())
    ref = one.generate([prompt], SamplingParams(max_tokens=1, ignore_eos=True, prompt_logprobs=0))[0].prompt_logprobs
    for j in range(1, len(prompt)):
        lp, top = plp[j]
        assert lp == pytest.approx(ref[j][0], abs=1e-4) and ref[j][1] == []
        assert len(top) == 3 and top[0][1] >= top[1][1] >= top[2][1] and lp <= top[0][1] + 1e-6
    # an independent path: force prompt[j] as the first generated token after prompt[:j] and read its log-probability
    for j in (1, 9, 22):
        forced = one.generate([prompt[:j]], SamplingParams(max_tokens=1, ignore_eos=True, logprobs=1,
                                                           allowed_token_ids=[prompt[j]]))[0]
        assert forced.output_token_ids == [prompt[j]]
        assert forced.logprobs[0][0] == pytest.approx(plp[j][0], abs=1e-4)
    # asking again hits no cached prefix (such requests always run their whole prompt) and gives the same values
    again = llm.generate([prompt], SamplingParams(max_tokens=1, ignore_eos=True, prompt_logprobs=0))[0].prompt_logprobs
    assert [e[0] for e in again[1:]] == pytest.approx([e[0] for e in plp[1:]], abs=1e-5)
    with pytest.raises(ValueError, match="prompt_logprobs"):
        llm.generate([prompt], SamplingParams(max_tokens=1, prompt_logprobs=21))


def test_server_returns_prompt_logprobs():
    from starlette.testclient import TestClient

    from omni_npu_b200.serving.api_server import build_app
    app = build_app(_llm(), None, "tiny")
    with TestClient(app) as c:
        r = c.post("/v1/completions", json={"prompt": [5, 6, 7, 8], "max_tokens": 2, "ignore_eos": True, "prompt_logprobs": 2})
        assert r.status_code == 200, r.text
        plp = r.json()["choices"][0]["prompt_logprobs"]
        assert plp[0] is None and len(plp) == 4
        assert all("%d" % t in e and 2 <= len(e) <= 3 and max(e.values()) <= 0.0 for t, e in zip([6, 7, 8], plp[1:]))
        r = c.post("/v1/completions", json={"prompt": [5, 6, 7, 8], "max_tokens": 2, "ignore_eos": True})
        assert "prompt_logprobs" not in r.json()["choices"][0]
        assert c.post("/v1/completions", json={"prompt": [5, 6], "max_tokens": 1, "prompt_logprobs": 50}).status_code == 400
    app.state.engine_loop.shutdown()
