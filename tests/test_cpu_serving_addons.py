"""Parsers, reasoning configuration, thinking-budget logits processor, patch framework."""
import json
import types

import pytest
import torch

from omni_npu_b200.patches.core import Patch, PatchRegistry, register_patch
from omni_npu_b200.sample.logits_processors import ThinkingTokenBudgetLogitsProcessor, find_last
from omni_npu_b200.serving.parsers import PanguReasoningParser, PanguToolParser
from omni_npu_b200.serving.parsers.pangu_tool_parser import partial_json_loads
from omni_npu_b200.serving.reasoning_config import ReasoningConfig


class Tok:
    def __init__(self, vocab):
        self.vocab = vocab

    def get_vocab(self):
        return self.vocab

    def tokenize(self, text):
        return [text]

    def convert_tokens_to_ids(self, toks):
        return [self.vocab[t] for t in toks]


# ------------------------------------------------------------------- reasoning
def test_reasoning_parser_picks_markers_and_splits():
    p = PanguReasoningParser(Tok({"<think>": 1, "</think>": 2}))
    assert (p.start_token, p.end_token) == ("<think>", "</think>")
    assert p.extract_reasoning("<think>why</think>answer") == ("why", "answer")
    assert p.extract_reasoning("why</think>answer") == ("why", "answer")
    assert p.extract_reasoning("still thinking") == ("still thinking", None)
    old = PanguReasoningParser(Tok({"[unused16]": 5, "[unused17]": 6}))
    assert (old.start_token, old.end_token) == ("[unused16]", "[unused17]")
    with pytest.raises(RuntimeError):
        PanguReasoningParser(Tok({"x": 1}))
    assert p.extract_content_ids([1, 9, 2, 7, 8]) == [7, 8]


def test_reasoning_parser_streaming():
    p = PanguReasoningParser(Tok({"<think>": 1, "</think>": 2}))
    d = p.extract_reasoning_streaming("", "<think>Hello", "<think>Hello", [], [1, 10], [1, 10])
    assert d.reasoning == "Hello" and d.content is None
    assert p.extract_reasoning_streaming("", "<think>", "<think>", [], [1], [1]) is None
    d = p.extract_reasoning_streaming("<think>a", "<think>ab</think>c", "b</think>c", [1, 10], [1, 10, 11, 2, 12], [11, 2, 12])
    assert (d.reasoning, d.content) == ("b", "c")
    d = p.extract_reasoning_streaming("<think>ab</think>c", "<think>ab</think>cd", "d", [1, 10, 2, 12], [1, 10, 2, 12, 13], [13])
    assert (d.reasoning, d.content) == (None, "d")
    assert not p.is_reasoning_end([1, 2, 3], [3])
    assert p.is_reasoning_end([1, 3, 2], [2])


# ------------------------------------------------------------------ tool calls
def test_tool_parser_one_shot():
    p = PanguToolParser(Tok({"<|tool_call_start|>": 1, "<|tool_call_end|>": 2}))
    out = p.extract_tool_calls('Let me check.<|tool_call_start|>[{"name": "get_weather", "arguments": {"city": "Paris"}},'
                               ' {"name": "now", "arguments": {}}]<|tool_call_end|>')
    assert out.tools_called and out.content == "Let me check."
    assert [c.function.name for c in out.tool_calls] == ["get_weather", "now"]
    assert json.loads(out.tool_calls[0].function.arguments) == {"city": "Paris"}
    plain = p.extract_tool_calls("no tools here")
    assert not plain.tools_called and plain.content == "no tools here"
    broken = p.extract_tool_calls("<|tool_call_start|>[{oops<|tool_call_end|>")
    assert not broken.tools_called
    assert PanguToolParser(Tok({"[unused11]": 3, "[unused12]": 4})).tool_call_start_token == "[unused11]"


def test_partial_json():
    assert partial_json_loads('[{"name": "f", "arguments": {"a": 1') == [{"name": "f", "arguments": {"a": 1}}]
    assert partial_json_loads('[{"name": "ge') == [{"name": "ge"}]
    assert partial_json_loads("") is None


def test_tool_parser_streaming_reassembles_arguments():
    p = PanguToolParser(Tok({"<|tool_call_start|>": 1, "<|tool_call_end|>": 2}))
    chunks = ["Sure. ", "<|tool_call_start|>", '[{"name": "get_', 'weather", "argum', 'ents": {"city": "Pa', 'ris", "days": 3}}]',
              "<|tool_call_end|>"]
    ids = [[10], [1], [11], [12], [13], [14], [2]]
    prev, prev_ids = "", []
    content, name, args = "", None, ""
    for ch, i in zip(chunks, ids):
        cur, cur_ids = prev + ch, prev_ids + i
        d = p.extract_tool_calls_streaming(prev, cur, ch, prev_ids, cur_ids, i)
        if d is not None:
            content += d.content or ""
            for tc in d.tool_calls:
                if tc.function.name:
                    name = tc.function.name
                args += tc.function.arguments or ""
        prev, prev_ids = cur, cur_ids
    assert content == "Sure. " and name == "get_weather"
    assert json.loads(args) == {"city": "Paris", "days": 3}


# --------------------------------------------------------------- think budget
def test_reasoning_config_and_budget_processor():
    cfg = ReasoningConfig.from_cli('{"think_start_str": "<think>", "think_end_str": "</think>"}')
    assert not cfg.is_thinking_enabled
    cfg.initialize_token_ids(Tok({"<think>": 1, "</think>": 2}))
    assert cfg.is_thinking_enabled and cfg.think_end_token_ids == [2]
    assert find_last([1, 5, 1, 6], [1]) == 2 and find_last([3], []) == -1

    lp = ThinkingTokenBudgetLogitsProcessor(cfg)
    lp.add_request("a", [9, 1], budget=2)          # prompt ends inside an open span
    lp.add_request("b", [9, 9], budget=2)          # not thinking
    lp.add_request("c", [9], budget=None)          # no budget: untouched
    outs = {"a": [], "b": [], "c": []}

    def step(tokens):
        logits = torch.zeros(3, 8)
        logits = lp.apply(logits, ["a", "b", "c"], [outs["a"], outs["b"], outs["c"]])
        for rid, t, row in zip("abc", tokens, logits):
            forced = torch.isinf(row).sum().item() == 7
            outs[rid].append(int(row.argmax()) if forced else t)
        return logits

    step([5, 1, 5])        # a: think 1/2 ; b opens a span
    step([5, 5, 5])        # a: think 2/2 -> next token forced ; b: 1/2
    l3 = step([5, 5, 5])   # a forced to </think> ; b: 2/2
    assert outs["a"][2] == 2 and torch.isinf(l3[0]).sum() == 7
    l4 = step([5, 5, 5])   # b forced now, a free again
    assert outs["b"][3] == 2 and not torch.isinf(l4[0]).any() and not torch.isinf(l4[2]).any()
    lp.remove_request("a")
    assert "a" not in lp.state


# ------------------------------------------------------------- patch framework
def test_patch_registry_apply_conflict_and_revert(monkeypatch):
    class Target:
        def f(self):
            return "orig"

    mod = types.ModuleType("fake_mod")
    mod.g = lambda: "orig"

    @register_patch("T_F", Target)
    class PF(Patch):
        attributes = ["f", "extra"]

        def f(self):
            return "patched"

        @classmethod
        def extra(cls):
            return cls.__name__

    @register_patch("T_F2", Target)
    class PF2(Patch):
        attributes = ["f"]

        def f(self):
            return "again"

    @register_patch("M_G", mod)
    class PG(Patch):
        attributes = ["g"]

        @staticmethod
        def g():
            return "patched"

    reg = PatchRegistry()
    monkeypatch.setenv("OMNI_B200_VLLM_PATCHES", "T_F, M_G,T_F2,Nope")
    reg.apply_from_env()
    assert reg.applied == ["T_F", "M_G"] and set(reg.failed) == {"T_F2", "Nope"}
    assert Target().f() == "patched" and Target.extra() == "Target" and mod.g() == "patched"
    reg.revert_all()
    assert Target().f() == "orig" and not hasattr(Target, "extra") and mod.g() == "orig"
    with pytest.raises(TypeError):
        register_patch("bad", 3)
    for n in ("T_F", "T_F2", "M_G"):
        PatchRegistry.registered.pop(n)


def test_hello_world_patch_and_auto_import(monkeypatch, tmp_path):
    import omni_npu_b200.patches as patches
    from omni_npu_b200.engine.request import Request
    import omni_npu_b200.patches.examples.hello_world  # noqa: F401
    reg = PatchRegistry()
    assert reg.apply_patch("HelloWorldRequest")
    assert Request("r7", [1]).hello() == "hello from request r7"
    reg.revert_all()
    assert not hasattr(Request, "hello")
    (tmp_path / "config.json").write_text('{"model_type": "deepseek_v3"}')
    assert patches.detect_model_type(["vllm", "serve", str(tmp_path)]) == "deepseek_v3"
    assert patches.detect_model_type(["x", "--model", str(tmp_path)]) == "deepseek_v3"
    assert "engine_args" in patches.auto_import_patches(["vllm", "serve", str(tmp_path)])
