"""Structured outputs in the standalone engine: a request may restrict its output to a choice of
strings, a JSON schema (or any JSON object), a regular expression or an EBNF grammar.

The grammar engine is the ``xgrammar`` package (a library: it compiles the grammar against the
tokenizer's vocabulary and, per request, tells which tokens may come next as a bitmask of
ceil(vocab / 32) int32 words).  This module keeps one matcher per request, feeds it the tokens the
request has produced since the last step and masks the request's logits row before sampling.
Every tensor-parallel rank runs the same matchers on the same tokens, so the ranks keep sampling
the same token.  (The reference leaves structured outputs to vLLM's scheduler, which does the same
with the same package; under vLLM this package's worker applies vLLM's bitmask instead:
``worker/vllm_worker.py:grammar_mask_fn``.)
"""
from __future__ import annotations

import json
from typing import Any, Dict, Optional, Sequence

import torch


def _ebnf_string(s: str) -> str:
    return '"' + s.replace("\\", "\\\\").replace('"', '\\"').replace("\n", "\\n") + '"'


class StructuredOutputManager:
    KINDS = ("choice", "json_schema", "json_object", "regex", "grammar")

    def __init__(self, tokenizer, vocab_size: int) -> None:
        import xgrammar as xgr
        self.xgr = xgr
        self.vocab_size = int(vocab_size)
        self.info = xgr.TokenizerInfo.from_huggingface(tokenizer, vocab_size=self.vocab_size)
        self.compiler = xgr.GrammarCompiler(self.info)
        self.stop_token_ids = [int(t) for t in (getattr(self.info, "stop_token_ids", None) or [])]
        self._compiled: Dict[str, Any] = {}
        self._matchers: Dict[str, Any] = {}
        self._fed: Dict[str, int] = {}           # output tokens already given to a request's matcher

    # ------------------------------------------------------------------ grammars
    @classmethod
    def check_spec(cls, spec: Dict[str, Any]) -> None:
        if not isinstance(spec, dict) or len(spec) != 1 or next(iter(spec)) not in cls.KINDS:
            raise ValueError(f"structured output: exactly one of {cls.KINDS} is expected, got {spec!r}")
        if "choice" in spec and (not spec["choice"] or not all(isinstance(c, str) and c for c in spec["choice"])):
            raise ValueError("structured output: 'choice' needs a non-empty list of non-empty strings")

    def compile(self, spec: Dict[str, Any]):
        self.check_spec(spec)
        key = json.dumps(spec, sort_keys=True)
        got = self._compiled.get(key)
        if got is not None:
            return got
        kind, val = next(iter(spec.items()))
        try:
            if kind == "choice":
                got = self.compiler.compile_grammar("root ::= " + " | ".join(_ebnf_string(c) for c in val))
            elif kind == "json_schema":
                got = self.compiler.compile_json_schema(val if isinstance(val, str) else json.dumps(val))
            elif kind == "json_object":
                got = self.compiler.compile_builtin_json_grammar()
            elif kind == "regex":
                got = self.compiler.compile_regex(val)
            else:
                got = self.compiler.compile_grammar(val)
        except Exception as e:                  # the grammar engine's own error types
            raise ValueError(f"structured output: cannot compile the {kind}: {e}") from e
        self._compiled[key] = got
        return got

    # ------------------------------------------------------------------ requests
    def has(self, rid: str) -> bool:
        return rid in self._matchers

    def add_request(self, rid: str, spec: Dict[str, Any]) -> None:
        self._matchers[rid] = self.xgr.GrammarMatcher(self.compile(spec))
        self._fed[rid] = 0

    def remove_request(self, rid: str) -> None:
        self._matchers.pop(rid, None)
        self._fed.pop(rid, None)

    def _sync(self, rid: str, output_token_ids: Sequence[int]) -> None:
        """Give the matcher the tokens produced since the last step.  A history shorter than what
        was fed (the request was recomputed from an earlier point) restarts the matcher."""
        m = self._matchers[rid]
        fed = self._fed[rid]
        if fed > len(output_token_ids):
            m.reset()
            fed = 0
        for t in output_token_ids[fed:]:
            if m.is_terminated():
                break
            if not m.accept_token(int(t)):
                # a token outside the grammar (cannot happen with the mask applied): stop constraining
                break
        self._fed[rid] = len(output_token_ids)

    def apply(self, logits: torch.Tensor, rids: Sequence[str], histories: Sequence[Sequence[int]]) -> torch.Tensor:
        """Mask row i of ``logits`` with what request ``rids[i]`` may produce next."""
        n = len(rids)
        bitmask = self.xgr.allocate_token_bitmask(n, self.vocab_size)
        for i, (rid, hist) in enumerate(zip(rids, histories)):
            self._sync(rid, hist)
            m = self._matchers[rid]
            if m.is_terminated():
                bitmask[i].fill_(-1)             # the grammar is complete: nothing left to constrain
            else:
                m.fill_next_token_bitmask(bitmask, i)
        vocab = logits.shape[-1]
        w = bitmask.to(logits.device)
        bits = (w.unsqueeze(-1) >> torch.arange(32, device=logits.device, dtype=torch.int32)) & 1
        allowed = bits.reshape(n, -1)[:, :vocab].bool()
        if allowed.shape[1] < vocab:
            allowed = torch.cat([allowed, allowed.new_zeros(n, vocab - allowed.shape[1])], dim=1)
        # a vocabulary that cannot continue the grammar (no token spells what must come next) would
        # leave a row with nothing to sample: such a request ends instead
        dead = ~allowed.any(dim=1)
        if bool(dead.any()) and self.stop_token_ids:
            allowed[dead.nonzero().flatten().unsqueeze(1), torch.tensor(self.stop_token_ids, device=allowed.device)] = True
        return logits.masked_fill(~allowed, float("-inf"))


def structured_spec_from_body(body: Dict[str, Any]) -> Optional[Dict[str, Any]]:
    """The structured-output request of an OpenAI-style body: ``structured_outputs: {choice | json |
    regex | grammar}``, the older ``guided_choice`` / ``guided_json`` / ``guided_regex`` /
    ``guided_grammar`` fields, or ``response_format`` of type ``json_object`` / ``json_schema``."""
    so = body.get("structured_outputs") or {}
    if so.get("choice") or body.get("guided_choice"):
        return {"choice": list(so.get("choice") or body["guided_choice"])}
    if so.get("json") or body.get("guided_json"):
        return {"json_schema": so.get("json") or body["guided_json"]}
    if so.get("regex") or body.get("guided_regex"):
        return {"regex": so.get("regex") or body["guided_regex"]}
    if so.get("grammar") or body.get("guided_grammar"):
        return {"grammar": so.get("grammar") or body["guided_grammar"]}
    rf = body.get("response_format") or {}
    if rf.get("type") == "json_object":
        return {"json_object": True}
    if rf.get("type") == "json_schema":
        js = rf.get("json_schema") or {}
        return {"json_schema": js.get("schema", js)}
    return None
