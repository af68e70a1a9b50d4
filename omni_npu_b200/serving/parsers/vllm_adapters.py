"""Adapters that expose the Pangu parsers through vLLM's parser base classes, so
that ``--reasoning-parser pangu`` / ``--tool-call-parser pangu`` work in
``vllm serve``.  Imported lazily (only when vLLM asks for the parser)."""
from __future__ import annotations

from ... import compat
from .pangu_reasoning_parser import PanguReasoningParser
from .pangu_tool_parser import PanguToolParser

_ReasoningBase = compat.try_import("vllm.reasoning:ReasoningParser")
_ToolBase = compat.try_import("vllm.tool_parsers:ToolParser",
                              "vllm.entrypoints.openai.tool_parsers:ToolParser")


class VllmPanguReasoningParser(_ReasoningBase):
    def __init__(self, tokenizer, *args, **kwargs):
        super().__init__(tokenizer, *args, **kwargs)
        self._impl = PanguReasoningParser(tokenizer)

    def is_reasoning_end(self, input_ids):
        return self._impl.is_reasoning_end(input_ids)

    def extract_content_ids(self, input_ids):
        return self._impl.extract_content_ids(input_ids)

    def extract_reasoning(self, model_output, request=None):
        return self._impl.extract_reasoning(model_output)

    extract_reasoning_content = extract_reasoning

    def extract_reasoning_streaming(self, previous_text, current_text, delta_text, previous_token_ids,
                                    current_token_ids, delta_token_ids):
        d = self._impl.extract_reasoning_streaming(previous_text, current_text, delta_text, previous_token_ids,
                                                   current_token_ids, delta_token_ids)
        if d is None:
            return None
        DeltaMessage = compat.try_import("vllm.entrypoints.openai.protocol:DeltaMessage",
                                         "vllm.entrypoints.openai.chat_completion.protocol:DeltaMessage")
        try:
            return DeltaMessage(reasoning=d.reasoning, content=d.content)
        except Exception:
            return DeltaMessage(reasoning_content=d.reasoning, content=d.content)

    extract_reasoning_content_streaming = extract_reasoning_streaming


class VllmPanguToolParser(_ToolBase):
    def __init__(self, tokenizer, *args, **kwargs):
        super().__init__(tokenizer, *args, **kwargs)
        self._impl = PanguToolParser(tokenizer)

    def extract_tool_calls(self, model_output, request=None):
        return self._impl.extract_tool_calls(model_output)

    def extract_tool_calls_streaming(self, previous_text, current_text, delta_text, previous_token_ids,
                                     current_token_ids, delta_token_ids, request=None):
        return self._impl.extract_tool_calls_streaming(previous_text, current_text, delta_text,
                                                       previous_token_ids, current_token_ids, delta_token_ids)
