"""Tool-call parser for Pangu models.

Tool calls are a JSON list between ``<|tool_call_start|>`` and
``<|tool_call_end|>`` (or ``[unused11]`` / ``[unused12]`` on older tokenizers):

    text before <|tool_call_start|>[{"name": "f", "arguments": {...}}, ...]<|tool_call_end|>

One-shot extraction returns the calls and the text before the first call.
Streaming re-parses the (possibly incomplete) JSON after every chunk with a
tolerant parser and emits, per tool, first its name and then the growing
arguments string as deltas (omni_npu/v1/parsers/pangu_tool_parser.py:26-284).
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence


@dataclass
class FunctionCall:
    name: Optional[str] = None
    arguments: Optional[str] = None


@dataclass
class ToolCall:
    function: FunctionCall
    id: str = field(default_factory=lambda: "chatcmpl-tool-" + uuid.uuid4().hex)
    type: str = "function"
    index: int = 0


@dataclass
class ExtractedToolCallInformation:
    tools_called: bool
    tool_calls: List[ToolCall]
    content: Optional[str]


@dataclass
class ToolDelta:
    content: Optional[str] = None
    tool_calls: List[ToolCall] = field(default_factory=list)


def partial_json_loads(text: str) -> Any:
    """Parse a JSON prefix: close open strings / brackets and retry, dropping the
    trailing incomplete member if necessary.  Returns None when nothing parses."""
    text = text.strip()
    if not text:
        return None
    for cut in range(len(text), 0, -1):
        cand = text[:cut]
        stack, in_str, esc = [], False, False
        for ch in cand:
            if in_str:
                if esc:
                    esc = False
                elif ch == "\\":
                    esc = True
                elif ch == '"':
                    in_str = False
            elif ch == '"':
                in_str = True
            elif ch in "[{":
                stack.append("]" if ch == "[" else "}")
            elif ch in "]}":
                if stack:
                    stack.pop()
        closed = cand + ('"' if in_str else "")
        closed = re.sub(r"[,:]\s*$", "", closed) if not in_str else closed
        closed += "".join(reversed(stack))
        try:
            return json.loads(closed)
        except json.JSONDecodeError:
            continue
    return None


def is_complete_json(text: str) -> bool:
    try:
        json.loads(text)
        return True
    except json.JSONDecodeError:
        return False


class PanguToolParser:
    def __init__(self, tokenizer) -> None:
        self.vocab: Dict[str, int] = dict(tokenizer.get_vocab()) if tokenizer is not None else {}
        self.tool_call_start_token = "<|tool_call_start|>" if "<|tool_call_start|>" in self.vocab else "[unused11]"
        self.tool_call_end_token = "<|tool_call_end|>" if "<|tool_call_end|>" in self.vocab else "[unused12]"
        self.tool_call_start_token_id = self.vocab.get(self.tool_call_start_token)
        self.tool_call_end_token_id = self.vocab.get(self.tool_call_end_token)
        if self.tool_call_start_token_id is None or self.tool_call_end_token_id is None:
            raise RuntimeError("the tokenizer lacks the Pangu tool-call marker tokens")
        self.tool_call_regex = re.compile(re.escape(self.tool_call_start_token) + "(.*?)" +
                                          re.escape(self.tool_call_end_token), re.DOTALL)
        # streaming state
        self.current_tool_id = -1
        self.current_tool_name_sent = False
        self.streamed_args: List[str] = []
        self.prev_tool_call_arr: List[Dict] = []

    # ------------------------------------------------------------- one shot
    def extract_tool_calls(self, model_output: str) -> ExtractedToolCallInformation:
        if self.tool_call_start_token not in model_output or self.tool_call_end_token not in model_output:
            return ExtractedToolCallInformation(False, [], model_output)
        try:
            calls: List[ToolCall] = []
            for blob in self.tool_call_regex.findall(model_output):
                parsed = json.loads(blob)
                for item in (parsed if isinstance(parsed, list) else [parsed]):
                    args = item.get("arguments", item.get("parameters", {}))
                    calls.append(ToolCall(FunctionCall(item["name"], json.dumps(args, ensure_ascii=False)),
                                          index=len(calls)))
            content = model_output[: model_output.find(self.tool_call_start_token)]
            return ExtractedToolCallInformation(bool(calls), calls, content or None)
        except Exception:
            return ExtractedToolCallInformation(False, [], model_output)

    # ------------------------------------------------------------ streaming
    def extract_tool_calls_streaming(self, previous_text: str, current_text: str, delta_text: str,
                                     previous_token_ids: Sequence[int], current_token_ids: Sequence[int],
                                     delta_token_ids: Sequence[int]) -> Optional[ToolDelta]:
        start, end = self.tool_call_start_token, self.tool_call_end_token
        if start not in current_text:
            return ToolDelta(content=delta_text)
        if len(delta_token_ids) == 1 and delta_token_ids[0] == self.tool_call_end_token_id:
            return self._flush(current_text)
        if end in current_text and end not in delta_text:
            return ToolDelta(content=delta_text)          # text after a finished call block
        if start in delta_text and start not in previous_text:
            before = delta_text.split(start, 1)[0]
            if before:
                return ToolDelta(content=before)
        portion = current_text.split(start)[-1].split(end)[0]
        arr = partial_json_loads(portion)
        if not isinstance(arr, list):
            arr = [arr] if isinstance(arr, dict) else []
        arr = [a for a in arr if isinstance(a, dict)]
        if not arr:
            return None
        out = ToolDelta()
        # a new element appeared: finish the previous one's arguments first
        while self.current_tool_id < len(arr) - 1:
            if self.current_tool_id >= 0:
                self._emit_args(arr[self.current_tool_id], out, final=True)
            self.current_tool_id += 1
            self.current_tool_name_sent = False
            self.streamed_args.append("")
        cur = arr[self.current_tool_id]
        if not self.current_tool_name_sent:
            name = cur.get("name")
            complete_name = isinstance(name, str) and (f'"{name}"' in portion)
            if complete_name:
                out.tool_calls.append(ToolCall(FunctionCall(name=name, arguments=""), index=self.current_tool_id))
                self.current_tool_name_sent = True
        if self.current_tool_name_sent:
            self._emit_args(cur, out, final=is_complete_json(portion) or end in delta_text)
        self.prev_tool_call_arr = arr
        return out if (out.tool_calls or out.content) else None

    def _emit_args(self, item: Dict, out: ToolDelta, final: bool) -> None:
        args = item.get("arguments", item.get("parameters"))
        if args is None:
            return
        text = json.dumps(args, ensure_ascii=False)
        if not final:
            # the tail of a partial dump may still change (closing brackets, open strings)
            text = text.rstrip('}]"')
        sent = self.streamed_args[self.current_tool_id]
        if text.startswith(sent) and len(text) > len(sent):
            out.tool_calls.append(ToolCall(FunctionCall(arguments=text[len(sent):]), index=self.current_tool_id,
                                           id=""))
            self.streamed_args[self.current_tool_id] = text

    def _flush(self, current_text: str) -> Optional[ToolDelta]:
        portion = current_text.split(self.tool_call_start_token)[-1].split(self.tool_call_end_token)[0]
        arr = partial_json_loads(portion)
        arr = arr if isinstance(arr, list) else ([arr] if isinstance(arr, dict) else [])
        out = ToolDelta()
        if 0 <= self.current_tool_id < len(arr) and self.current_tool_name_sent:
            self._emit_args(arr[self.current_tool_id], out, final=True)
        return out if out.tool_calls else None
