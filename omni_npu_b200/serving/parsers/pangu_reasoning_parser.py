"""Reasoning parser for Pangu models.

The reasoning span is enclosed in ``<think>`` ... ``</think>`` when the
tokenizer knows those tokens, else in ``[unused16]`` ... ``[unused17]``
(omni_npu/v1/parsers/pangu_reasoning_parser.py:11-74).  Output before the end
marker is reasoning, everything after it is content; a start marker is optional
(models often open the span implicitly).  Streaming handles the start marker
and the first reasoning text arriving in one chunk, and the end marker splitting
a chunk into reasoning and content.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Sequence, Tuple


@dataclass
class DeltaMessage:
    reasoning: Optional[str] = None
    content: Optional[str] = None

    @property
    def reasoning_content(self) -> Optional[str]:      # name used by older OpenAI-compatible servers
        return self.reasoning


class PanguReasoningParser:
    def __init__(self, tokenizer) -> None:
        self.vocab: Dict[str, int] = dict(tokenizer.get_vocab()) if tokenizer is not None else {}
        self.start_token = "<think>" if "<think>" in self.vocab else "[unused16]"
        self.end_token = "</think>" if "</think>" in self.vocab else "[unused17]"
        self.start_token_id = self.vocab.get(self.start_token)
        self.end_token_id = self.vocab.get(self.end_token)
        if self.end_token_id is None:
            raise RuntimeError("the tokenizer has neither </think> nor [unused17]: "
                               "cannot locate the end of the reasoning span")
        self._end_seen = 0

    # ------------------------------------------------------------ one shot
    def extract_reasoning(self, model_output: str) -> Tuple[Optional[str], Optional[str]]:
        """(reasoning, content) of a complete response."""
        text = model_output
        if self.start_token in text:
            text = text.split(self.start_token, 1)[1]
        if self.end_token not in text:
            return (text or None), None
        reasoning, content = text.split(self.end_token, 1)
        return (reasoning or None), (content or None)

    def is_reasoning_end(self, input_ids: Sequence[int], delta_token_ids: Optional[Sequence[int]] = None) -> bool:
        """True from the step in which the end marker is generated (not when it merely
        appears in the prompt)."""
        if delta_token_ids is None:
            return self.end_token_id in input_ids
        if self.end_token_id in input_ids and self.end_token_id in delta_token_ids:
            self._end_seen += 1
        return self._end_seen >= 1

    def extract_content_ids(self, input_ids: Sequence[int]) -> list:
        ids = list(input_ids)
        if self.end_token_id not in ids[:-1]:
            return []
        return ids[ids.index(self.end_token_id) + 1:]

    # ------------------------------------------------------------ streaming
    def extract_reasoning_streaming(self, previous_text: str, current_text: str, delta_text: str,
                                    previous_token_ids: Sequence[int], current_token_ids: Sequence[int],
                                    delta_token_ids: Sequence[int]) -> Optional[DeltaMessage]:
        start_id, end_id = self.start_token_id, self.end_token_id
        if len(delta_token_ids) == 1 and delta_token_ids[0] in (start_id, end_id):
            return None                                   # a bare marker carries no text
        if end_id in previous_token_ids:
            return DeltaMessage(content=delta_text)       # span already closed
        if end_id in delta_token_ids:
            head, tail = delta_text.split(self.end_token, 1)
            if self.start_token in head:
                head = head.split(self.start_token, 1)[1]
            return DeltaMessage(reasoning=head or None, content=tail or None)
        if start_id is not None and start_id in delta_token_ids:
            # start marker and first reasoning text in one chunk
            return DeltaMessage(reasoning=delta_text.split(self.start_token, 1)[1])
        return DeltaMessage(reasoning=delta_text)
