"""Reasoning ("thinking") configuration: which strings / token ids open and close a
model's reasoning span.  Needed by the thinking-token-budget logits processor.
Counterpart of omni_npu/v1/config/reasoning_config.py:14-60."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional


@dataclass
class ReasoningConfig:
    think_start_str: Optional[str] = None
    think_end_str: Optional[str] = None
    think_start_token_ids: Optional[List[int]] = None
    think_end_token_ids: Optional[List[int]] = None

    @classmethod
    def from_cli(cls, value: Any) -> Optional["ReasoningConfig"]:
        """Accepts a dict, a JSON string or a path to a JSON file."""
        if value is None or isinstance(value, cls):
            return value
        if isinstance(value, str):
            value = json.load(open(value)) if os.path.exists(value) else json.loads(value)
        return cls(**{k: v for k, v in dict(value).items() if k in cls.__dataclass_fields__})

    @property
    def is_thinking_enabled(self) -> bool:
        return bool(self.think_start_token_ids) and bool(self.think_end_token_ids)

    def initialize_token_ids(self, tokenizer) -> None:
        """Derive token ids from the strings (ids given explicitly win)."""
        if tokenizer is None:
            return
        if self.think_start_str is not None and not self.think_start_token_ids:
            self.think_start_token_ids = _encode(tokenizer, self.think_start_str)
        if self.think_end_str is not None and not self.think_end_token_ids:
            self.think_end_token_ids = _encode(tokenizer, self.think_end_str)


def _encode(tokenizer, text: str) -> List[int]:
    if hasattr(tokenizer, "tokenize") and hasattr(tokenizer, "convert_tokens_to_ids"):
        return list(tokenizer.convert_tokens_to_ids(tokenizer.tokenize(text)))
    if hasattr(tokenizer, "encode"):
        try:
            return list(tokenizer.encode(text, add_special_tokens=False))
        except TypeError:
            return list(tokenizer.encode(text))
    vocab = tokenizer.get_vocab()
    return [vocab[text]] if text in vocab else []
