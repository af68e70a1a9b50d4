"""Streaming text while a request is inside its reasoning span.

With stop strings configured, an incremental detokenizer holds back the last
``stop_buffer_length`` characters of the output so that a stop string can still be removed
before the client sees it.  Stop strings are not meant to apply inside a reasoning span, and
holding text back there delays (and, when the request ends right after the span, truncates)
the closing marker.  Rule implemented here: nothing is held back while the request has not
finished reasoning, nor for the chunk that contains the closing marker.

"Finished reasoning" = the think-end token followed by a newline token was seen among the last
few output tokens (Qwen3: ``</think>`` 151668 then ``\\n\\n`` 271 / ``\\n`` 9612; DeepSeek-R1:
128799 then 201 / 271), or a reasoning config supplies other ids.

``hold_back`` is the pure rule; ``ThinkAwareDetokenizerPatch`` installs it on vLLM's
``BaseIncrementalDetokenizer.get_next_output_text`` (patch name ``ThinkingStopBufferPatch``).
Same behaviour as omni_npu/v0/patches/thinking_tag_bug_fix_patch.py:37-91.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence, Tuple

from ... import compat
from ..core import Patch, register_patch

# think-end token id -> token ids that may follow it when the span is really over
DEFAULT_MARKERS: Dict[int, Tuple[int, ...]] = {
    151668: (271, 9612),        # Qwen3
    128799: (201, 271),         # DeepSeek-R1
}
WINDOW = 16
END_TEXT = "</think>"


def reasoning_finished(token_ids: Sequence[int], markers: Optional[Dict[int, Tuple[int, ...]]] = None) -> bool:
    """True once a think-end token followed by one of its successor tokens occurs in the tail."""
    tail = list(token_ids[-WINDOW:])
    if len(tail) <= 1:
        return False
    for end_id, after in (markers or DEFAULT_MARKERS).items():
        if end_id in tail:
            i = tail.index(end_id) + 1
            if i < len(tail) and tail[i] in after:
                return True
    return False


def hold_back(stop_buffer_length: int, finished: bool, done_reasoning: bool, new_text: str) -> int:
    """How many trailing characters to keep from the client for now."""
    if finished or not done_reasoning or END_TEXT in new_text:
        return 0
    return stop_buffer_length


if compat.vllm_available():
    try:
        from vllm.v1.engine.detokenizer import BaseIncrementalDetokenizer as _Detok

        @register_patch("ThinkingStopBufferPatch", _Detok)
        class ThinkAwareDetokenizerPatch(Patch):
            attributes = ["get_next_output_text", "is_cot_end"]

            def is_cot_end(self) -> bool:
                if getattr(self, "_cot_end_seen", False):
                    return True
                if reasoning_finished(self.token_ids):
                    self._cot_end_seen = True
                return getattr(self, "_cot_end_seen", False)

            def get_next_output_text(self, finished: bool, delta: bool) -> str:
                text = self.output_text
                keep = hold_back(self.stop_buffer_length, finished, self.is_cot_end(),
                                 text[self._last_output_text_offset:])
                if not delta:
                    return text[:-keep] if keep else text
                length = len(text) - keep
                last = self._last_output_text_offset
                if last < length:
                    self._last_output_text_offset = length
                    return text[last:length]
                return ""
    except Exception:  # pragma: no cover - depends on the vLLM version
        pass
