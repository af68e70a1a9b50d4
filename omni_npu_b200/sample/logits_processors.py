"""Logits processors.

``ThinkingTokenBudgetLogitsProcessor`` caps the number of tokens a request may
spend inside its reasoning span: once ``thinking_token_budget`` tokens have been
generated after the think-start marker, the think-end marker token(s) are
forced, one per step, by masking every other logit.  A per-request state
machine tracks the span over prompt and output tokens (prompts may already end
inside an open span).  Behaviourally equivalent to
omni_npu/v1/sample/logits_processor/thinking_token_budget_logits_processor.py:18-272.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..serving.reasoning_config import ReasoningConfig


def find_last(haystack: Sequence[int], needle: Sequence[int]) -> int:
    n = len(needle)
    if n == 0:
        return -1
    for i in range(len(haystack) - n, -1, -1):
        if list(haystack[i:i + n]) == list(needle):
            return i
    return -1


@dataclass
class _ThinkState:
    budget: int
    in_think: bool = False
    think_count: int = 0
    forcing: bool = False       # currently emitting the end marker
    end_emitted: int = 0        # how many end-marker tokens have been forced
    seen_outputs: int = 0


class ThinkingTokenBudgetLogitsProcessor:
    def __init__(self, reasoning_config: Optional[ReasoningConfig], max_num_seqs: int = 256,
                 device: Optional[torch.device] = None) -> None:
        self.cfg = reasoning_config
        self.enabled = reasoning_config is not None and reasoning_config.is_thinking_enabled
        self.start_ids: List[int] = list(reasoning_config.think_start_token_ids or []) if self.enabled else []
        self.end_ids: List[int] = list(reasoning_config.think_end_token_ids or []) if self.enabled else []
        self.state: Dict[str, _ThinkState] = {}
        self.device = device

    def is_argmax_invariant(self) -> bool:
        return False

    # ----------------------------------------------------------- bookkeeping
    def add_request(self, request_id: str, prompt_token_ids: Sequence[int], budget: Optional[int]) -> None:
        if not self.enabled or budget is None or budget < 0:
            return
        st = _ThinkState(budget=int(budget))
        ls, le = find_last(prompt_token_ids, self.start_ids), find_last(prompt_token_ids, self.end_ids)
        if ls > le:
            st.in_think = True
            st.think_count = len(prompt_token_ids) - (ls + len(self.start_ids))
            st.forcing = st.think_count >= st.budget
        self.state[request_id] = st

    def remove_request(self, request_id: str) -> None:
        self.state.pop(request_id, None)

    def _advance(self, st: _ThinkState, outputs: Sequence[int]) -> None:
        """Consume output tokens not seen yet."""
        for pos in range(st.seen_outputs, len(outputs)):
            upto = outputs[: pos + 1]
            if st.forcing:
                st.end_emitted += 1
                if st.end_emitted >= len(self.end_ids):
                    st.forcing, st.in_think, st.end_emitted, st.think_count = False, False, 0, 0
                continue
            if st.in_think:
                if len(upto) >= len(self.end_ids) and list(upto[-len(self.end_ids):]) == self.end_ids:
                    st.in_think, st.think_count = False, 0      # the model closed the span itself
                else:
                    st.think_count += 1
                    if st.think_count >= st.budget:
                        st.forcing = True
            elif len(upto) >= len(self.start_ids) and list(upto[-len(self.start_ids):]) == self.start_ids:
                st.in_think, st.think_count = True, 0
                st.forcing = st.budget == 0
        st.seen_outputs = len(outputs)

    # ----------------------------------------------------------------- apply
    def apply(self, logits: torch.Tensor, request_ids: Sequence[str],
              output_token_ids: Sequence[Sequence[int]]) -> torch.Tensor:
        """logits [B,V]; row i belongs to request_ids[i] whose generated tokens so far
        are output_token_ids[i].  Rows that must emit the end marker get every other
        logit set to -inf."""
        if not self.enabled or not self.state:
            return logits
        rows, toks = [], []
        for i, rid in enumerate(request_ids):
            st = self.state.get(rid)
            if st is None:
                continue
            self._advance(st, output_token_ids[i])
            if st.forcing:
                rows.append(i)
                toks.append(self.end_ids[min(st.end_emitted, len(self.end_ids) - 1)])
        if rows:
            r = torch.tensor(rows, device=logits.device)
            t = torch.tensor(toks, device=logits.device)
            keep = logits[r, t].clone()
            logits[r] = float("-inf")
            logits[r, t] = torch.where(torch.isinf(keep), torch.zeros_like(keep), keep)
        return logits
