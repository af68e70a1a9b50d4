"""The thinking-token budget as a vLLM V1 logits processor.

vLLM keeps a persistent batch and tells its logits processors how rows are added, removed
and moved (``BatchUpdate``); the processor itself only sees row indices.  This adapter maps
rows to the per-request state machines of ``ThinkingTokenBudgetLogitsProcessor`` and reads
each request's budget from ``SamplingParams.extra_args["thinking_token_budget"]``.  The
reasoning markers come from ``additional_config["reasoning_config"]`` of the vLLM config
(the ``--reasoning-config`` flag added by ``patches/common/engine_args.py``).

Pass it to vLLM with ``--logits-processors
omni_npu_b200.sample.vllm_logits_processor:ThinkingBudgetLogitsProcessor``.
Counterpart of omni_npu/v1/sample/logits_processor/thinking_token_budget_logits_processor.py:18-272.
"""
from __future__ import annotations

import itertools
from typing import Dict, List, Optional, Tuple

import torch

from .. import compat
from ..serving.reasoning_config import ReasoningConfig
from .logits_processors import ThinkingTokenBudgetLogitsProcessor

if compat.vllm_available():
    from vllm.v1.sample.logits_processor import LogitsProcessor as _Base
    from vllm.v1.sample.logits_processor import MoveDirectionality
else:                                            # pragma: no cover - exercised only without vLLM
    _Base = object
    MoveDirectionality = None

BUDGET_KEY = "thinking_token_budget"


def reasoning_config_from_vllm(vllm_config) -> Optional[ReasoningConfig]:
    extra = getattr(vllm_config, "additional_config", None) or {}
    cfg = extra.get("reasoning_config") if isinstance(extra, dict) else None
    if not cfg:
        return None
    return cfg if isinstance(cfg, ReasoningConfig) else ReasoningConfig(**cfg)


class ThinkingBudgetLogitsProcessor(_Base):
    def __init__(self, vllm_config=None, device: Optional[torch.device] = None, is_pin_memory: bool = False,
                 reasoning_config: Optional[ReasoningConfig] = None) -> None:
        cfg = reasoning_config if reasoning_config is not None else reasoning_config_from_vllm(vllm_config)
        self.inner = ThinkingTokenBudgetLogitsProcessor(cfg, device=device)
        self._ids = itertools.count()
        self.rows: Dict[int, Tuple[str, List[int]]] = {}      # batch row -> (state key, live output token list)

    @classmethod
    def validate_params(cls, sampling_params) -> None:
        extra = getattr(sampling_params, "extra_args", None) or {}
        budget = extra.get(BUDGET_KEY)
        if budget is not None and (not isinstance(budget, int) or budget < 0):
            raise ValueError(f"{BUDGET_KEY} must be a non-negative integer, got {budget!r}")

    def is_argmax_invariant(self) -> bool:
        return False

    def _drop(self, row: int) -> None:
        old = self.rows.pop(row, None)
        if old is not None:
            self.inner.remove_request(old[0])

    def update_state(self, batch_update) -> None:
        if batch_update is None:
            return
        for row in batch_update.removed:
            self._drop(row)
        for row, params, prompt_ids, output_ids in batch_update.added:
            self._drop(row)
            extra = getattr(params, "extra_args", None) or {}
            budget = extra.get(BUDGET_KEY)
            if budget is None or not self.inner.enabled:
                continue
            key = f"row{next(self._ids)}"
            self.inner.add_request(key, list(prompt_ids or []), int(budget))
            self.rows[row] = (key, output_ids)
        for a, b, direction in batch_update.moved:
            ra, rb = self.rows.pop(a, None), self.rows.pop(b, None)
            swap = MoveDirectionality is not None and direction == MoveDirectionality.SWAP
            if ra is not None:
                self.rows[b] = ra
            elif rb is not None and not swap:
                self.inner.remove_request(rb[0])          # overwritten by a row without a budget
            if swap and rb is not None:
                self.rows[a] = rb
            elif not swap and ra is not None and rb is not None:
                self.inner.remove_request(rb[0])

    def apply(self, logits: torch.Tensor) -> torch.Tensor:
        if not self.rows:
            return logits
        order = sorted(r for r in self.rows if r < logits.shape[0])
        if not order:
            return logits
        idx = torch.tensor(order, device=logits.device)
        sub = logits.index_select(0, idx)
        sub = self.inner.apply(sub, [self.rows[r][0] for r in order], [self.rows[r][1] for r in order])
        logits.index_copy_(0, idx, sub)
        return logits
