"""Drafts from the model's multi-token-prediction head.

The MTP layer runs inside the model runner right after the target model, in the same
step and (for decode) inside the same CUDA graph: it needs the target's hidden states
of every fed position and writes its own KV-cache layer at the same slots.  This class
only hands the drafts the runner produced to the engine.  One draft token per step
(the checkpoints carry one MTP layer); a larger request is clamped.

The reference reaches the same flow by overriding vLLM's EagleProposer for graph mode
(omni_npu/vllm_patches/patches/common/patch_eagle.py:35-724).
"""
from __future__ import annotations

from typing import List

from ..logger import logger


class MTPProposer:
    needs_hidden_states = True

    def __init__(self, runner, k: int) -> None:
        self.runner = runner
        if k > 1:
            logger.warning("the MTP head drafts one token per step; num_speculative_tokens=%d is clamped to 1", k)
        self.k = 1

    def propose(self, out, tokens) -> List[List[int]]:
        drafts = self.runner.last_drafts
        if len(drafts) != len(out.seqs):
            return [[] for _ in out.seqs]
        return drafts
