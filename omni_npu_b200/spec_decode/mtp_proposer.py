"""Drafts from the model's multi-token-prediction head.

The MTP layer runs inside the model runner right after the target model, in the same
step and (for decode) inside the same CUDA graph: it needs the target's hidden states
of every fed position and writes its own KV-cache layer at the same slots.  This class
only hands the drafts the runner produced to the engine.  With k > 1 draft tokens the head
is run k times in a chain (its own output and the token it just drafted are the input of the
next step, one position further; checkpoints with one MTP layer reuse it for every step), and
the scheduler keeps k - 1 cache slots past the scheduled tokens allocated for the chain's keys.

The reference reaches the same flow by overriding vLLM's EagleProposer for graph mode
(omni_npu/vllm_patches/patches/common/patch_eagle.py:35-724).
"""
from __future__ import annotations

from typing import List


class MTPProposer:
    needs_hidden_states = True

    def __init__(self, runner, k: int) -> None:
        self.runner = runner
        self.k = max(1, int(k))

    def propose(self, out, tokens) -> List[List[int]]:
        drafts = self.runner.last_drafts
        if len(drafts) != len(out.seqs):
            return [[] for _ in out.seqs]
        return drafts
