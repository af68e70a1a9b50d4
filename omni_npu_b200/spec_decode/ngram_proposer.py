"""Prompt-lookup drafts: find the most recent earlier occurrence of the request's last
n tokens (n from ``max_n`` down to ``min_n``) and propose the k tokens that followed it.
Runs on the host over the token lists; no model involved, so it works for every model
family and exercises the whole verification path.

The reference reaches the same proposer through vLLM's spec-decode configuration
(``--speculative-config '{"method": "ngram", ...}'``); its own code only adapts the
model-based proposer (omni_npu/vllm_patches/patches/common/patch_eagle.py:35-724).
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np


class NgramProposer:
    needs_hidden_states = False

    def __init__(self, k: int, min_n: int = 2, max_n: int = 4) -> None:
        assert k >= 1 and 1 <= min_n <= max_n
        self.k, self.min_n, self.max_n = k, min_n, max_n

    def propose_one(self, tokens: Sequence[int]) -> List[int]:
        arr = np.asarray(tokens, dtype=np.int64)
        total = arr.shape[0]
        for n in range(min(self.max_n, total - 1), self.min_n - 1, -1):
            tail = arr[total - n:]
            # windows that end before the tail itself begins
            limit = total - n
            if limit <= 0:
                continue
            win = np.lib.stride_tricks.sliding_window_view(arr[: total - 1], n)[:limit]
            hits = np.nonzero((win == tail).all(axis=1))[0]
            if hits.size:
                start = int(hits[-1]) + n          # most recent match
                out = arr[start: start + self.k].tolist()
                if out:
                    return out
        return []

    def propose(self, requests, sampled=None, hidden=None) -> List[List[int]]:
        return [self.propose_one(r.all_token_ids) for r in requests]
