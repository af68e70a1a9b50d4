"""Sampler state that lives on the device across steps.

``PenaltyCache`` keeps, per request, the mask of prompt tokens and the occurrence counts of the
generated tokens, so that a decode step only adds the tokens sampled since the last step instead
of rebuilding [rows, vocab] tensors from the whole history.  ``ProbCache`` keeps the draft model's
top-k token ids and probabilities of the draft positions for the sparse rejection sampler.

Rows are addressed through stable slots: a request keeps its slot from admission to completion and
a step names the slots of its rows in an index tensor, so nothing is moved when the batch is
re-ordered (the reference permutes its cached rows to follow the batch order:
omni_npu/v0/layers/npu_sampler_cache.py:5-20,36-50).  Same role as ``PenaltyCache`` / ``ProbCache``
of omni_npu/v0/layers/npu_sampler_cache.py:22-145.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .sampler import apply_penalties


class _Slots:
    """Stable row numbers for request ids."""

    def __init__(self, capacity: int) -> None:
        self.capacity = capacity
        self.slot_of: Dict[str, int] = {}
        self.free: List[int] = list(range(capacity - 1, -1, -1))

    def acquire(self, request_id: str) -> int:
        s = self.slot_of.get(request_id)
        if s is not None:
            return s
        if not self.free:
            raise RuntimeError(f"sampler cache is full ({self.capacity} requests)")
        s = self.free.pop()
        self.slot_of[request_id] = s
        return s

    def release(self, request_id: str) -> Optional[int]:
        s = self.slot_of.pop(request_id, None)
        if s is not None:
            self.free.append(s)
        return s


class PenaltyCache:
    def __init__(self, max_requests: int, vocab_size: int, device) -> None:
        self.vocab_size = vocab_size
        self.device = torch.device(device)
        self.slots = _Slots(max_requests)
        self.prompt_mask = torch.zeros(max_requests, vocab_size, dtype=torch.bool, device=self.device)
        self.output_counts = torch.zeros(max_requests, vocab_size, dtype=torch.int32, device=self.device)
        self.synced: Dict[str, int] = {}       # generated tokens of the request already counted

    # ------------------------------------------------------------- membership
    def has(self, request_id: str) -> bool:
        return request_id in self.slots.slot_of

    def add_request(self, request_id: str, prompt_token_ids: Sequence[int]) -> int:
        s = self.slots.acquire(request_id)
        self.output_counts[s].zero_()
        self.prompt_mask[s].zero_()
        ids = torch.tensor([t for t in prompt_token_ids if 0 <= t < self.vocab_size], dtype=torch.long)
        if ids.numel():
            self.prompt_mask[s, ids.to(self.device)] = True
        self.synced[request_id] = 0
        return s

    def remove_request(self, request_id: str) -> None:
        self.slots.release(request_id)
        self.synced.pop(request_id, None)

    def slot_index(self, request_ids: Sequence[str]) -> torch.Tensor:
        return torch.tensor([self.slots.slot_of[r] for r in request_ids], dtype=torch.long, device=self.device)

    # ---------------------------------------------------------------- updates
    def record(self, slots: torch.Tensor, token_ids: torch.Tensor) -> None:
        """Count one generated token per row (device tensors, no host read).  Negative ids
        (placeholders of rejected positions) are ignored."""
        ok = (token_ids >= 0) & (token_ids < self.vocab_size)
        tok = token_ids.clamp(0, self.vocab_size - 1).long()
        self.output_counts.index_put_((slots.long(), tok), ok.to(torch.int32), accumulate=True)

    def revert(self, slots: torch.Tensor, token_ids: torch.Tensor, accepted: torch.Tensor) -> None:
        """Take back tokens that were counted when they were drafted and then rejected:
        ``token_ids`` / ``accepted`` [rows, n] (omni_npu/v0/layers/npu_sampler_cache.py:101-107)."""
        rows = slots.long().unsqueeze(1).expand_as(token_ids)
        ok = (~accepted) & (token_ids >= 0) & (token_ids < self.vocab_size)
        tok = token_ids.clamp(0, self.vocab_size - 1).long()
        self.output_counts.index_put_((rows.reshape(-1), tok.reshape(-1)), -ok.reshape(-1).to(torch.int32),
                                      accumulate=True)

    def sync_from_history(self, request_id: str, output_token_ids: Sequence[int]) -> None:
        """Bring the counts of one request up to date from its token list: only the tokens added
        since the last call travel to the device (one per decode step)."""
        done = self.synced.get(request_id, 0)
        new = [t for t in output_token_ids[done:] if 0 <= t < self.vocab_size]
        if len(output_token_ids) < done:        # the request was rolled back (preempted and recomputed)
            s = self.slots.slot_of[request_id]
            self.output_counts[s].zero_()
            new = [t for t in output_token_ids if 0 <= t < self.vocab_size]
        if new:
            s = self.slots.slot_of[request_id]
            tok = torch.tensor(new, dtype=torch.long, device=self.device)
            self.output_counts[s].index_put_((tok,), torch.ones(len(new), dtype=torch.int32, device=self.device),
                                             accumulate=True)
        self.synced[request_id] = len(output_token_ids)

    # ------------------------------------------------------------------ apply
    def apply(self, logits: torch.Tensor, slots: torch.Tensor, presence: torch.Tensor, frequency: torch.Tensor,
              repetition: torch.Tensor) -> torch.Tensor:
        """Penalised copy of ``logits`` [rows, V]; row i uses the state of ``slots[i]``."""
        counts = self.output_counts.index_select(0, slots.long()).to(logits.dtype)
        pmask = self.prompt_mask.index_select(0, slots.long())
        return apply_penalties(logits, pmask, counts, presence, frequency, repetition)


class ProbCache:
    """Draft distributions of the positions being verified, kept sparse: the draft model's
    ``topk`` most likely tokens and their probabilities per position, plus which of them it chose.
    ``computed[slot]`` is false until the drafter has run for the request (its first drafts are
    then rejected rather than accepted against an empty distribution)."""

    def __init__(self, max_requests: int, num_draft_tokens: int, topk: int, device) -> None:
        self.device = torch.device(device)
        self.topk, self.num_draft_tokens = topk, num_draft_tokens
        self.slots = _Slots(max_requests)
        self.topk_ids = torch.zeros(max_requests, num_draft_tokens, topk, dtype=torch.long, device=self.device)
        self.topk_probs = torch.zeros(max_requests, num_draft_tokens, topk, dtype=torch.float32, device=self.device)
        self.selected = torch.zeros(max_requests, num_draft_tokens, dtype=torch.long, device=self.device)
        self.computed = torch.zeros(max_requests, dtype=torch.bool, device=self.device)

    def add_request(self, request_id: str) -> int:
        s = self.slots.acquire(request_id)
        self.topk_probs[s].zero_()
        self.computed[s] = False
        return s

    def remove_request(self, request_id: str) -> None:
        self.slots.release(request_id)

    def slot_index(self, request_ids: Sequence[str]) -> torch.Tensor:
        return torch.tensor([self.slots.slot_of[r] for r in request_ids], dtype=torch.long, device=self.device)

    def update(self, slots: torch.Tensor, position: int, draft_probs: torch.Tensor,
               generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """Store draft position ``position`` of the rows ``slots`` from the drafter's full
        distribution [rows, V] and return the drafted token ids: the top-k entries are kept,
        renormalised, and the draft token is sampled among them."""
        probs, ids = torch.topk(draft_probs.float(), self.topk, dim=-1)
        probs = probs / probs.sum(dim=-1, keepdim=True).clamp_min(1e-20)
        pick = torch.multinomial(probs, 1, generator=generator).squeeze(1)
        s = slots.long()
        self.topk_ids[s, position] = ids
        self.topk_probs[s, position] = probs
        self.selected[s, position] = pick
        self.computed[s] = True
        return ids.gather(1, pick.unsqueeze(1)).squeeze(1)
