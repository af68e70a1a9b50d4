"""Verification of speculative (draft) tokens.

The target model scores, in one forward pass, the position of every draft token of
every request plus the position after the last draft.  ``RejectionSampler`` then

1. samples a token from the target distribution at each of those positions with the
   regular sampler (temperature / top-k / top-p, greedy rows stay greedy), and
2. keeps draft tokens while they equal the target's samples, emits the target's own
   sample at the first disagreement, and the bonus token if nothing disagreed.

Every emitted token is a sample of the target distribution given its prefix, so the
output distribution is exactly the target model's whatever the drafts were; drafts only
decide how many positions one pass settles.  A ``strict`` mode implements the classic
accept-with-probability min(1, p/q) rule for proposers that return draft probabilities.

Same role and decision rule as ``NPURejectionSampler`` / ``simple_verify``
(omni_npu/sample/rejection_sampler.py:25-130,253-291).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import ops

MAX_SPEC_LEN = 32
PLACEHOLDER_TOKEN_ID = -1


@dataclass
class SpecDecodeMetadata:
    """Layout of one verification pass.  Logits rows are ordered request by request:
    ``n_b`` draft positions followed by one bonus position."""
    draft_token_ids: torch.Tensor          # [T] int32, all requests' drafts back to back
    num_draft_tokens: List[int]            # per request
    cu_num_draft_tokens: torch.Tensor      # [B+1] int32 exclusive prefix sums
    target_logits_indices: torch.Tensor    # [T] rows of the logits at draft positions
    bonus_logits_indices: torch.Tensor     # [B] row of the logits after the last draft
    max_spec_len: int

    @classmethod
    def make(cls, drafts: Sequence[Sequence[int]], device) -> "SpecDecodeMetadata":
        n = [len(d) for d in drafts]
        cu = [0]
        for x in n:
            cu.append(cu[-1] + x)
        flat = [t for d in drafts for t in d]
        tgt, bonus, row = [], [], 0
        for x in n:
            tgt.extend(range(row, row + x))
            bonus.append(row + x)
            row += x + 1
        i32 = dict(dtype=torch.int32, device=device)
        return cls(torch.tensor(flat, **i32), n, torch.tensor(cu, **i32),
                   torch.tensor(tgt, dtype=torch.long, device=device),
                   torch.tensor(bonus, dtype=torch.long, device=device), max(n) if n else 0)


def expand_batch_to_tokens(x: torch.Tensor, num_per_request: torch.Tensor, num_tokens: int) -> torch.Tensor:
    """[B] -> [T]: request b's value repeated for each of its positions."""
    return torch.repeat_interleave(x, num_per_request.to(torch.long), output_size=num_tokens)


class RejectionSampler(torch.nn.Module):
    def __init__(self, sampler) -> None:
        super().__init__()
        self.sampler = sampler

    def forward(self, metadata: SpecDecodeMetadata, draft_probs: Optional[torch.Tensor], logits: torch.Tensor,
                temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                seeds: Optional[torch.Tensor] = None, step_offset: Optional[torch.Tensor] = None,
                strict: bool = False):
        """logits [T + B, V]; per-request sampling tensors [B].  Returns
        (tokens [B, max_spec_len + 1] int32 with -1 padding, count [B] int32)."""
        assert metadata.max_spec_len <= MAX_SPEC_LEN
        b = len(metadata.num_draft_tokens)
        t = int(metadata.draft_token_ids.numel())
        # per-row sampling parameters: every position of a request uses the request's own
        per_req = torch.tensor([n + 1 for n in metadata.num_draft_tokens], device=logits.device)
        rows = t + b

        def rowwise(x):
            return None if x is None else expand_batch_to_tokens(x, per_req, rows)

        if strict and draft_probs is not None:
            return self._strict(metadata, draft_probs, logits, rowwise(temperature), rowwise(top_k), rowwise(top_p))
        # the sampling kernel derives a row's random stream from (seed, step offset, row index),
        # so the positions of one request already draw from distinct streams
        sampled = self.sampler(logits, rowwise(temperature), rowwise(top_k), rowwise(top_p), rowwise(seeds),
                               step_offset)
        sampled = sampled.to(torch.int32)
        target = sampled[metadata.target_logits_indices]
        bonus = sampled[metadata.bonus_logits_indices]
        return ops.spec_verify(metadata.draft_token_ids, target, bonus, metadata.cu_num_draft_tokens,
                               metadata.max_spec_len)

    # ------------------------------------------------------------------ strict
    def _strict(self, md: SpecDecodeMetadata, draft_probs, logits, temperature, top_k, top_p):
        """Accept draft x with probability min(1, p(x)/q(x)); on rejection sample from
        normalise(max(p - q, 0)).  Tensor ops; used for testing and for proposers that
        return probabilities."""
        from ..ops.ref import apply_top_k_top_p
        lg = logits.float()
        greedy = temperature < 1e-5
        lg = lg / torch.where(greedy, torch.ones_like(temperature), temperature).unsqueeze(1)
        lg = apply_top_k_top_p(lg, top_k, top_p)
        probs = torch.softmax(lg, dim=-1)
        onehot = torch.zeros_like(probs).scatter_(1, lg.argmax(-1, keepdim=True), 1.0)
        probs = torch.where(greedy.unsqueeze(1), onehot, probs)
        b = len(md.num_draft_tokens)
        out = torch.full((b, md.max_spec_len + 1), PLACEHOLDER_TOKEN_ID, dtype=torch.int32, device=logits.device)
        num = torch.zeros(b, dtype=torch.int32, device=logits.device)
        cu = md.cu_num_draft_tokens.tolist()
        drafts = md.draft_token_ids.tolist()
        gen = getattr(self.sampler, "generator", None)
        for r in range(b):
            emitted, all_ok = 0, True
            for i in range(cu[r], cu[r + 1]):
                row = int(md.target_logits_indices[i])
                x = drafts[i]
                p, q = probs[row, x], draft_probs[i, x].clamp_min(1e-20)
                u = torch.rand((), generator=gen, device="cpu" if gen is not None else logits.device).to(p.device)
                if u <= torch.clamp(p / q, max=1.0):
                    out[r, emitted] = x
                    emitted += 1
                    continue
                resid = (probs[row] - draft_probs[i].to(probs.dtype)).clamp_min(0)
                resid = resid / resid.sum().clamp_min(1e-20) if resid.sum() > 0 else probs[row]
                out[r, emitted] = int(torch.multinomial(resid.cpu(), 1, generator=gen))
                emitted += 1
                all_ok = False
                break
            if all_ok:
                row = int(md.bonus_logits_indices[r])
                out[r, emitted] = int(torch.multinomial(probs[row].cpu(), 1, generator=gen))
                emitted += 1
            num[r] = emitted
        return out, num


def parse_output(tokens: torch.Tensor, counts: torch.Tensor) -> List[List[int]]:
    """[B, S+1] padded tokens + counts -> ragged python lists."""
    tl, cl = tokens.tolist(), counts.tolist()
    return [row[:n] for row, n in zip(tl, cl)]


class SparseRejectionSampler:
    """Accept / reject rule for a drafter that samples from the top-k of its own distribution.

    The draft distribution of every position is kept sparse in a ``ProbCache`` (k token ids and
    their renormalised probabilities, the distribution the draft token was actually drawn from).
    Draft token x at a position is accepted with probability min(1, p(x) / q(x)); at the first
    rejection a token is drawn from the recovered distribution max(p - q, 0) (q scattered from its
    k entries), and when every draft is accepted the bonus token is drawn from the target
    distribution of the last position.  The emitted tokens are then distributed exactly as the
    target model's.  Rows whose draft distribution was never computed reject their drafts.
    Everything stays on the device.  Same decision rule as ``SparseRejectionSampler`` of
    omni_npu/v0/layers/sampler.py:952-1092."""

    def __init__(self, prob_cache, penalty_cache=None) -> None:
        self.prob_cache = prob_cache
        self.penalty_cache = penalty_cache

    def forward(self, target_probs: torch.Tensor, slots: torch.Tensor,
                generator: Optional[torch.Generator] = None):
        """``target_probs`` [B, n + 1, V]: the target distributions at the n draft positions and
        the bonus position; ``slots`` [B]: rows of the prob cache.  Returns ``(tokens [B, n + 1]
        with -1 after the last emitted token, num_emitted [B])``."""
        pc = self.prob_cache
        b, n1, v = target_probs.shape
        n = n1 - 1
        s = slots.long()
        ids = pc.topk_ids[s, :n]                                   # [B, n, k]
        q_all = pc.topk_probs[s, :n]
        sel = pc.selected[s, :n].unsqueeze(-1)
        draft = ids.gather(2, sel).squeeze(-1)                     # [B, n]
        q = q_all.gather(2, sel).squeeze(-1)
        p = target_probs[:, :n].gather(2, draft.unsqueeze(-1)).squeeze(-1)
        u = torch.rand(p.shape, device=p.device, generator=generator)
        ok = (u * q < p) & pc.computed[s].unsqueeze(1)             # u < p / q without dividing by zero
        accepted = torch.cumprod(ok.to(torch.int32), dim=1).bool() # a rejection ends the run
        num_acc = accepted.sum(dim=1)                              # [B] in 0..n
        rows = torch.arange(b, device=p.device)
        # distribution of the token emitted after the accepted run
        p_next = target_probs[rows, num_acc]                       # [B, V]
        rejected_here = num_acc < n
        j = num_acc.clamp(max=max(n - 1, 0))
        if n > 0:
            q_dense = torch.zeros(b, v, dtype=p_next.dtype, device=p.device)
            q_dense.scatter_(1, ids[rows, j], q_all[rows, j].to(p_next.dtype))
            q_dense = q_dense * pc.computed[s].unsqueeze(1)        # no draft distribution: sample the target's
            recovered = (p_next - q_dense).clamp_min(0)
            total = recovered.sum(dim=1, keepdim=True)
            recovered = torch.where(total > 0, recovered / total.clamp_min(1e-20), p_next)
            p_next = torch.where(rejected_here.unsqueeze(1), recovered, p_next)
        nxt = torch.multinomial(p_next.float(), 1, generator=generator).squeeze(1)
        out = torch.full((b, n1), PLACEHOLDER_TOKEN_ID, dtype=torch.long, device=p.device)
        if n > 0:
            out[:, :n] = torch.where(accepted, draft, torch.full_like(draft, PLACEHOLDER_TOKEN_ID))
        out[rows, num_acc] = nxt
        if self.penalty_cache is not None:
            for i in range(n1):
                self.penalty_cache.record(s, out[:, i])
        return out, num_acc + 1

    __call__ = forward
