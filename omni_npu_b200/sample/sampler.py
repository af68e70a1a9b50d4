"""Sampler: logits -> token ids.

Greedy rows and random rows go through one fused kernel (temperature, top-k,
top-p, exponential race) on CUDA; penalties, when any request asks for them,
are applied to the logits beforehand with tensor ops.  The reference does the
same split: fused ``npu_top_k_top_p_sample`` plus torch fall-backs for
penalties (omni_npu/sample/sampler.py:24-165,
omni_npu/sample/ops/topk_topp_sampler.py:41-88).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops


def apply_penalties(logits: torch.Tensor, prompt_mask: Optional[torch.Tensor],
                    output_counts: torch.Tensor, presence: torch.Tensor, frequency: torch.Tensor,
                    repetition: torch.Tensor) -> torch.Tensor:
    """logits [B,V]; output_counts [B,V] occurrences among generated tokens;
    prompt_mask [B,V] bool of tokens present in the prompt."""
    seen = output_counts > 0
    if prompt_mask is not None:
        seen = seen | prompt_mask
    rep = repetition.unsqueeze(1)
    rep_factor = torch.where(seen, rep, torch.ones_like(rep))
    logits = torch.where(logits > 0, logits / rep_factor, logits * rep_factor)
    logits = logits - frequency.unsqueeze(1) * output_counts
    logits = logits - presence.unsqueeze(1) * (output_counts > 0).to(logits.dtype)
    return logits


class Sampler(torch.nn.Module):
    def __init__(self, config=None, device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.device = device
        self.generator: Optional[torch.Generator] = None
        if device is not None and device.type == "cpu":
            self.generator = torch.Generator(device="cpu")
            self.generator.manual_seed(getattr(config, "seed", 0) if config is not None else 0)

    def forward(self, logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
                top_p: torch.Tensor, seeds: Optional[torch.Tensor] = None,
                step_offset: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.sample(logits, temperature, top_k, top_p, seeds, step_offset,
                          generator=self.generator)
