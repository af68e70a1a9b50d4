"""SiLU-and-mul (SwiGLU gate); counterpart of NPUSiluAndMul
(omni_npu/layers/activation.py:11-33)."""
from __future__ import annotations

import torch
from torch import nn

from .. import ops


class SiluAndMul(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.silu_and_mul(x)
