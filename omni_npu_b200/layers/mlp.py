"""Gated MLP: gate_up projection -> SiLU-and-mul -> down projection.

On CUDA the activation is folded into the gate_up GEMM epilogue (the weight
stores gate and up rows interleaved in groups of eight), so the [T, 2I]
intermediate is never written.  The reference runs the same three stages as
separate stream-labelled ops (omni_npu/v1/layers/fused_mlp/layer.py:16-165).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .activation import SiluAndMul
from .linear import MergedColumnParallelLinear, RowParallelLinear, row_parallel_add_rms_norm


class FusedMLP(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int, dtype=torch.bfloat16, device=None,
                 quant_method_factory=None, prefix: str = "", group=None,
                 reduce_results: bool = True, fuse_swiglu: bool = True) -> None:
        super().__init__()
        qm = quant_method_factory or (lambda: None)
        self.fuse_swiglu = fuse_swiglu
        self.gate_up_proj = MergedColumnParallelLinear(
            hidden_size, [intermediate_size, intermediate_size], dtype=dtype, device=device,
            swiglu_interleave=fuse_swiglu, quant_method=qm(), prefix=f"{prefix}.gate_up_proj",
            group=group)
        self.down_proj = RowParallelLinear(intermediate_size, hidden_size, dtype=dtype, device=device,
                                           quant_method=qm(), prefix=f"{prefix}.down_proj",
                                           group=group, reduce_results=reduce_results)
        self.act = SiluAndMul()

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
                reduce: bool = True) -> torch.Tensor:
        if self.fuse_swiglu:
            h = self.gate_up_proj(x, fuse_swiglu=True)
        else:
            h = self.act(self.gate_up_proj(x))
        return self.down_proj(h, residual=residual, reduce=reduce)

    def forward_add_rms_norm(self, x: torch.Tensor, norm, residual: torch.Tensor):
        """MLP whose down projection, tensor-parallel reduction, residual add and the FOLLOWING
        RMSNorm run as one kernel when the group has peer-mapped memory.  Returns
        (norm(residual + mlp(x)), residual)."""
        if self.fuse_swiglu:
            h = self.gate_up_proj(x, fuse_swiglu=True)
        else:
            h = self.act(self.gate_up_proj(x))
        return row_parallel_add_rms_norm(self.down_proj, h, norm, residual)
