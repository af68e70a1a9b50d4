"""RMSNorm (optionally fused with the residual add) and LayerNorm.

Counterpart of ``NPURMSNorm`` (omni_npu/layers/npu_rms_norm.py:12-33): calling
with a residual performs ``residual += x`` and normalises the sum in one
kernel; ``y_transform="AG"`` all-gathers the normalised rows over the tensor
parallel group (sequence-parallel residual stream).
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch
from torch import nn

from .. import ops
from ..parallel import state as pstate


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, dtype: torch.dtype = torch.bfloat16,
                 device=None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=dtype, device=device),
                                   requires_grad=False)
        self.eps = eps

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
                y_transform: Optional[str] = None
                ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
        if residual is None:
            y = ops.rms_norm(x, self.weight, self.eps)
            if y_transform == "AG":
                y = pstate.get_tp_group().all_gather(y, dim=0)
            return y
        y = ops.fused_add_rms_norm(x, residual, self.weight, self.eps)
        if y_transform == "AG":
            y = pstate.get_tp_group().all_gather(y, dim=0)
        return y, residual

    def forward_quant(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None, kind: str = "int8",
                      want_bf16: bool = False):
        """Norm fused with the per-token activation quantisation of the W8A8 linear that follows:
        returns ``((q, scale), residual, bf16 row or None)``; the pair is accepted by the quantised
        linear methods in place of a bf16 activation (the reference fuses the same pair of ops,
        omni_npu/v1/layers/layernorm.py and npu_compressed_tensors_linear.py:149-231)."""
        q, s, y = ops.rms_norm_quant(x, self.weight, self.eps, residual, kind, want_bf16)
        return (q, s), residual, y


def reduce_add_rms_norm(norm: RMSNorm, x_partial: torch.Tensor, residual: torch.Tensor, group):
    """``residual += all_reduce(x_partial)``; returns (RMSNorm(residual), residual).

    This is the tail of every row-parallel projection (o_proj, down_proj).  With
    symmetric memory attached to the group it runs as one peer-memory kernel
    (GEMM -> all-reduce + residual + RMSNorm); otherwise as an all-reduce followed
    by the fused add+norm kernel."""
    if group.world_size == 1:
        return norm(x_partial, residual)
    symm = group.comm.symm
    if symm is not None and symm.can_all_reduce(x_partial):
        y = symm.all_reduce_add_rms_norm(x_partial, residual, norm.weight, norm.eps)
        return y, residual
    return norm(group.all_reduce(x_partial), residual)


class LayerNorm(nn.Module):
    """Plain LayerNorm in fp32 (used by the sparse-attention indexer key path)."""

    def __init__(self, dim: int, eps: float = 1e-6, dtype=torch.float32, device=None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device), requires_grad=False)
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device), requires_grad=False)
        self.eps = eps
        self.dim = dim

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.layer_norm(x.float(), (self.dim,), self.weight.float(),
                                              self.bias.float(), self.eps).to(x.dtype)
