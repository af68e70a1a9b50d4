"""fp8 (e4m3) block-scaled linear algebra helpers.

Weights carry one fp32 scale per 128x128 block (HF ``weight_scale_inv``);
activations are quantised on the fly per token per 128 columns.  The product
is accumulated per 128-wide K block and promoted with both scales, which is
what the DeepSeek-V3 family checkpoints assume.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import ops
from ..ops import ref


def quantize_weight_block(w: torch.Tensor, block: Tuple[int, int] = (128, 128)):
    """[N,K] float -> (e4m3 [N,K], fp32 scales [ceil(N/bn), ceil(K/bk)])."""
    n, k = w.shape[-2:]
    bn, bk = block
    pn, pk = (n + bn - 1) // bn * bn, (k + bk - 1) // bk * bk
    wp = torch.zeros(*w.shape[:-2], pn, pk, dtype=torch.float32, device=w.device)
    wp[..., :n, :k] = w.float()
    blocks = wp.view(*w.shape[:-2], pn // bn, bn, pk // bk, bk)
    amax = blocks.abs().amax(dim=(-3, -1)).clamp_min(1e-10)
    scale = amax / 448.0
    q = (blocks / scale[..., :, None, :, None]).clamp(-448, 448)
    q = q.view(*w.shape[:-2], pn, pk)[..., :n, :k].to(torch.float8_e4m3fn)
    return q.contiguous(), scale.contiguous()


def fp8_block_gemm(x: torch.Tensor, wq: torch.Tensor, w_scale: torch.Tensor,
                   bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                   block: Tuple[int, int] = (128, 128), swiglu: bool = False,
                   out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """x [M,K] bf16 times block-scaled e4m3 weights [N,K]."""
    if x.is_cuda and x.dim() == 2 and x.shape[1] % 128 == 0 and tuple(block) == (128, 128) and not swiglu \
            and x.dtype == torch.bfloat16 and wq.dim() == 2:
        # native path: per-token-per-128 activation quantisation, then the block-scaled tcgen05 kernel
        xq, xs = ops.quant_fp8_1x128(x.contiguous())
        return ops.gemm_fp8_block(xq, xs, wq, w_scale, bias, residual, out_dtype)
    w = ref.dequant_fp8_block(wq, w_scale, block).to(x.dtype if x.dtype.itemsize > 1 else torch.bfloat16)
    return ops.gemm(x, w, bias, residual, out_dtype, swiglu)
