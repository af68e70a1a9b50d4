"""Out-of-tree overrides of vLLM custom ops (``CustomOp.register_oot``).

Importing this module (the platform does it once, when vLLM is importable) makes vLLM
construct these classes wherever a model asks for the named op, so stock vLLM models get
this package's kernels without any change to their code: SiLU-and-mul, RMSNorm (plain and
fused with the residual add) and the rotary-embedding family.  The reference registers the
same set for its NPU kernels (omni_npu/layers/activation.py:11-33,
omni_npu/layers/npu_rms_norm.py:12-33, omni_npu/layers/rotary_embedding/*.py).
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from .. import compat, ops

REGISTERED = []

if compat.vllm_available():
    from vllm.model_executor.custom_op import CustomOp
    from vllm.model_executor.layers.activation import SiluAndMul
    from vllm.model_executor.layers.layernorm import RMSNorm

    def _fast(x: torch.Tensor) -> bool:
        return x.is_cuda and x.dtype == torch.bfloat16

    @SiluAndMul.register_oot
    class B200SiluAndMul(SiluAndMul):
        def forward_oot(self, x: torch.Tensor) -> torch.Tensor:
            if not _fast(x):
                return self.forward_native(x)
            shape = x.shape
            return ops.silu_and_mul(x.reshape(-1, shape[-1])).view(*shape[:-1], shape[-1] // 2)

    @RMSNorm.register_oot
    class B200RMSNorm(RMSNorm):
        def forward_oot(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None
                        ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
            if not _fast(x) or getattr(self, "variance_size_override", None) is not None \
                    or not getattr(self, "has_weight", True):
                return self.forward_native(x, residual)
            shape = x.shape
            x2 = x.reshape(-1, shape[-1])
            if residual is None:
                return ops.rms_norm(x2, self.weight.data, self.variance_epsilon).view(shape)
            r2 = residual.reshape(-1, shape[-1])
            y = ops.fused_add_rms_norm(x2, r2, self.weight.data, self.variance_epsilon)   # r2 updated in place
            return y.view(shape), r2.view(shape)

    REGISTERED += ["SiluAndMul", "RMSNorm"]

    try:
        from vllm.model_executor.layers.rotary_embedding import RotaryEmbedding

        @RotaryEmbedding.register_oot
        class B200RotaryEmbedding(RotaryEmbedding):
            """Rotates q and k in place with the fused kernel (neox or interleaved, partial
            rotary supported); falls back to the native path for anything else."""

            def forward_oot(self, positions: torch.Tensor, query: torch.Tensor, key: Optional[torch.Tensor] = None,
                            *args, **kw):
                if key is None or not _fast(query) or positions.dim() != 1 or args or kw:
                    return self.forward_native(positions, query, key, *args, **kw)
                cs = getattr(self, "_b200_cos_sin", None)
                if cs is None or cs.device != query.device:
                    cs = self.cos_sin_cache.to(device=query.device, dtype=torch.float32).contiguous()
                    self._b200_cos_sin = cs
                t = positions.shape[0]
                q2, k2 = query.reshape(t, -1), key.reshape(t, -1)
                ops.rope_qk_(q2, k2, positions.to(torch.int32), cs, self.head_size, self.rotary_dim,
                             bool(self.is_neox_style))
                return q2.view(query.shape), k2.view(key.shape)

        REGISTERED.append("RotaryEmbedding")
    except Exception:                                     # layout of the rotary module differs in this vLLM
        pass
