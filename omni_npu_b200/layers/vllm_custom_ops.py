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

        def _oot_variant(mod: str, name: str) -> None:
            """The scaling variants (YaRN, DeepSeek-YaRN, linear, Llama-3) only change how the cos/sin
            table is built; the rotation itself is the same fused kernel."""
            try:
                base = getattr(__import__(mod, fromlist=[name]), name)
            except Exception:
                return
            if not issubclass(base, RotaryEmbedding):
                return
            cls = type("B200" + name, (base,), {"forward_oot": B200RotaryEmbedding.forward_oot,
                                                "__doc__": f"{name} rotating with the fused kernel."})
            base.register_oot(cls)
            REGISTERED.append(name)

        _rp = "vllm.model_executor.layers.rotary_embedding."
        for _mod, _name in ((_rp + "deepseek_scaling_rope", "DeepseekScalingRotaryEmbedding"),
                            (_rp + "linear_scaling_rope", "LinearScalingRotaryEmbedding"),
                            (_rp + "llama3_rope", "Llama3RotaryEmbedding"),
                            (_rp + "yarn_scaling_rope", "YaRNScalingRotaryEmbedding")):
            _oot_variant(_mod, _name)

        # multimodal rotary embedding: positions [3, T] (temporal, row, column), frequency bands taken
        # from the axis that owns them (reference: MRotaryEmbedding override,
        # omni_npu/v1/layers/rotary_embedding/mrope.py:17-206)
        try:
            from vllm.model_executor.layers.rotary_embedding.mrope import MRotaryEmbedding

            def _mrope_forward_oot(self, positions: torch.Tensor, query: torch.Tensor,
                                   key: Optional[torch.Tensor] = None, *args, **kw):
                sec = getattr(self, "mrope_section", None)
                if key is None or not _fast(query) or args or kw or (positions.dim() == 2 and (not sec or len(sec) != 3)):
                    return self.forward_native(positions, query, key, *args, **kw)
                cs = getattr(self, "_b200_cos_sin", None)
                if cs is None or cs.device != query.device:
                    cs = self.cos_sin_cache.to(device=query.device, dtype=torch.float32).contiguous()
                    self._b200_cos_sin = cs
                t = positions.shape[-1]
                q2, k2 = query.reshape(t, -1), key.reshape(t, -1)
                ops.rope_qk_(q2, k2, positions.to(torch.int32).contiguous(), cs, self.head_size, self.rotary_dim,
                             bool(self.is_neox_style), tuple(int(x) for x in sec) if positions.dim() == 2 else None,
                             bool(getattr(self, "mrope_interleaved", False)))
                return q2.view(query.shape), k2.view(key.shape)

            MRotaryEmbedding.register_oot(type("B200MRotaryEmbedding", (MRotaryEmbedding,),
                                               {"forward_oot": _mrope_forward_oot,
                                                "__doc__": "M-RoPE rotating with the fused kernel."}))
            REGISTERED.append("MRotaryEmbedding")
        except Exception:
            pass
    except Exception:                                     # layout of the rotary module differs in this vLLM
        pass

    # ---- quantisation config: the name this platform's loaders answer to
    try:
        from vllm.model_executor.layers.quantization import register_quantization_config
        from vllm.model_executor.layers.quantization.base_config import QuantizationConfig

        from .quant_int8 import QUANT_NAME, CompressedTensorsConfig

        @register_quantization_config(QUANT_NAME)
        class B200CompressedTensorsQuantConfig(QuantizationConfig):
            """vLLM-facing name of this package's compressed-tensors (W8A8 int8) support.  Checkpoints
            whose HF ``quant_method`` is ``compressed-tensors`` select it automatically on this
            platform (the reference does the same for its ``npu-compressed-tensors``:
            omni_npu/layers/quantization/compressed_tensors/compressed_tensors.py:32-36,176-182).
            The weights themselves are loaded by this package's own model classes
            (``layers/quant_int8.py``); this class parses and carries the config."""

            def __init__(self, inner: Optional[CompressedTensorsConfig] = None) -> None:
                super().__init__()
                self.inner = inner

            def get_name(self) -> str:
                return QUANT_NAME

            @classmethod
            def get_supported_act_dtypes(cls):
                return [torch.bfloat16, torch.float16]

            @classmethod
            def get_min_capability(cls) -> int:
                return 100

            @classmethod
            def get_config_filenames(cls):
                return []

            @classmethod
            def from_config(cls, config):
                return cls(CompressedTensorsConfig.from_config(config))

            @classmethod
            def override_quantization_method(cls, hf_quant_cfg, user_quant, *args, **kw):
                method = (hf_quant_cfg or {}).get("quant_method")
                if method == "compressed-tensors" and user_quant in (None, QUANT_NAME, "compressed-tensors"):
                    return QUANT_NAME
                return None

            def get_quant_method(self, layer, prefix: str):
                return None          # vLLM's own layers are not built under this platform's worker

        REGISTERED.append("quantization:" + QUANT_NAME)
    except Exception:
        pass
