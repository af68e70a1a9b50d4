"""int8 W8A8 quantisation in the compressed-tensors checkpoint format.

Scheme (the only one the format's int-quantised checkpoints of this model family use):
weights int8, symmetric, one static scale per output channel; activations int8,
symmetric, one dynamic scale per token.  A linear layer then is

    y = (quant(x) @ w_q^T) * s_x[:, None] * s_w[None, :]  (+ bias)

with the integer product accumulated exactly in 32 bits on the tensor cores
(``tcgen05.mma.kind::i8``, ``ops.gemm_scaled``) and both scales applied in the GEMM
epilogue.  ``CompressedTensorsConfig`` parses the ``quantization_config`` block of an HF
config (targets, ignore list, per-group schemes), picks the method per layer, and refuses
4-bit weight schemes.

Counterpart of ``NPUCompressedTensorsConfig`` and its W8A8 linear / MoE methods
(omni_npu/layers/quantization/compressed_tensors/compressed_tensors.py:32-221,
compressed_tensors_linear.py, compressed_tensors_moe.py; v1 variant with fused
dequant + SwiGLU + requant: omni_npu/v1/layers/quantization/compressed_tensors/
npu_compressed_tensors_linear.py:149-231).
"""
from __future__ import annotations

import fnmatch
import re
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional

import torch
from torch import nn

from .. import ops

QUANT_NAME = "b200-compressed-tensors"


# ------------------------------------------------------------------- helpers
def quantize_weight_per_channel(w: torch.Tensor):
    """[N,K] float -> (int8 [N,K], fp32 scale [N]) symmetric per output channel."""
    wf = w.float()
    scale = wf.abs().amax(dim=-1).clamp_min(1e-10) / 127.0
    q = torch.round(wf / scale.unsqueeze(-1)).clamp_(-127, 127).to(torch.int8)
    return q.contiguous(), scale.contiguous()


def int8_linear(x: torch.Tensor, w_q: torch.Tensor, w_scale: torch.Tensor, bias: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    if isinstance(x, tuple):
        # already quantised by the producing kernel (norm + quant, SwiGLU + quant): (q [T,K], scale [T])
        xq, xs = x
        return ops.gemm_scaled(xq, w_q, xs, w_scale, bias, residual, out_dtype or torch.bfloat16)
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    xq, xs = ops.quant_int8_per_token(x2)
    y = ops.gemm_scaled(xq, w_q, xs, w_scale, bias, residual, out_dtype or (x.dtype if x.dtype.itemsize > 1 else None))
    return y.reshape(*shape[:-1], w_q.shape[0])


# ------------------------------------------------------------------- methods
class W8A8Int8LinearMethod:
    """int8 weights (per-channel static scale) x int8 activations (per-token dynamic scale)."""

    def create_weights(self, layer, in_features: int, out_features: int, dtype, device) -> None:
        layer.weight = nn.Parameter(torch.zeros(out_features, in_features, dtype=torch.int8, device=device),
                                    requires_grad=False)
        layer.weight_scale = nn.Parameter(torch.ones(out_features, 1, dtype=torch.float32, device=device),
                                          requires_grad=False)

    def process_weights_after_loading(self, layer) -> None:
        layer.weight_scale.data = layer.weight_scale.data.float().reshape(-1, 1).contiguous()

    def apply(self, layer, x, bias, residual=None, swiglu=False, out_dtype=None):
        y = int8_linear(x, layer.weight, layer.weight_scale.view(-1), bias, residual,
                        torch.float32 if swiglu else out_dtype)
        if swiglu:
            # gate/up rows are interleaved in groups of 8 (the fused bf16 epilogue's layout):
            # undo it on the product and apply the activation
            n = y.shape[-1]
            y = y.view(*y.shape[:-1], n // 16, 2, 8)
            gate, up = y[..., 0, :].reshape(*y.shape[:-3], n // 2), y[..., 1, :].reshape(*y.shape[:-3], n // 2)
            y = (torch.nn.functional.silu(gate) * up).to(out_dtype or torch.bfloat16)
        return y


class W8A8Int8MoEMethod:
    """Expert weights int8 per channel; tokens quantised per row after permutation.  The
    grouped product runs expert by expert through ``gemm_scaled`` (the offsets are already on
    the host at this point of the eager MoE path)."""

    def quantize_experts(self, w: torch.Tensor):
        q, s = quantize_weight_per_channel(w.reshape(-1, w.shape[-1]))
        return q.view(w.shape), s.view(w.shape[0], w.shape[1])

    def apply_expert(self, x: torch.Tensor, w_q: torch.Tensor, w_scale: torch.Tensor) -> torch.Tensor:
        return int8_linear(x, w_q, w_scale)


# -------------------------------------------------------------------- config
@dataclass
class QuantArgs:
    num_bits: int = 8
    type: str = "int"
    symmetric: bool = True
    strategy: str = "channel"          # tensor | channel | token | group
    dynamic: bool = False

    @classmethod
    def from_dict(cls, d: Optional[Mapping[str, Any]]) -> Optional["QuantArgs"]:
        if not d:
            return None
        bits = d.get("num_bits", 8)
        if isinstance(bits, Mapping):
            bits = min(bits.values())
        return cls(int(bits), d.get("type", "int"), bool(d.get("symmetric", True)),
                   d.get("strategy", "tensor"), bool(d.get("dynamic", False)))


@dataclass
class CompressedTensorsConfig:
    target_scheme_map: Dict[str, Dict[str, Optional[QuantArgs]]] = field(default_factory=dict)
    ignore: List[str] = field(default_factory=list)
    quant_format: str = "int-quantized"
    kv_cache_scheme: Any = None

    @classmethod
    def get_name(cls) -> str:
        return QUANT_NAME

    @classmethod
    def override_quantization_method(cls, hf_quant_cfg: Mapping[str, Any], user_quant: Optional[str]) -> Optional[str]:
        """HF checkpoints say ``compressed-tensors``; this implementation takes them over."""
        if (hf_quant_cfg or {}).get("quant_method") == "compressed-tensors":
            return QUANT_NAME
        return None

    @classmethod
    def from_config(cls, cfg: Mapping[str, Any]) -> "CompressedTensorsConfig":
        tmap: Dict[str, Dict[str, Optional[QuantArgs]]] = {}
        for group in (cfg.get("config_groups") or {}).values():
            scheme = {"weights": QuantArgs.from_dict(group.get("weights")),
                      "input_activations": QuantArgs.from_dict(group.get("input_activations"))}
            for target in group.get("targets", ["Linear"]):
                tmap[target] = scheme
        return cls(tmap, list(cfg.get("ignore") or []), cfg.get("format", "int-quantized"),
                   cfg.get("kv_cache_scheme"))

    # ------------------------------------------------------------- matching
    def is_ignored(self, layer_name: str) -> bool:
        for pat in self.ignore:
            if pat.startswith("re:"):
                if re.match(pat[3:], layer_name):
                    return True
            elif pat == layer_name or layer_name.endswith("." + pat) or fnmatch.fnmatch(layer_name, pat):
                return True
        return False

    def scheme_for(self, layer_name: str, module_type: str = "Linear") -> Optional[Dict[str, Optional[QuantArgs]]]:
        if self.is_ignored(layer_name):
            return None
        for target, scheme in self.target_scheme_map.items():
            if target == module_type or target == layer_name or layer_name.endswith(target) or \
                    (target.startswith("re:") and re.match(target[3:], layer_name)):
                return scheme
        return None

    @staticmethod
    def is_dynamic_token_w8a8(w: Optional[QuantArgs], a: Optional[QuantArgs]) -> bool:
        if w is None or a is None:
            return False
        return (w.num_bits == 8 and a.num_bits == 8 and w.type == "int" and a.type == "int"
                and w.symmetric and w.strategy in ("channel", "tensor") and not w.dynamic
                and a.dynamic and a.strategy == "token" and a.symmetric)

    def get_quant_method(self, layer_name: str, module_type: str = "Linear"):
        """A linear / MoE method for the layer, or None to leave it unquantised."""
        scheme = self.scheme_for(layer_name, module_type)
        if scheme is None:
            return None
        w, a = scheme["weights"], scheme["input_activations"]
        if w is not None and w.num_bits == 4:
            raise NotImplementedError("4-bit weight schemes (w4a8 / w4a16) are not supported")
        if self.is_dynamic_token_w8a8(w, a):
            return W8A8Int8MoEMethod() if module_type == "FusedMoE" else W8A8Int8LinearMethod()
        raise NotImplementedError(f"unsupported compressed-tensors scheme for {layer_name}: {scheme}")
