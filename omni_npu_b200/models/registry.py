"""Architecture name -> model class.

Mirrors the set of architectures the reference registers with vLLM's
ModelRegistry (omni_npu/v1/models/__init__.py:4-43, omni_npu/v0/models/__init__.py:6-10).
Classes are imported lazily so importing the package stays cheap.
"""
from __future__ import annotations

import importlib
from typing import Dict, Tuple, Type

_REGISTRY: Dict[str, Tuple[str, str]] = {
    "LlamaForCausalLM": ("omni_npu_b200.models.llama", "LlamaForCausalLM"),
    "MistralForCausalLM": ("omni_npu_b200.models.llama", "LlamaForCausalLM"),
    "Qwen2ForCausalLM": ("omni_npu_b200.models.llama", "LlamaForCausalLM"),
    "Qwen3ForCausalLM": ("omni_npu_b200.models.llama", "LlamaForCausalLM"),
    "Qwen3MoeForCausalLM": ("omni_npu_b200.models.qwen3_moe", "Qwen3MoeForCausalLM"),
    "DeepseekV2ForCausalLM": ("omni_npu_b200.models.deepseek", "DeepseekForCausalLM"),
    "DeepseekV3ForCausalLM": ("omni_npu_b200.models.deepseek", "DeepseekForCausalLM"),
    "DeepseekV32ForCausalLM": ("omni_npu_b200.models.deepseek", "DeepseekForCausalLM"),
    "DeepSeekMTPModel": ("omni_npu_b200.models.mtp", "DeepSeekMTP"),
    "PanguUltraMoEForCausalLM": ("omni_npu_b200.models.pangu", "PanguUltraMoEForCausalLM"),
    "OpenPanguMTPModel": ("omni_npu_b200.models.mtp", "OpenPanguMTP"),
    "PanguProMoEV2ForCausalLM": ("omni_npu_b200.models.pangu", "PanguProMoEV2ForCausalLM"),
    "Qwen3VLForConditionalGeneration": ("omni_npu_b200.models.qwen3_vl", "Qwen3VLForConditionalGeneration"),
    "OpenPanguVLForConditionalGeneration": ("omni_npu_b200.models.openpangu_vl", "OpenPanguVLForConditionalGeneration"),
    "MockModel": ("omni_npu_b200.models.mock", "MockModelForCausalLM"),
}


def register_model(arch: str, module: str, cls_name: str) -> None:
    _REGISTRY[arch] = (module, cls_name)


def supported_architectures():
    return sorted(_REGISTRY)


def resolve_model_cls(arch: str) -> Type:
    if arch not in _REGISTRY:
        raise ValueError(f"architecture {arch!r} is not supported; known: {supported_architectures()}")
    module, name = _REGISTRY[arch]
    return getattr(importlib.import_module(module), name)


def register_models() -> None:
    """Entry point for ``vllm.general_plugins``: make the architectures above
    known to vLLM's ModelRegistry when vLLM is importable."""
    try:
        from vllm import ModelRegistry
    except Exception:
        return
    from .vllm_adapters import ADAPTERS
    known = set(ModelRegistry.get_supported_archs()) if hasattr(ModelRegistry, "get_supported_archs") else set()
    for arch, path in ADAPTERS.items():
        if arch in known:
            continue            # vLLM's own class already runs on this platform with our kernels underneath
        try:
            ModelRegistry.register_model(arch, path)
        except Exception:
            pass
