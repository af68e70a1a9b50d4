"""Which architectures this package offers to vLLM's ``ModelRegistry`` and how.

On a CUDA platform vLLM already ships model classes for most architectures listed in
``models/registry.py``; they pick up this package's kernels through the out-of-tree custom
ops, the attention backend, the communicator and the quantisation method, so they need no
replacement.  Registered here are the architectures vLLM does not know (the openPangu
family and the mock model) through ``StandaloneModelAdapter``, a thin vLLM-style class
(``__init__(*, vllm_config, prefix)``, ``forward(input_ids, positions, ...)``,
``compute_logits``, ``load_weights``) around the standalone implementation.  The adapter
translates vLLM's forward context (per-layer attention metadata from
``attention/vllm_backends.py`` and the KV caches bound to its attention-layer stand-ins)
into this package's forward context.

Counterpart of the ``register_models`` entry points
(omni_npu/v1/models/__init__.py:4-43, omni_npu/v0/models/__init__.py:6-10).
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, Optional, Tuple

import torch
from torch import nn

from .. import compat
from ..attention.metadata import AttentionMetadata, set_forward_context
from ..config import CacheConfig, EngineConfig, ModelConfig, ParallelConfig, SchedulerConfig

# architecture -> "module:class" handed to ModelRegistry.register_model (lazy import by vLLM)
ADAPTERS: Dict[str, str] = {
    "PanguUltraMoEForCausalLM": "omni_npu_b200.models.vllm_adapters:PanguUltraMoEForCausalLM",
    "PanguProMoEV2ForCausalLM": "omni_npu_b200.models.vllm_adapters:PanguProMoEV2ForCausalLM",
    "OpenPanguMTPModel": "omni_npu_b200.models.vllm_adapters:OpenPanguMTPModel",
    "MockModel": "omni_npu_b200.models.vllm_adapters:MockModel",
}


def engine_config_from_vllm(vllm_config) -> EngineConfig:
    mc = vllm_config.model_config
    hf = mc.hf_config.to_dict() if hasattr(mc.hf_config, "to_dict") else dict(vars(mc.hf_config))
    model = ModelConfig.from_hf_dict(hf, dtype=getattr(mc, "dtype", None))
    cache = getattr(vllm_config, "cache_config", None)
    par = getattr(vllm_config, "parallel_config", None)
    sch = getattr(vllm_config, "scheduler_config", None)
    return EngineConfig(
        model=model,
        cache=CacheConfig(block_size=int(getattr(cache, "block_size", 16) or 16)),
        parallel=ParallelConfig(tensor_parallel_size=int(getattr(par, "tensor_parallel_size", 1) or 1),
                                enable_expert_parallel=bool(getattr(par, "enable_expert_parallel", False))),
        scheduler=SchedulerConfig(max_num_seqs=int(getattr(sch, "max_num_seqs", 128) or 128),
                                  max_num_batched_tokens=int(getattr(sch, "max_num_batched_tokens", 8192) or 8192),
                                  max_model_len=int(getattr(mc, "max_model_len", 8192) or 8192)),
        additional_config=dict(getattr(vllm_config, "additional_config", None) or {}))


def metadata_from_vllm(md, positions: torch.Tensor) -> AttentionMetadata:
    """``B200AttentionMetadata`` (attention/vllm_backends.py) -> this package's metadata."""
    n_tok, n_req = md.num_actual_tokens, md.num_reqs
    return AttentionMetadata(
        is_prefill=not md.is_decode, num_seqs=n_req, num_tokens=n_tok, max_q_len=md.max_query_len,
        max_seq_len=md.max_seq_len, q_len=1 if md.is_decode else 0, positions=positions[:n_tok].to(torch.int32),
        slot_mapping=md.slot_mapping[:n_tok].to(torch.int32), block_tables=md.block_table, seq_lens=md.seq_lens,
        cu_q=md.query_start_loc, num_actual_tokens=n_tok, num_actual_seqs=n_req)


class StandaloneModelAdapter(nn.Module):
    """vLLM-facing shell around a standalone model class of this package."""
    architecture: str = ""

    def __init__(self, *, vllm_config, prefix: str = "") -> None:
        super().__init__()
        from .registry import resolve_model_cls
        self.vllm_config = vllm_config
        self.engine_config = engine_config_from_vllm(vllm_config)
        self.engine_config.model.architecture = self.architecture or self.engine_config.model.architecture
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.inner = resolve_model_cls(self.engine_config.model.architecture)(self.engine_config, device=device)
        self.kv_caches: list = []          # bound by bind_kv_caches() once vLLM has allocated them

    def bind_kv_caches(self, kv_caches: list) -> None:
        self.kv_caches = list(kv_caches)

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor, intermediate_tensors: Any = None,
                inputs_embeds: Optional[torch.Tensor] = None, **kw: Any) -> torch.Tensor:
        md = None
        if compat.vllm_available():
            try:
                from vllm.forward_context import get_forward_context as vllm_ctx
                am = vllm_ctx().attn_metadata
                md = next(iter(am.values())) if isinstance(am, dict) and am else am
            except Exception:
                md = None
        if md is None:                                     # profiling run without attention metadata
            return torch.zeros(input_ids.shape[0], self.engine_config.model.hidden_size,
                               dtype=self.engine_config.model.dtype, device=input_ids.device)
        with set_forward_context(metadata_from_vllm(md, positions), self.kv_caches, self.engine_config):
            return self.inner(input_ids, positions, inputs_embeds)

    def compute_logits(self, hidden_states: torch.Tensor, *a: Any, **k: Any) -> torch.Tensor:
        return self.inner.compute_logits(hidden_states)

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        loaded = self.inner.load_weights(weights)
        for m in self.inner.modules():
            hook = getattr(m, "process_weights_after_loading", None)
            if callable(hook):
                hook()
        return {"inner." + n for n in loaded}


class PanguUltraMoEForCausalLM(StandaloneModelAdapter):
    architecture = "PanguUltraMoEForCausalLM"


class PanguProMoEV2ForCausalLM(StandaloneModelAdapter):
    architecture = "PanguProMoEV2ForCausalLM"


class OpenPanguMTPModel(StandaloneModelAdapter):
    architecture = "OpenPanguMTPModel"


class MockModel(StandaloneModelAdapter):
    architecture = "MockModel"
