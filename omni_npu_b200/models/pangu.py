"""openPangu model family.

``PanguUltraMoEForCausalLM``: multi-head latent attention + a shared/routed mixture of
experts with sigmoid routing (one expert group, optional per-expert bias correction) and
an optional *sandwich norm*: the attention output and the MLP output are each normalised
again before they join the residual stream (post_attention_layernorm / post_mlp_layernorm
act on the branch, pre_mlp_layernorm does the residual add + norm).  Everything else is
the DeepSeek decoder, which this module reuses.  Counterpart of
omni_npu/v1/models/pangu/pangu_ultra_moe.py:102-341 (MoE :102-224, decoder layer
:226-343) and, for the MTP variant, pangu_ultra_moe_mtp.py:45-315 (served here by the
generic multi-token predictor over this decoder layer).

``PanguProMoEV2ForCausalLM``: grouped-query attention with learned *sink* key/value
tokens that every sequence attends to, separate K and V head sizes, sliding-window layers
interleaved with full-attention layers, and a softmax-routed MoE.  Counterpart of
omni_npu/v1/models/pangu/pangu_pro_moe.py:324-693,935-1217.
"""
from __future__ import annotations

import dataclasses
from typing import Iterable, Tuple

import torch

from ..config import EngineConfig
from ..layers.norm import RMSNorm, reduce_add_rms_norm
from .deepseek import DeepseekDecoderLayer, DeepseekForCausalLM


class PanguUltraDecoderLayer(DeepseekDecoderLayer):
    def __init__(self, engine: EngineConfig, layer_idx: int, device, prefix: str) -> None:
        super().__init__(engine, layer_idx, device, prefix)
        cfg = engine.model
        self.sandwich_norm = bool(cfg.hf_config.get("sandwich_norm", False))
        if self.sandwich_norm:
            self.pre_mlp_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)
            self.post_mlp_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)

    def forward(self, hidden, residual, pending_reduce: bool):
        if not self.sandwich_norm:
            return super().forward(hidden, residual, pending_reduce)
        tp = self.tp_group
        if residual is None:
            residual = hidden
            hidden = self.input_layernorm(hidden)
        elif pending_reduce:
            hidden, residual = reduce_add_rms_norm(self.input_layernorm, hidden, residual, tp)
        else:
            hidden, residual = self.input_layernorm(hidden, residual)
        # the branch outputs are normalised on their own, so they must be fully reduced first
        hidden = self.self_attn(hidden, reduce=True)
        hidden = self.post_attention_layernorm(hidden)
        hidden, residual = self.pre_mlp_layernorm(hidden, residual)
        hidden = self.mlp(hidden) if self.is_moe else self.mlp(hidden, reduce=True)
        hidden = self.post_mlp_layernorm(hidden)
        return hidden, residual, False


def _ultra_config(engine: EngineConfig) -> EngineConfig:
    """Routing of openPangu Ultra: sigmoid scores, one group, bias only when the
    checkpoint says so (pangu_ultra_moe.py:131-141,178-190)."""
    cfg = engine.model
    hf = cfg.hf_config or {}
    model = dataclasses.replace(cfg, scoring_func="sigmoid", n_group=1, topk_group=1,
                                router_bias=bool(hf.get("router_enable_expert_bias", cfg.router_bias)))
    return dataclasses.replace(engine, model=model)


class PanguUltraMoEForCausalLM(DeepseekForCausalLM):
    decoder_layer_cls = PanguUltraDecoderLayer

    def __init__(self, engine_config: EngineConfig, device=None) -> None:
        super().__init__(_ultra_config(engine_config), device)

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        # the router bias is stored next to the gate weight under either name
        renamed = ((n.replace(".mlp.gate.e_score_correction_bias", ".mlp.e_score_correction_bias")
                    .replace(".mlp.gate.bias", ".mlp.e_score_correction_bias"), t) for n, t in weights)
        return super().load_weights(renamed)
