"""Qwen3-MoE (e.g. Qwen3-30B-A3B): GQA attention with per-head q/k RMSNorm and a
softmax-gated top-k mixture of experts in every layer (optionally interleaved
with dense MLP layers).

The reference's Qwen3-MoE implementation keeps the residual stream sharded over
tokens across the tensor-parallel group ("FlashComm-1") and offers four MoE
data paths (omni_npu/v0/models/qwen/qwen3_moe.py:216-464,
omni_npu/v0/models/qwen/fused_moe/layer.py:528-704); here one dispatch/combine
path covers prefill and decode and the all-reduce tails are fused with the
following norm.
"""
from __future__ import annotations

import re
from typing import Iterable, Optional, Tuple

import torch
from torch import nn

from ..config import EngineConfig, ModelConfig
from ..layers.embedding import ParallelLMHead, VocabParallelEmbedding
from ..layers.mlp import FusedMLP
from ..layers.moe import FusedMoE
from ..layers.norm import RMSNorm, reduce_add_rms_norm
from ..parallel import state as pstate
from .llama import LlamaAttention
from .utils import load_stacked_weights

_EXPERT_RE = re.compile(r"(.*)\.mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.(weight|weight_scale_inv)$")


class Qwen3MoeDecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device, prefix: str, engine: EngineConfig) -> None:
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)
        self.self_attn = LlamaAttention(cfg, layer_idx, device, f"{prefix}.self_attn")
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)
        self.is_moe = cfg.layer_is_moe(layer_idx)
        if self.is_moe:
            self.mlp = FusedMoE(cfg.num_experts, cfg.num_experts_per_tok, cfg.hidden_size,
                                cfg.moe_intermediate_size, cfg.dtype, device, cfg.scoring_func,
                                cfg.norm_topk_prob, cfg.routed_scaling_factor, cfg.n_group,
                                cfg.topk_group, cfg.router_bias, cfg.num_shared_experts,
                                enable_expert_parallel=engine.parallel.enable_expert_parallel
                                or engine.parallel.tensor_parallel_size > 1,
                                prefix=f"{prefix}.mlp",
                                max_tokens=engine.scheduler.max_num_batched_tokens,
                                num_redundant_experts=engine.parallel.num_redundant_experts)
        else:
            self.mlp = FusedMLP(cfg.hidden_size, cfg.intermediate_size, cfg.dtype, device,
                                prefix=f"{prefix}.mlp")
        self.tp_group = pstate.get_tp_group()

    def forward(self, hidden: torch.Tensor, residual: Optional[torch.Tensor], pending_reduce: bool):
        """``pending_reduce`` tells whether ``hidden`` still has to be summed over the
        tensor-parallel group (true after a dense MLP, false after an MoE block)."""
        tp = self.tp_group
        if residual is None:
            residual = hidden
            hidden = self.input_layernorm(hidden)
        elif pending_reduce:
            hidden, residual = reduce_add_rms_norm(self.input_layernorm, hidden, residual, tp)
        else:
            hidden, residual = self.input_layernorm(hidden, residual)
        hidden = self.self_attn(hidden, reduce=False)
        hidden, residual = reduce_add_rms_norm(self.post_attention_layernorm, hidden, residual, tp)
        if self.is_moe:
            return self.mlp(hidden), residual, False
        return self.mlp(hidden, reduce=False), residual, True

    def forward_sequence_parallel(self, sp, hidden: Optional[torch.Tensor], residual: torch.Tensor):
        """Token-sharded residual stream (layers/flashcomm.py): attention between an
        all-gather and a reduce-scatter; the MoE block consumes the gathered rows and its
        (already complete) output is sliced back to this rank's tokens."""
        hidden, residual = sp.block(self.input_layernorm, hidden, residual,
                                    lambda full: self.self_attn(full, reduce=False))
        if not self.is_moe:
            return sp.block(self.post_attention_layernorm, hidden, residual,
                            lambda full: self.mlp(full, reduce=False))
        normed, residual = self.post_attention_layernorm(hidden, residual)
        full = sp.gather(normed)[: sp.num_tokens]
        return sp.scatter(self.mlp(full)), residual


class Qwen3MoeModel(nn.Module):
    def __init__(self, engine: EngineConfig, device) -> None:
        super().__init__()
        cfg = engine.model
        self.sequence_parallel = bool(engine.parallel.sequence_parallel_residual)
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype, device)
        self.layers = nn.ModuleList([Qwen3MoeDecoderLayer(cfg, i, device, f"model.layers.{i}", engine)
                                     for i in range(cfg.num_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)

    def forward(self, input_ids, positions, inputs_embeds=None) -> torch.Tensor:
        hidden = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
        tp = pstate.get_tp_group()
        if self.sequence_parallel and tp.world_size > 1:
            from ..layers.flashcomm import SequenceParallelStream
            sp = SequenceParallelStream(tp)
            residual, hidden = sp.scatter(hidden), None
            for layer in self.layers:
                hidden, residual = layer.forward_sequence_parallel(sp, hidden, residual)
            hidden, _ = self.norm(hidden, residual)
            return sp.gather(hidden, trim=True)
        residual, pending = None, False
        for layer in self.layers:
            hidden, residual, pending = layer(hidden, residual, pending)
        if pending:
            hidden, _ = reduce_add_rms_norm(self.norm, hidden, residual, pstate.get_tp_group())
        else:
            hidden, _ = self.norm(hidden, residual)
        return hidden


class Qwen3MoeForCausalLM(nn.Module):
    stacked_params_mapping = [
        (".qkv_proj", ".q_proj", "q"), (".qkv_proj", ".k_proj", "k"), (".qkv_proj", ".v_proj", "v"),
        (".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1),
    ]

    def __init__(self, engine_config: EngineConfig, device=None) -> None:
        super().__init__()
        self.config = engine_config.model
        self.model = Qwen3MoeModel(engine_config, device)
        self.lm_head = ParallelLMHead(self.config.vocab_size, self.config.hidden_size, self.config.dtype, device)

    def forward(self, input_ids, positions, inputs_embeds=None):
        return self.model(input_ids, positions, inputs_embeds)

    def compute_logits(self, hidden):
        return self.lm_head.compute_logits(hidden)

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        loaded = set()
        rest = []
        params = dict(self.named_parameters())
        for name, tensor in weights:
            m = _EXPERT_RE.match(name)
            if m is None:
                rest.append((name, tensor))
                continue
            prefix, eid, proj, kind = m.group(1), int(m.group(2)), m.group(3), m.group(4)
            moe: FusedMoE = self.get_submodule(prefix + ".mlp")
            pname = {"gate_proj": "w13", "up_proj": "w13", "down_proj": "w2"}[proj]
            if kind != "weight":
                pname += "_scale"
            shard = {"gate_proj": "gate", "up_proj": "up", "down_proj": "down"}[proj]
            if moe.weight_loader(getattr(moe, pname), tensor, eid, shard):
                loaded.add(f"{prefix}.mlp.{pname}")
        loaded |= load_stacked_weights(self, rest, self.stacked_params_mapping,
                                       skip_substrings=("rotary_emb.inv_freq",))
        return loaded
