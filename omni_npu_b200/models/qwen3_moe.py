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
from ..layers.linear import ReducedShard, ReplicatedLinear
from ..layers.mlp import FusedMLP
from ..layers.moe import FusedMoE
from ..layers.norm import RMSNorm, reduce_add_rms_norm
from ..parallel import state as pstate
from .llama import LlamaAttention
from .utils import IntermediateTensors, PPMissingLayer, build_pipeline_layers, load_stacked_weights

_EXPERT_RE = re.compile(r"(.*)\.mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.(weight|weight_scale_inv)$")


class HeadToSequenceAttention(LlamaAttention):
    """Attention whose output leaves the head-sharded layout by an all-to-all instead of a
    reduction (Ulysses style), for steps on the token-sharded residual stream.

    After attention every rank holds all tokens for ITS heads, ``[T, heads/tp * d]``.  The
    row-parallel o_proj would turn that into partial sums of ``[T, hidden]`` and reduce-scatter
    them (``T * hidden * (tp-1)/tp`` elements through each rank's links).  Here the rows are
    exchanged instead: tokens scattered, heads gathered -> ``[T/tp, heads * d]``, and a
    REPLICATED o_proj on those rows gives this rank's token shard complete, with
    ``T * heads * d * (tp-1) / tp**2`` elements per rank on the wire, tp times fewer.  The price
    is a full copy of the o_proj weight per rank; steps on the replicated stream (decode) keep
    using the rank's column slice of it as an ordinary row-parallel projection.
    (reference: ``prefill_enable_mla_alltoall`` and the replicated o_proj on the local
    sequence shard, omni_npu/v0/models/qwen/qwen3_moe.py:164-169,238-252; the DP<->TP o_proj
    linears omni_npu/v0/layers/linear.py:389-444)"""

    def __init__(self, cfg: ModelConfig, layer_idx: int, device, prefix: str) -> None:
        super().__init__(cfg, layer_idx, device, prefix)
        self.tp = pstate.get_tp_group()
        width = cfg.num_heads * cfg.head_dim
        if cfg.num_heads % self.tp.world_size:
            raise ValueError("head-to-sequence all-to-all needs num_heads divisible by the tensor-parallel size")
        self.o_proj_full = ReplicatedLinear(width, cfg.hidden_size, dtype=cfg.dtype, device=device,
                                            prefix=f"{prefix}.o_proj_full", x_transform="NoOp", y_transform="NoOp")
        per = width // self.tp.world_size
        self._cols = slice(self.tp.rank_in_group * per, (self.tp.rank_in_group + 1) * per)

    def process_weights_after_loading(self) -> None:
        # one source of truth: the row-parallel shard is this rank's columns of the full weight
        self.o_proj.weight.data.copy_(self.o_proj_full.weight.data[:, self._cols])

    def forward(self, hidden, reduce: bool = True, fuse_norm=None, stream=None):
        if stream is None or not stream.enabled:
            return super().forward(hidden, reduce=reduce, fuse_norm=fuse_norm)
        q, k, v = self.qkv_proj(hidden)
        if self.qk_norm:
            t = q.shape[0]
            q = self.q_norm(q.reshape(-1, self.head_dim)).view(t, -1)
            k = self.k_norm(k.reshape(-1, self.head_dim)).view(t, -1)
        o = self.attn(q, k, v, self.rotary.cos_sin_cache)
        if o.shape[0] != stream.padded:
            o = torch.cat([o, o.new_zeros(stream.padded - o.shape[0], o.shape[1])], dim=0)
        o = self.tp.comm.all_to_all(o, scatter_dim=0, gather_dim=-1)        # [T/tp, heads * d]
        return ReducedShard(self.o_proj_full(o))


class Qwen3MoeDecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device, prefix: str, engine: EngineConfig) -> None:
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)
        # additional_config["attn_output_all_to_all"]: head <-> sequence exchange after attention
        self.head_to_sequence = bool(engine.additional_config.get("attn_output_all_to_all", False)) \
            and pstate.get_tp_group().world_size > 1
        attn_cls = HeadToSequenceAttention if self.head_to_sequence else LlamaAttention
        self.self_attn = attn_cls(cfg, layer_idx, device, f"{prefix}.self_attn")
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
        if self.head_to_sequence:
            hidden, residual = sp.block(self.input_layernorm, hidden, residual,
                                        lambda full: self.self_attn(full, stream=sp))
        else:
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
        pp = pstate.get_pp_group()
        self.pp_group = pp if pp.world_size > 1 else None
        first = self.pp_group is None or pp.is_first_rank
        last = self.pp_group is None or pp.is_last_rank
        self.hidden_size = cfg.hidden_size
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype, device) \
            if first else PPMissingLayer()
        self.layers, self.start_layer, self.end_layer = build_pipeline_layers(
            cfg.num_layers, lambda i: Qwen3MoeDecoderLayer(cfg, i, device, f"model.layers.{i}", engine),
            self.pp_group)
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device) if last else PPMissingLayer()

    def _stage_layers(self):
        """This stage's decoder layers (all of them without pipeline parallelism), as a plain list
        built once: slicing the ``ModuleList`` would construct a new module on every forward."""
        cached = self.__dict__.get("_stage_layer_list")
        if cached is None:
            cached = list(self.layers)[self.start_layer:self.end_layer]
            self.__dict__["_stage_layer_list"] = cached
        return cached

    def make_empty_intermediate_tensors(self, num_tokens: int, dtype, device) -> IntermediateTensors:
        return IntermediateTensors({k: torch.empty(num_tokens, self.hidden_size, dtype=dtype, device=device)
                                    for k in ("hidden_states", "residual")})

    def _forward_stage(self, input_ids, inputs_embeds, intermediate_tensors):
        """This rank's pipeline stage on the replicated stream; a reduction still pending at the
        boundary is done before the hand-over."""
        pp = self.pp_group
        residual, pending = None, False
        if pp.is_first_rank:
            hidden = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
        else:
            hidden, residual = intermediate_tensors["hidden_states"], intermediate_tensors["residual"]
        for layer in self._stage_layers():
            hidden, residual, pending = layer(hidden, residual, pending)
        if not pp.is_last_rank:
            if pending:
                hidden = pstate.get_tp_group().all_reduce(hidden)
            if residual is None:
                residual = torch.zeros_like(hidden)
            return IntermediateTensors({"hidden_states": hidden, "residual": residual})
        if pending:
            hidden, _ = reduce_add_rms_norm(self.norm, hidden, residual, pstate.get_tp_group())
        else:
            hidden, _ = self.norm(hidden, residual)
        return hidden

    def forward(self, input_ids, positions, inputs_embeds=None, intermediate_tensors=None):
        if self.pp_group is not None:
            return self._forward_stage(input_ids, inputs_embeds, intermediate_tensors)
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
        pp = self.model.pp_group
        self.lm_head = ParallelLMHead(self.config.vocab_size, self.config.hidden_size, self.config.dtype, device) \
            if pp is None or pp.is_last_rank else PPMissingLayer()
        self.num_kv_layers = self.model.end_layer - self.model.start_layer

    def forward(self, input_ids, positions, inputs_embeds=None, intermediate_tensors=None):
        return self.model(input_ids, positions, inputs_embeds, intermediate_tensors)

    def make_empty_intermediate_tensors(self, num_tokens: int, dtype, device):
        return self.model.make_empty_intermediate_tensors(num_tokens, dtype, device)

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
                if name.endswith(".self_attn.o_proj.weight") and \
                        name.replace(".o_proj.", ".o_proj_full.") in params:
                    rest.append((name.replace(".o_proj.", ".o_proj_full."), tensor))
                continue
            prefix, eid, proj, kind = m.group(1), int(m.group(2)), m.group(3), m.group(4)
            try:
                moe: FusedMoE = self.get_submodule(prefix + ".mlp")
            except AttributeError:        # a layer of another pipeline stage
                continue
            pname = {"gate_proj": "w13", "up_proj": "w13", "down_proj": "w2"}[proj]
            if kind != "weight":
                pname += "_scale"
            shard = {"gate_proj": "gate", "up_proj": "up", "down_proj": "down"}[proj]
            if moe.weight_loader(getattr(moe, pname), tensor, eid, shard):
                loaded.add(f"{prefix}.mlp.{pname}")
        loaded |= load_stacked_weights(self, rest, self.stacked_params_mapping,
                                       skip_substrings=("rotary_emb.inv_freq",))
        return loaded
