"""Dense decoder-only transformer (Llama / Qwen2 / Qwen3 family).

One implementation covers the three: Qwen2 adds QKV bias, Qwen3 adds per-head
RMSNorm on q and k (reference: omni_npu/v1/models/qwen/qwen3.py:60-173).
"""
from __future__ import annotations

import os

from typing import Iterable, Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..attention.gqa import GQAAttention
from ..config import EngineConfig, ModelConfig
from ..layers.embedding import ParallelLMHead, VocabParallelEmbedding
from ..layers.linear import row_parallel_add_rms_norm
from ..layers.linear import QKVParallelLinear, RowParallelLinear
from ..layers.mlp import FusedMLP
from ..layers.norm import RMSNorm, reduce_add_rms_norm
from ..layers.rope import get_rope
from ..attention.metadata import get_forward_context
from ..parallel import state as pstate
from .utils import IntermediateTensors, PPMissingLayer, load_stacked_weights, pp_layer_range


class LlamaAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device, prefix: str) -> None:
        super().__init__()
        self.head_dim = cfg.head_dim
        self.qkv_proj = QKVParallelLinear(cfg.hidden_size, cfg.head_dim, cfg.num_heads,
                                          cfg.num_kv_heads, bias=cfg.attention_bias, dtype=cfg.dtype,
                                          device=device, prefix=f"{prefix}.qkv_proj")
        self.o_proj = RowParallelLinear(cfg.num_heads * cfg.head_dim, cfg.hidden_size, dtype=cfg.dtype,
                                        device=device, prefix=f"{prefix}.o_proj")
        self.qk_norm = cfg.qk_norm
        if cfg.qk_norm:
            self.q_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, cfg.dtype, device)
            self.k_norm = RMSNorm(cfg.head_dim, cfg.rms_norm_eps, cfg.dtype, device)
        self.rotary = get_rope(cfg.head_dim, cfg.rotary_dim, cfg.max_position_embeddings,
                               cfg.rope_theta, cfg.rope_neox, cfg.rope_scaling, device)
        self.attn = GQAAttention(layer_idx, self.qkv_proj.num_heads, self.qkv_proj.num_kv_heads,
                                 cfg.head_dim, cfg.head_dim ** -0.5 * self.rotary.mscale ** 2
                                 if self.rotary.mscale != 1.0 else cfg.head_dim ** -0.5,
                                 cfg.rotary_dim, cfg.rope_neox, cfg.sliding_window)

    def forward(self, hidden: torch.Tensor, reduce: bool = True, fuse_norm=None):
        q, k, v = self.qkv_proj(hidden)
        if self.qk_norm:
            t = q.shape[0]
            q = self.q_norm(q.reshape(-1, self.head_dim)).view(t, -1)
            k = self.k_norm(k.reshape(-1, self.head_dim)).view(t, -1)
        o = self.attn(q, k, v, self.rotary.cos_sin_cache)
        if fuse_norm is not None:
            # o_proj + tensor-parallel reduction + residual add + the following RMSNorm
            return row_parallel_add_rms_norm(self.o_proj, o, fuse_norm[0], fuse_norm[1])
        return self.o_proj(o, reduce=reduce)


class LlamaDecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device, prefix: str) -> None:
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)
        self.self_attn = LlamaAttention(cfg, layer_idx, device, f"{prefix}.self_attn")
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)
        self.mlp = FusedMLP(cfg.hidden_size, cfg.intermediate_size, cfg.dtype, device,
                            prefix=f"{prefix}.mlp")
        self.tp_group = pstate.get_tp_group()

    def forward(self, hidden: torch.Tensor, residual: Optional[torch.Tensor]):
        """``hidden`` is the previous layer's MLP output BEFORE its tensor-parallel
        reduction (or the embeddings for the first layer); the reduction is fused
        with this layer's residual add + input norm.  The returned ``hidden`` is
        likewise un-reduced."""
        tp = self.tp_group
        if residual is None:
            residual = hidden
            hidden = self.input_layernorm(hidden)
        else:
            hidden, residual = reduce_add_rms_norm(self.input_layernorm, hidden, residual, tp)
        hidden = self.self_attn(hidden, reduce=False)
        hidden, residual = reduce_add_rms_norm(self.post_attention_layernorm, hidden, residual, tp)
        hidden = self.mlp(hidden, reduce=False)
        return hidden, residual

    def forward_fused(self, hidden: torch.Tensor, residual: torch.Tensor, next_norm):
        """``hidden`` is this layer's input AFTER its input norm, ``residual`` the stream.  Both
        row-parallel projections run fused with their reduction, the residual add and the norm
        that follows them (this layer's post-attention norm; ``next_norm`` = the next layer's
        input norm or the model's final norm).  Returns (next layer's normed input, residual)."""
        hidden, residual = self.self_attn(hidden, fuse_norm=(self.post_attention_layernorm, residual))
        return self.mlp.forward_add_rms_norm(hidden, next_norm, residual)

    def forward_sequence_parallel(self, sp, hidden: Optional[torch.Tensor], residual: torch.Tensor):
        """The same layer on a token-sharded residual stream (layers/flashcomm.py)."""
        mode = sp.scatter_mode      # "scatter": o_proj / down_proj push their tiles to the row owners
        hidden, residual = sp.block(self.input_layernorm, hidden, residual,
                                    lambda full: self.self_attn(full, reduce=mode))
        return sp.block(self.post_attention_layernorm, hidden, residual,
                        lambda full: self.mlp(full, reduce=mode))


class LlamaModel(nn.Module):
    sequence_parallel = False       # set by the owning model from ParallelConfig
    # OMNI_B200_AUTO_SP=1: large prefill steps under tensor parallelism run on the token-sharded stream
    # (all-gather / reduce-scatter inside the GEMMs); default: replicated stream, all-reduce after the GEMMs
    auto_sequence_parallel = os.environ.get("OMNI_B200_AUTO_SP", "0") == "1"
    fused_tail = True               # GEMM + all-reduce + add + norm in one kernel where possible

    def __init__(self, cfg: ModelConfig, device, prefix: str = "model") -> None:
        super().__init__()
        # pipeline stage: this rank owns layers [start, end); the first stage embeds, the last one
        # applies the final norm.  KV caches are indexed by the layer's position within the stage.
        pp = pstate.get_pp_group() if pstate.model_parallel_is_initialized() else None
        self.pp_group = pp if pp is not None and pp.world_size > 1 else None
        first = self.pp_group is None or self.pp_group.is_first_rank
        last = self.pp_group is None or self.pp_group.is_last_rank
        self.start_layer, self.end_layer = (0, cfg.num_layers) if self.pp_group is None else \
            pp_layer_range(cfg.num_layers, pp.rank_in_group, pp.world_size)
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype, device) \
            if first or (last and cfg.tie_word_embeddings) else PPMissingLayer()
        self.layers = nn.ModuleList([
            LlamaDecoderLayer(cfg, i - self.start_layer, device, f"{prefix}.layers.{i}")
            if self.start_layer <= i < self.end_layer else PPMissingLayer()
            for i in range(cfg.num_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device) if last else PPMissingLayer()
        self.hidden_size = cfg.hidden_size

    def forward(self, input_ids: torch.Tensor, positions: torch.Tensor,
                inputs_embeds: Optional[torch.Tensor] = None,
                intermediate_tensors: Optional[IntermediateTensors] = None):
        if self.pp_group is not None:
            return self._forward_stage(input_ids, inputs_embeds, intermediate_tensors)
        hidden = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
        tp = pstate.get_tp_group()
        use_sp = self.sequence_parallel
        if not use_sp and self.auto_sequence_parallel and tp.world_size > 1 and hidden.is_cuda:
            # prefill steps whose rows split into whole 128-row tiles per rank run on the token-sharded
            # stream: the all-gathers and reduce-scatters then live inside the projections' GEMMs
            try:
                md = get_forward_context().attn_metadata
            except RuntimeError:          # called outside an engine step
                md = None
            use_sp = (md is not None and md.is_prefill and getattr(tp.comm, "symm", None) is not None
                      and hidden.shape[0] % (128 * tp.world_size) == 0)
        if use_sp and tp.world_size > 1:
            from ..layers.flashcomm import SequenceParallelStream
            sp = SequenceParallelStream(tp)
            sp.fused_gather = True      # qkv_proj / gate_up_proj read the token shards inside their GEMM
            residual, hidden = sp.scatter(hidden), None
            for layer in self.layers:
                hidden, residual = layer.forward_sequence_parallel(sp, hidden, residual)
            hidden, _ = self.norm(hidden, residual)
            return sp.gather(hidden, trim=True)
        if tp.world_size > 1 and getattr(tp.comm, "symm", None) is not None and self.fused_tail:
            # every row-parallel projection carries its reduction, residual add and next norm
            residual = hidden
            hidden = self.layers[0].input_layernorm(hidden)
            n = len(self.layers)
            for i, layer in enumerate(self.layers):
                nxt = self.layers[i + 1].input_layernorm if i + 1 < n else self.norm
                hidden, residual = layer.forward_fused(hidden, residual, nxt)
            return hidden
        residual = None
        for layer in self.layers:
            hidden, residual = layer(hidden, residual)
        hidden, _ = reduce_add_rms_norm(self.norm, hidden, residual, tp)
        return hidden

    def _forward_stage(self, input_ids, inputs_embeds, intermediate_tensors):
        """One pipeline stage.  ``hidden`` crosses the stage boundary BEFORE its tensor-parallel
        reduction, together with the residual stream: pipeline neighbours have the same
        tensor-parallel rank, so each rank forwards its own partial sum and the first layer of
        the next stage folds the reduction into its input norm as usual.  Returns the normed
        hidden states on the last stage and ``IntermediateTensors`` elsewhere."""
        pp, tp = self.pp_group, pstate.get_tp_group()
        if pp.is_first_rank:
            hidden = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
            residual = None
        else:
            hidden, residual = intermediate_tensors["hidden_states"], intermediate_tensors["residual"]
        for layer in self._stage_layers():
            hidden, residual = layer(hidden, residual)
        if not pp.is_last_rank:
            if residual is None:        # a stage without layers passes the embeddings on
                residual = torch.zeros_like(hidden)
            return IntermediateTensors({"hidden_states": hidden, "residual": residual})
        hidden, _ = reduce_add_rms_norm(self.norm, hidden, residual, tp)
        return hidden

    def _stage_layers(self):
        """This stage's decoder layers (all of them without pipeline parallelism), as a plain list
        built once: slicing the ``ModuleList`` would construct a new module on every forward."""
        cached = self.__dict__.get("_stage_layer_list")
        if cached is None:
            cached = list(self.layers)[self.start_layer:self.end_layer]
            self.__dict__["_stage_layer_list"] = cached
        return cached

    def make_empty_intermediate_tensors(self, num_tokens: int, dtype: torch.dtype, device) -> IntermediateTensors:
        h = self.hidden_size
        return IntermediateTensors({"hidden_states": torch.empty(num_tokens, h, dtype=dtype, device=device),
                                    "residual": torch.empty(num_tokens, h, dtype=dtype, device=device)})


class LlamaForCausalLM(nn.Module):
    stacked_params_mapping = [
        # (fused parameter, checkpoint name, shard id)
        (".qkv_proj", ".q_proj", "q"), (".qkv_proj", ".k_proj", "k"), (".qkv_proj", ".v_proj", "v"),
        (".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1),
    ]

    def __init__(self, engine_config: EngineConfig, device=None) -> None:
        super().__init__()
        cfg = engine_config.model
        self.config = cfg
        self.model = LlamaModel(cfg, device)
        self.model.sequence_parallel = bool(engine_config.parallel.sequence_parallel_residual)
        pp = self.model.pp_group
        if pp is not None and not pp.is_last_rank:
            self.lm_head = PPMissingLayer()          # logits and sampling happen on the last stage
        elif cfg.tie_word_embeddings:
            self.lm_head = self.model.embed_tokens
            self.lm_head.__class__ = ParallelLMHead
        else:
            self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype, device)
        self.mtp = None
        self.num_kv_layers = self.model.end_layer - self.model.start_layer
        spec = engine_config.speculative
        if spec.method in ("mtp", "deepseek_mtp") and spec.num_speculative_tokens > 0:
            from .mtp import MultiTokenPredictor
            self.mtp = MultiTokenPredictor(engine_config, device,
                                           lambda idx, prefix: LlamaDecoderLayer(cfg, idx, device, prefix))
            self.num_kv_layers += self.mtp.num_mtp_layers

    def forward(self, input_ids, positions, inputs_embeds=None, intermediate_tensors=None):
        return self.model(input_ids, positions, inputs_embeds, intermediate_tensors)

    def make_empty_intermediate_tensors(self, num_tokens: int, dtype: torch.dtype, device):
        return self.model.make_empty_intermediate_tensors(num_tokens, dtype, device)

    def mtp_forward(self, next_ids: torch.Tensor, positions: torch.Tensor, hidden: torch.Tensor,
                    spec_step: int = 0) -> torch.Tensor:
        """Hidden states of the MTP head for (embedding of the next token, target hidden state)."""
        return self.mtp(self.model.embed_tokens(next_ids), hidden, spec_step)

    def mtp_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        head = self.mtp.own_head or self.lm_head
        return head.compute_logits(hidden)

    def embed_input_ids(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.model.embed_tokens(input_ids)

    def compute_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.lm_head.compute_logits(hidden)

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        skip = ("rotary_emb.inv_freq",)
        if self.config.tie_word_embeddings:
            skip = skip + ("lm_head.weight",)
        if self.mtp is not None:
            weights, mtp_weights = self.mtp.split_weights(weights)
            loaded = load_stacked_weights(self, weights, self.stacked_params_mapping, skip_substrings=skip)
            return loaded | load_stacked_weights(self, [("mtp." + n, t) for n, t in mtp_weights],
                                                 self.stacked_params_mapping, skip_substrings=skip)
        return load_stacked_weights(self, weights, self.stacked_params_mapping, skip_substrings=skip)


# Qwen2 / Qwen3 dense share the implementation; differences come from ModelConfig.
Qwen2ForCausalLM = LlamaForCausalLM
Qwen3ForCausalLM = LlamaForCausalLM
MistralForCausalLM = LlamaForCausalLM
