"""DeepSeek V2 / V2-Lite / V3 / V3.2 decoder.

Multi-head latent attention (optionally DeepSeek sparse attention when the
config carries ``index_topk``), dense FFN in the first ``first_k_dense_replace``
layers and a shared + routed mixture of experts afterwards.  Mirrors the
structure of omni_npu/v1/models/deepseek/deepseek_v3.py:64-777: the decoder
layer picks the sparse attention block when the HF config has ``index_topk``
(:288-306), weights of gate/up and of the experts are stacked at load time
(:591-777), MTP layers are skipped by the main model.
"""
from __future__ import annotations

import re
from typing import Iterable, List, Optional, Tuple

import torch
from torch import nn

from ..attention.mla import MLAAttention, MLABackend, StaticSinkMLAAttention
from ..config import EngineConfig, ModelConfig
from ..layers.embedding import ParallelLMHead, VocabParallelEmbedding
from ..layers.linear import Fp8BlockLinearMethod
from ..layers.mlp import FusedMLP
from ..layers.moe import FusedMoE
from ..layers.norm import RMSNorm, reduce_add_rms_norm
from ..parallel import state as pstate
from .utils import IntermediateTensors, PPMissingLayer, build_pipeline_layers, load_stacked_weights

_EXPERT_RE = re.compile(r"(.*)\.mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.(weight|weight_scale_inv)$")


def _quant_factory(cfg: ModelConfig):
    if cfg.quant_method == "fp8":
        return lambda: Fp8BlockLinearMethod(cfg.weight_block_size)
    return lambda: None


class DeepseekDecoderLayer(nn.Module):
    takes_pending = True      # forward(hidden, residual, pending_reduce) -> (hidden, residual, pending)

    def __init__(self, engine: EngineConfig, layer_idx: int, device, prefix: str) -> None:
        super().__init__()
        cfg = engine.model
        qf = _quant_factory(cfg)
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)
        if cfg.use_sparse:
            from ..attention.dsa import SparseMLAAttention
            self.self_attn = SparseMLAAttention(cfg, layer_idx, device, f"{prefix}.self_attn", qf)
        elif int((cfg.hf_config or {}).get("param_sink_number", 0)) or cfg.sliding_window:
            # learned static sink tokens and / or a sliding window on the latent cache
            self.self_attn = StaticSinkMLAAttention(cfg, layer_idx, device, f"{prefix}.self_attn", qf,
                                                    sink_len=int((cfg.hf_config or {}).get("param_sink_number", 0)),
                                                    sliding_window=cfg.sliding_window)
        else:
            self.self_attn = MLAAttention(cfg, layer_idx, device, f"{prefix}.self_attn", qf)
        if engine.parallel.decode_context_parallel_size > 1 and pstate.get_tp_group().world_size > 1:
            self.self_attn.cp_group = pstate.get_tp_group()
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)
        self.is_moe = cfg.layer_is_moe(layer_idx)
        if self.is_moe:
            self.mlp = FusedMoE(cfg.num_experts, cfg.num_experts_per_tok, cfg.hidden_size,
                                cfg.moe_intermediate_size, cfg.dtype, device, cfg.scoring_func,
                                cfg.norm_topk_prob, cfg.routed_scaling_factor, cfg.n_group, cfg.topk_group,
                                cfg.router_bias, cfg.num_shared_experts,
                                enable_expert_parallel=engine.parallel.enable_expert_parallel
                                or engine.parallel.tensor_parallel_size > 1,
                                prefix=f"{prefix}.mlp", max_tokens=engine.scheduler.max_num_batched_tokens,
                                quant="fp8" if cfg.quant_method == "fp8" else None,
                                shared_quant_factory=qf if cfg.quant_method == "fp8" else None,
                                num_redundant_experts=engine.parallel.num_redundant_experts)
        else:
            self.mlp = FusedMLP(cfg.hidden_size, cfg.intermediate_size, cfg.dtype, device,
                                quant_method_factory=qf, prefix=f"{prefix}.mlp",
                                fuse_swiglu=cfg.quant_method is None)
        self.tp_group = pstate.get_tp_group()
        self.prefetcher = None            # set by the model's post_load when weight prefetch is on
        self.next_attn = None

    def forward(self, hidden, residual, pending_reduce: bool):
        tp = self.tp_group
        pf = self.prefetcher
        if pf is not None:                # this layer's MLP / expert weights, while attention runs
            pf.prefetch_moe(self.mlp) if self.is_moe else pf.prefetch_mlp(self.mlp)
        if residual is None:
            residual = hidden
            hidden = self.input_layernorm(hidden)
        elif pending_reduce:
            hidden, residual = reduce_add_rms_norm(self.input_layernorm, hidden, residual, tp)
        else:
            hidden, residual = self.input_layernorm(hidden, residual)
        hidden = self.self_attn(hidden, reduce=False)
        hidden, residual = reduce_add_rms_norm(self.post_attention_layernorm, hidden, residual, tp)
        if pf is not None and self.next_attn is not None:      # the next layer's projections, while the MLP runs
            pf.prefetch_attention(self.next_attn)
        if self.is_moe:
            return self.mlp(hidden), residual, False
        return self.mlp(hidden, reduce=False), residual, True


class DeepseekModel(nn.Module):
    def __init__(self, engine: EngineConfig, device, layer_cls=None) -> None:
        super().__init__()
        cfg = engine.model
        layer_cls = layer_cls or DeepseekDecoderLayer
        pp = pstate.get_pp_group()
        self.pp_group = pp if pp.world_size > 1 else None
        first = self.pp_group is None or pp.is_first_rank
        last = self.pp_group is None or pp.is_last_rank
        self.hidden_size = cfg.hidden_size
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype, device) \
            if first else PPMissingLayer()
        self.layers, self.start_layer, self.end_layer = build_pipeline_layers(
            cfg.num_layers, lambda i: layer_cls(engine, i, device, f"model.layers.{i}"), self.pp_group)
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

    def forward(self, input_ids, positions, inputs_embeds=None, return_prenorm: bool = False,
                intermediate_tensors: Optional[IntermediateTensors] = None):
        """With pipeline stages: the first stage embeds, later ones start from the received
        (hidden, residual); a stage that is not the last returns ``IntermediateTensors``.  A
        tensor-parallel reduction still pending at the boundary is done before the hand-over,
        so the next stage always starts from a reduced ``hidden``."""
        pp = self.pp_group
        residual, pending = None, False
        if pp is None or pp.is_first_rank:
            hidden = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
        else:
            hidden, residual = intermediate_tensors["hidden_states"], intermediate_tensors["residual"]
        for layer in self._stage_layers():
            hidden, residual, pending = layer(hidden, residual, pending)
        if pp is not None and not pp.is_last_rank:
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


class DeepseekForCausalLM(nn.Module):
    stacked_params_mapping = [(".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1)]
    decoder_layer_cls = None          # subclasses may swap the decoder layer

    def __init__(self, engine_config: EngineConfig, device=None) -> None:
        super().__init__()
        self.config = engine_config.model
        self.engine_config = engine_config
        layer_cls = type(self).decoder_layer_cls or DeepseekDecoderLayer
        self.model = DeepseekModel(engine_config, device, layer_cls)
        pp = self.model.pp_group
        self.lm_head = ParallelLMHead(self.config.vocab_size, self.config.hidden_size, self.config.dtype, device) \
            if pp is None or pp.is_last_rank else PPMissingLayer()
        self.mtp = None
        self.num_kv_layers = self.model.end_layer - self.model.start_layer
        spec = engine_config.speculative
        if spec.method in ("mtp", "deepseek_mtp") and spec.num_speculative_tokens > 0:
            from .mtp import MultiTokenPredictor
            self.mtp = MultiTokenPredictor(
                engine_config, device,
                lambda idx, prefix: layer_cls(engine_config, idx, device, prefix))
            self.num_kv_layers += self.mtp.num_mtp_layers
        self.prefetcher = None

    def post_load(self) -> None:
        """After the weights are in place: wire the L2 weight prefetcher into the decoder layers when
        the deployment plan (or ``additional_config["weight_prefetch"]``) asks for it.  Each layer
        then hints its own MLP / expert weights into L2 while its attention runs and the next
        layer's attention projections while its MLP runs
        (reference: ``prefetch_post_load`` and the per-layer hints,
        omni_npu/v1/models/deepseek/deepseek_v3.py:165-218,398-428)."""
        from ..layers.prefetch import Prefetcher
        from .config_loader import model_extra_config
        want = self.engine_config.additional_config.get("weight_prefetch")
        plan = model_extra_config.kernels
        if want is None:
            want = model_extra_config.source is not None and plan.enable_prefetch
        dev = next(self.parameters()).device
        if not want or dev.type != "cuda":
            return
        self.prefetcher = Prefetcher.from_plan(dev, plan)
        layers = self.model._stage_layers()
        for i, layer in enumerate(layers):
            layer.prefetcher = self.prefetcher
            layer.next_attn = layers[i + 1].self_attn if i + 1 < len(layers) else None

    def forward(self, input_ids, positions, inputs_embeds=None, intermediate_tensors=None):
        return self.model(input_ids, positions, inputs_embeds, intermediate_tensors=intermediate_tensors)

    def make_empty_intermediate_tensors(self, num_tokens: int, dtype, device):
        return self.model.make_empty_intermediate_tensors(num_tokens, dtype, device)

    def mtp_forward(self, next_ids, positions, hidden, spec_step: int = 0):
        return self.mtp(self.model.embed_tokens(next_ids), hidden, spec_step)

    def mtp_logits(self, hidden):
        return (self.mtp.own_head or self.lm_head).compute_logits(hidden)

    def compute_logits(self, hidden):
        return self.lm_head.compute_logits(hidden)

    # ---- KV cache: one latent cache per layer (+ indexer key cache for sparse attention)
    def get_kv_cache_spec(self, block_size: int):
        from ..worker.model_runner import KVCacheSpec
        c = self.config
        per = MLABackend.bytes_per_block(block_size, c.kv_lora_rank, c.qk_rope_head_dim, c.dtype)
        shapes = {"latent": (block_size, c.kv_lora_rank + c.qk_rope_head_dim)}
        if c.use_sparse:
            per += block_size * c.index_head_dim * c.dtype.itemsize
            shapes["index_key"] = (block_size, c.index_head_dim)
        n = self.num_kv_layers
        return KVCacheSpec("dsa" if c.use_sparse else "mla", n, block_size, per * n, shapes)

    def allocate_kv_cache(self, num_blocks: int, block_size: int, device) -> List:
        c = self.config
        caches = []
        for _ in range(self.num_kv_layers):
            lat = MLABackend.allocate_kv_cache(num_blocks, block_size, c.kv_lora_rank, c.qk_rope_head_dim,
                                               c.dtype, device)
            if c.use_sparse:
                idx = torch.zeros(num_blocks, block_size, c.index_head_dim, dtype=c.dtype, device=device)
                caches.append((lat, idx))
            else:
                caches.append(lat)
        return caches

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        loaded, rest = set(), []
        n_layers = self.config.num_layers
        for name, tensor in weights:
            m = re.match(r"model\.layers\.(\d+)\.", name)
            if m and int(m.group(1)) >= n_layers:
                # multi-token-prediction layers: loaded only when the head is in use
                new = self.mtp.rewrite_name(name) if self.mtp is not None else None
                if new is None or new.startswith("__"):
                    continue
                name = "mtp." + new
            em = _EXPERT_RE.match(name)
            if em is None:
                rest.append((name.replace(".mlp.gate.e_score_correction_bias", ".mlp.e_score_correction_bias"),
                             tensor))
                continue
            prefix, eid, proj, kind = em.group(1), int(em.group(2)), em.group(3), em.group(4)
            try:
                moe: FusedMoE = self.get_submodule(prefix + ".mlp")
            except AttributeError:        # a layer of another pipeline stage
                continue
            pname = ("w13" if proj != "down_proj" else "w2") + ("" if kind == "weight" else "_scale")
            if not hasattr(moe, pname):
                continue
            shard = {"gate_proj": "gate", "up_proj": "up", "down_proj": "down"}[proj]
            if moe.weight_loader(getattr(moe, pname), tensor, eid, shard):
                loaded.add(f"{prefix}.mlp.{pname}")
        loaded |= load_stacked_weights(self, rest, self.stacked_params_mapping,
                                       skip_substrings=("rotary_emb.inv_freq",))
        return loaded


DeepseekV2ForCausalLM = DeepseekForCausalLM
DeepseekV3ForCausalLM = DeepseekForCausalLM
DeepseekV32ForCausalLM = DeepseekForCausalLM
