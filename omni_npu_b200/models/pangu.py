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


# ===================================================================== Pangu Pro MoE V2
from typing import List, Optional  # noqa: E402

from torch import nn  # noqa: E402

from .. import ops  # noqa: E402
from ..attention.gqa import GQABackend  # noqa: E402
from ..attention.metadata import get_forward_context  # noqa: E402
from ..layers.embedding import ParallelLMHead, VocabParallelEmbedding  # noqa: E402
from ..layers.linear import ColumnParallelLinear, RowParallelLinear  # noqa: E402
from ..layers.rope import get_rope  # noqa: E402
from ..parallel import state as pstate  # noqa: E402
from .qwen3_moe import Qwen3MoeDecoderLayer  # noqa: E402
from .utils import load_stacked_weights  # noqa: E402

_CUDA_HEAD_DIMS = {(128, 128), (64, 64), (192, 128)}     # (qk, v) pairs the attention kernels are built for


class PanguSinkAttention(nn.Module):
    """Grouped-query attention with learned attention sinks.

    ``param_sink_number`` key/value vectors per KV head are parameters of the layer.  They
    are normalised like ordinary keys (k_layernorm), laid out like rotated keys (the rotary
    part de-interleaved, no rotation applied) and written ONCE into reserved blocks of the
    layer's KV cache; every sequence's block table is prefixed with those blocks, so the
    sinks are simply the first tokens of every context.  Sliding-window layers keep the
    sinks visible (``sink`` argument of the attention kernels).  K and V may have different
    head sizes.  Counterpart of OpenPanguSinkAttention / StaticSinkAttention
    (omni_npu/v1/models/pangu/pangu_pro_moe.py:500-693,935-1217)."""

    def __init__(self, cfg, layer_idx: int, device, prefix: str) -> None:
        super().__init__()
        hf = cfg.hf_config or {}
        tp = pstate.get_tp_group()
        self.layer_idx = layer_idx
        self.head_dim = cfg.head_dim
        self.v_dim = int(hf.get("v_channels", cfg.head_dim))
        self.rope_dim = int(hf.get("qk_rope_dim", cfg.rotary_dim))
        self.num_heads = cfg.num_heads // tp.world_size
        self.num_kv_heads = max(1, cfg.num_kv_heads // tp.world_size)
        self.kv_head_start = (tp.rank_in_group * cfg.num_kv_heads) // tp.world_size
        self.sink_len = int(hf.get("param_sink_number", 0))
        self.sink_with_value = bool(hf.get("param_sink_with_value", False))
        win = hf.get("interleaved_sliding_window")
        if isinstance(win, list):
            win = win[layer_idx % len(win)]
        self.window = int(win or 0)
        dt = cfg.dtype
        kw = dict(dtype=dt, device=device, bias=cfg.attention_bias)
        self.q_proj = ColumnParallelLinear(cfg.hidden_size, cfg.num_heads * self.head_dim, prefix=f"{prefix}.q_proj", **kw)
        self.k_proj = ColumnParallelLinear(cfg.hidden_size, cfg.num_kv_heads * self.head_dim, prefix=f"{prefix}.k_proj", **kw)
        self.v_proj = ColumnParallelLinear(cfg.hidden_size, cfg.num_kv_heads * self.v_dim, prefix=f"{prefix}.v_proj", **kw)
        self.o_proj = RowParallelLinear(cfg.num_heads * self.v_dim, cfg.hidden_size, dtype=dt, device=device,
                                        prefix=f"{prefix}.o_proj")
        self.k_layernorm = RMSNorm(self.head_dim, cfg.rms_norm_eps, dt, device)
        self.rotary = get_rope(self.head_dim, self.rope_dim, cfg.max_position_embeddings, cfg.rope_theta, False,
                               cfg.rope_scaling, device)
        self.scale = self.head_dim ** -0.5
        if self.sink_len > 0:
            self.param_sink_key = nn.Parameter(torch.zeros(self.sink_len, cfg.num_kv_heads, self.head_dim,
                                                           dtype=dt, device=device), requires_grad=False)
            self.param_sink_value = nn.Parameter(torch.zeros(self.sink_len, cfg.num_kv_heads, self.v_dim,
                                                             dtype=dt, device=device), requires_grad=False)
        # the value head size the cache is allocated with: padded to the key size when the
        # attention kernels have no (qk, v) variant for it
        self.cache_v_dim = self.v_dim
        self._sink_written_into = None
        self._sink_bt: Optional[torch.Tensor] = None

    def pick_cache_v_dim(self, device) -> int:
        if torch.device(device).type == "cuda" and (self.head_dim, self.v_dim) not in _CUDA_HEAD_DIMS:
            self.cache_v_dim = self.head_dim
        return self.cache_v_dim

    # ------------------------------------------------------------------ sinks
    def sink_key_layout(self, key: torch.Tensor) -> torch.Tensor:
        """Sink keys are stored the way rotated keys are: the rotary part de-interleaved
        (even lanes first, then odd lanes), the rest unchanged; no rotation is applied."""
        rot, rest = key[..., : self.rope_dim], key[..., self.rope_dim:]
        return torch.cat([rot[..., 0::2], rot[..., 1::2], rest], dim=-1)

    def _populate_sinks(self, k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
        s, bs = self.sink_len, k_cache.shape[2]
        if s % bs != 0:
            raise ValueError(f"param_sink_number={s} must be a multiple of the KV block size {bs}")
        lo = self.kv_head_start
        key = self.k_layernorm(self.param_sink_key[:, lo: lo + self.num_kv_heads].reshape(-1, self.head_dim))
        key = self.sink_key_layout(key.view(s, self.num_kv_heads, self.head_dim))
        val = self.param_sink_value[:, lo: lo + self.num_kv_heads]
        if not self.sink_with_value:
            val = torch.zeros_like(val)
        nb = s // bs
        # cache layout [block, head, token, dim]; sink token t lives in block 1 + t // bs
        k_cache[1: 1 + nb] = key.view(nb, bs, self.num_kv_heads, self.head_dim).permute(0, 2, 1, 3).to(k_cache.dtype)
        v_cache[1: 1 + nb].zero_()
        v_cache[1: 1 + nb, :, :, : self.v_dim] = val.reshape(nb, bs, self.num_kv_heads, self.v_dim).permute(0, 2, 1, 3).to(v_cache.dtype)
        self._sink_written_into = k_cache.data_ptr()
        self._sink_bt = torch.arange(1, 1 + nb, dtype=torch.int32, device=k_cache.device).view(1, nb)

    # ---------------------------------------------------------------- forward
    def forward(self, hidden: torch.Tensor, reduce: bool = True) -> torch.Tensor:
        ctx = get_forward_context()
        md = ctx.attn_metadata
        k_cache, v_cache = ctx.kv_caches[self.layer_idx]
        t = hidden.shape[0]
        q, k, v = self.q_proj(hidden), self.k_proj(hidden), self.v_proj(hidden)
        k = self.k_layernorm(k.reshape(-1, self.head_dim)).view(t, -1)
        q, k = self.rotary(md.positions, q.contiguous(), k.contiguous())
        if self.cache_v_dim != self.v_dim:
            v = torch.nn.functional.pad(v.view(t, self.num_kv_heads, self.v_dim), (0, self.cache_v_dim - self.v_dim))
            v = v.reshape(t, -1)
        ops.gqa_cache_write(k, v.contiguous(), k_cache, v_cache, md.slot_mapping)
        bt, lens, sink = md.block_tables, md.seq_lens, 0
        if self.sink_len > 0:
            if self._sink_written_into != k_cache.data_ptr():
                self._populate_sinks(k_cache, v_cache)
            sink = self.sink_len
            bt = torch.cat([self._sink_bt.expand(bt.shape[0], -1), bt], dim=1).contiguous()
            lens = lens + sink
        if md.is_prefill:
            o = ops.gqa_prefill(q, k_cache, v_cache, bt, md.cu_q, lens, md.num_seqs, md.max_q_len, self.num_heads,
                                self.scale, True, self.window, sink=sink)
        else:
            o = ops.gqa_decode(q, k_cache, v_cache, bt, lens, md.num_seqs, self.num_heads, self.scale, md.q_len,
                               self.window, max_seq_len=md.max_seq_len + sink, sink=sink)
        if self.cache_v_dim != self.v_dim:
            o = o.view(t, self.num_heads, self.cache_v_dim)[..., : self.v_dim].reshape(t, -1)
        return self.o_proj(o, reduce=reduce)


class PanguProDecoderLayer(Qwen3MoeDecoderLayer):
    def __init__(self, cfg, layer_idx: int, device, prefix: str, engine: EngineConfig) -> None:
        super().__init__(cfg, layer_idx, device, prefix, engine)
        self.self_attn = PanguSinkAttention(cfg, layer_idx, device, f"{prefix}.self_attn")


class PanguProModel(nn.Module):
    def __init__(self, engine: EngineConfig, device) -> None:
        super().__init__()
        cfg = engine.model
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype, device)
        self.layers = nn.ModuleList([PanguProDecoderLayer(cfg, i, device, f"model.layers.{i}", engine)
                                     for i in range(cfg.num_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)

    def forward(self, input_ids, positions, inputs_embeds=None):
        hidden = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
        residual, pending = None, False
        for layer in self.layers:
            hidden, residual, pending = layer(hidden, residual, pending)
        if pending:
            hidden, _ = reduce_add_rms_norm(self.norm, hidden, residual, pstate.get_tp_group())
        else:
            hidden, _ = self.norm(hidden, residual)
        return hidden


class PanguProMoEV2ForCausalLM(nn.Module):
    stacked_params_mapping = [(".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1)]

    def __init__(self, engine_config: EngineConfig, device=None) -> None:
        super().__init__()
        self.config = engine_config.model
        self.engine_config = engine_config
        self.model = PanguProModel(engine_config, device)
        self.lm_head = ParallelLMHead(self.config.vocab_size, self.config.hidden_size, self.config.dtype, device)
        sink = int((self.config.hf_config or {}).get("param_sink_number", 0))
        bs = engine_config.cache.block_size
        # block 0 is the null block, the next ones hold the sink tokens of every layer's cache
        self.num_reserved_kv_blocks = 1 + (sink + bs - 1) // bs if sink > 0 else 0

    def forward(self, input_ids, positions, inputs_embeds=None):
        return self.model(input_ids, positions, inputs_embeds)

    def compute_logits(self, hidden):
        return self.lm_head.compute_logits(hidden)

    # ---- KV cache with separate key / value head sizes
    def _attn0(self) -> PanguSinkAttention:
        return self.model.layers[0].self_attn

    def get_kv_cache_spec(self, block_size: int):
        from ..worker.model_runner import KVCacheSpec
        a, c = self._attn0(), self.config
        dv = a.pick_cache_v_dim(self.lm_head.weight.device)
        per = GQABackend.bytes_per_block(block_size, a.num_kv_heads, a.head_dim, c.dtype, dv)
        k_shape, v_shape = GQABackend.get_kv_cache_shape(1, block_size, a.num_kv_heads, a.head_dim, dv)
        return KVCacheSpec("gqa", c.num_layers, block_size, per * c.num_layers, {"k": k_shape[1:], "v": v_shape[1:]})

    def allocate_kv_cache(self, num_blocks: int, block_size: int, device) -> List:
        caches = []
        for layer in self.model.layers:
            a = layer.self_attn
            dv = a.pick_cache_v_dim(device)
            caches.append(GQABackend.allocate_kv_cache(num_blocks, block_size, a.num_kv_heads, a.head_dim,
                                                       self.config.dtype, device, dv))
        return caches

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        import re
        expert_re = re.compile(r"(.*)\.mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")
        loaded, rest = set(), []
        for name, tensor in weights:
            m = expert_re.match(name)
            if m is None:
                rest.append((name.replace(".mlp.gate.e_score_correction_bias", ".mlp.e_score_correction_bias"), tensor))
                continue
            moe = self.get_submodule(m.group(1) + ".mlp")
            shard = {"gate_proj": "gate", "up_proj": "up", "down_proj": "down"}[m.group(3)]
            pname = "w13" if shard != "down" else "w2"
            if moe.weight_loader(getattr(moe, pname), tensor, int(m.group(2)), shard):
                loaded.add(f"{m.group(1)}.mlp.{pname}")
        return loaded | load_stacked_weights(self, rest, self.stacked_params_mapping,
                                             skip_substrings=("rotary_emb.inv_freq",))
