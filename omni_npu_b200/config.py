"""Typed configuration objects.

One ``EngineConfig`` is built per engine from keyword arguments, an HF
``config.json`` dictionary and the free-form ``additional_config`` mapping; no
module-level singleton is mutated at import time.  (The reference scatters the
same information over ``VllmConfig``, ``additional_config`` keys, environment
variables and per-model JSON presets: omni_npu/platform.py:18-35,
omni_npu/worker/npu_model_runner.py:103-114,
omni_npu/v1/models/config_loader/loader.py:76-183.)
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16,
           "fp16": torch.float16, "float32": torch.float32, "fp32": torch.float32,
           "auto": torch.bfloat16}


def to_dtype(x) -> torch.dtype:
    if isinstance(x, torch.dtype):
        return x
    return _DTYPES[str(x).replace("torch.", "")]


@dataclass
class ModelConfig:
    architecture: str = "LlamaForCausalLM"
    model_type: str = "llama"
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 14336
    vocab_size: int = 128256
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    rope_scaling: Optional[Dict[str, Any]] = None
    partial_rotary_factor: float = 1.0
    rope_neox: bool = True
    max_position_embeddings: int = 8192
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    qk_norm: bool = False                 # Qwen3: per-head RMSNorm on q and k
    sliding_window: int = 0
    dtype: torch.dtype = torch.bfloat16
    # --- mixture of experts
    num_experts: int = 0                  # routed experts (0 = dense model)
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    num_shared_experts: int = 0
    first_k_dense: int = 0                # leading layers with a dense FFN
    moe_layer_freq: int = 1
    scoring_func: str = "softmax"         # "softmax" | "sigmoid"
    norm_topk_prob: bool = False
    routed_scaling_factor: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    router_bias: bool = False             # e_score_correction_bias (noaux_tc)
    # --- multi-head latent attention
    use_mla: bool = False
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    # --- DeepSeek sparse attention (lightning indexer)
    index_topk: int = 0
    index_n_heads: int = 0
    index_head_dim: int = 0
    # --- multi-token prediction
    num_nextn_predict_layers: int = 0
    # --- quantisation
    quant_method: Optional[str] = None    # None | "fp8" (128x128 block scales)
    weight_block_size: Tuple[int, int] = (128, 128)
    # --- misc
    eos_token_id: Optional[int] = None
    hf_config: Dict[str, Any] = field(default_factory=dict)

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def use_sparse(self) -> bool:
        return self.index_topk > 0

    @property
    def rotary_dim(self) -> int:
        if self.use_mla:
            return self.qk_rope_head_dim
        return int(self.head_dim * self.partial_rotary_factor)

    def layer_is_moe(self, idx: int) -> bool:
        return (self.is_moe and idx >= self.first_k_dense
                and (idx - self.first_k_dense) % max(1, self.moe_layer_freq) == 0)

    def kv_bytes_per_token(self) -> int:
        """Bytes of KV cache one token occupies across all layers (per TP-1 rank)."""
        esz = self.dtype.itemsize
        if self.use_mla:
            per = self.kv_lora_rank + self.qk_rope_head_dim + (self.index_head_dim if self.use_sparse else 0)
            return self.num_layers * per * esz
        return self.num_layers * 2 * self.num_kv_heads * self.head_dim * esz

    @classmethod
    def from_hf_dict(cls, d: Dict[str, Any], dtype=None) -> "ModelConfig":
        """Build from the contents of an HF ``config.json``."""
        if "text_config" in d and isinstance(d["text_config"], dict):
            merged = dict(d["text_config"])
            merged.setdefault("architectures", d.get("architectures"))
            d = merged
        arch = (d.get("architectures") or ["LlamaForCausalLM"])[0]
        heads = d.get("num_attention_heads", 32)
        hidden = d.get("hidden_size", 4096)
        c = cls(
            architecture=arch,
            model_type=d.get("model_type", "llama"),
            hidden_size=hidden,
            num_layers=d.get("num_hidden_layers", 32),
            num_heads=heads,
            num_kv_heads=d.get("num_key_value_heads", heads),
            head_dim=d.get("head_dim") or hidden // heads,
            intermediate_size=d.get("intermediate_size", 4 * hidden),
            vocab_size=d.get("vocab_size", 32000),
            rms_norm_eps=d.get("rms_norm_eps", 1e-6),
            rope_theta=d.get("rope_theta", 10000.0),
            rope_scaling=d.get("rope_scaling"),
            partial_rotary_factor=d.get("partial_rotary_factor", 1.0),
            max_position_embeddings=d.get("max_position_embeddings", 8192),
            tie_word_embeddings=d.get("tie_word_embeddings", False),
            attention_bias=d.get("attention_bias", False) or arch.startswith("Qwen2"),
            qk_norm=arch.startswith("Qwen3"),
            sliding_window=d.get("sliding_window") or 0 if d.get("use_sliding_window", False) else 0,
            dtype=to_dtype(dtype or d.get("torch_dtype", "bfloat16")),
            eos_token_id=d.get("eos_token_id") if isinstance(d.get("eos_token_id"), int) else None,
            hf_config=d,
        )
        # MoE (DeepSeek / Qwen3-MoE / Pangu naming variants)
        c.num_experts = d.get("n_routed_experts") or d.get("num_experts") or d.get("num_local_experts") or 0
        c.num_experts_per_tok = d.get("num_experts_per_tok", 0) if c.num_experts else 0
        c.moe_intermediate_size = d.get("moe_intermediate_size", 0)
        c.num_shared_experts = d.get("n_shared_experts") or 0
        c.first_k_dense = d.get("first_k_dense_replace", 0)
        c.moe_layer_freq = d.get("moe_layer_freq", 1) or 1
        c.scoring_func = d.get("scoring_func", "softmax")
        c.norm_topk_prob = d.get("norm_topk_prob", False)
        c.routed_scaling_factor = d.get("routed_scaling_factor", 1.0)
        c.n_group = d.get("n_group") or 1
        c.topk_group = d.get("topk_group") or 1
        c.router_bias = d.get("topk_method") == "noaux_tc"
        # MLA
        if d.get("kv_lora_rank"):
            c.use_mla = True
            c.q_lora_rank = d.get("q_lora_rank") or 0
            c.kv_lora_rank = d["kv_lora_rank"]
            c.qk_nope_head_dim = d.get("qk_nope_head_dim", 128)
            c.qk_rope_head_dim = d.get("qk_rope_head_dim", 64)
            c.v_head_dim = d.get("v_head_dim", 128)
            c.rope_neox = False
        c.index_topk = d.get("index_topk") or 0
        c.index_n_heads = d.get("index_n_heads") or 0
        c.index_head_dim = d.get("index_head_dim") or 0
        c.num_nextn_predict_layers = d.get("num_nextn_predict_layers") or 0
        q = d.get("quantization_config") or {}
        if q.get("quant_method") in ("fp8",):
            c.quant_method = "fp8"
            wbs = q.get("weight_block_size") or [128, 128]
            c.weight_block_size = (int(wbs[0]), int(wbs[1]))
        return c

    @classmethod
    def from_pretrained(cls, path: str, dtype=None) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_hf_dict(json.load(f), dtype=dtype)


# ----------------------------------------------------------------- presets
def tiny_llama(dtype=torch.float32) -> ModelConfig:
    """2 layers, hidden 256, 4 heads (head_dim 64), 2 KV heads, FFN 512, vocab 1024."""
    return ModelConfig(hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                       intermediate_size=512, vocab_size=1024, rope_theta=10000.0,
                       max_position_embeddings=2048, dtype=dtype)


def llama3_8b() -> ModelConfig:
    return ModelConfig()


def qwen3_30b_a3b() -> ModelConfig:
    return ModelConfig(architecture="Qwen3MoeForCausalLM", model_type="qwen3_moe", hidden_size=2048,
                       num_layers=48, num_heads=32, num_kv_heads=4, head_dim=128,
                       intermediate_size=6144, vocab_size=151936, rms_norm_eps=1e-6,
                       rope_theta=1000000.0, max_position_embeddings=40960, qk_norm=True,
                       num_experts=128, num_experts_per_tok=8, moe_intermediate_size=768,
                       norm_topk_prob=True)


def deepseek_v2_lite() -> ModelConfig:
    return ModelConfig(architecture="DeepseekV2ForCausalLM", model_type="deepseek_v2",
                       hidden_size=2048, num_layers=27, num_heads=16, num_kv_heads=16, head_dim=192,
                       intermediate_size=10944, vocab_size=102400, rms_norm_eps=1e-6,
                       rope_theta=10000.0, max_position_embeddings=163840, rope_neox=False,
                       num_experts=64, num_experts_per_tok=6, moe_intermediate_size=1408,
                       num_shared_experts=2, first_k_dense=1, scoring_func="softmax",
                       use_mla=True, q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=128,
                       qk_rope_head_dim=64, v_head_dim=128)


def deepseek_v32() -> ModelConfig:
    return ModelConfig(architecture="DeepseekV32ForCausalLM", model_type="deepseek_v32",
                       hidden_size=7168, num_layers=61, num_heads=128, num_kv_heads=128,
                       head_dim=192, intermediate_size=18432, vocab_size=129280, rms_norm_eps=1e-6,
                       rope_theta=10000.0, max_position_embeddings=163840, rope_neox=False,
                       num_experts=256, num_experts_per_tok=8, moe_intermediate_size=2048,
                       num_shared_experts=1, first_k_dense=3, scoring_func="sigmoid",
                       norm_topk_prob=True, routed_scaling_factor=2.5, n_group=8, topk_group=4,
                       router_bias=True, use_mla=True, q_lora_rank=1536, kv_lora_rank=512,
                       qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, index_topk=2048,
                       index_n_heads=64, index_head_dim=128, num_nextn_predict_layers=1,
                       quant_method="fp8")


PRESETS = {"tiny-llama": tiny_llama, "llama-3-8b": llama3_8b, "qwen3-30b-a3b": qwen3_30b_a3b,
           "deepseek-v2-lite": deepseek_v2_lite, "deepseek-v3.2": deepseek_v32}


@dataclass
class CacheConfig:
    block_size: int = 16
    gpu_memory_utilization: float = 0.9
    num_gpu_blocks: Optional[int] = None      # override of the profiled value
    enable_prefix_caching: bool = False
    cache_dtype: str = "auto"


@dataclass
class ParallelConfig:
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    data_parallel_size: int = 1
    enable_expert_parallel: bool = False
    decode_context_parallel_size: int = 1
    # prefill context parallelism: the tokens of a prefill step are split over this many ranks (each
    # with its own tensor-parallel group); every layer gathers the step's keys and values, so all
    # ranks hold the whole KV cache and decode steps run replicated
    prefill_context_parallel_size: int = 1
    # keep the residual stream sharded by tokens inside the tensor-parallel group
    # (reduce-scatter / all-gather around every block instead of all-reduce)
    sequence_parallel_residual: bool = False
    # expert-parallel load balancing: spare expert slots that hold copies of the hottest experts, and
    # how often (engine steps, 0 = never) the placement is re-planned from the measured load
    num_redundant_experts: int = 0
    eplb_step_interval: int = 0
    # per-layer overrides: {"layer name suffix": {"tp_size_or_ranks": ..., "x_transform": ..., ...}}
    layer_parallel_config: Dict[str, Any] = field(default_factory=dict)

    @property
    def world_size(self) -> int:
        return (self.tensor_parallel_size * self.pipeline_parallel_size * self.data_parallel_size
                * self.prefill_context_parallel_size)


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 128
    max_num_batched_tokens: int = 8192
    max_model_len: int = 8192
    enable_chunked_prefill: bool = True
    # requests that are decoding take their next token inside the prefill steps of others (one row
    # each, counted against max_num_batched_tokens first) instead of waiting for the prompts to finish
    enable_mixed_batches: bool = False
    policy: str = "fcfs"          # "fcfs" | "priority" (SamplingParams.priority: lower first, preempted last)
    # cache slots kept allocated past the tokens a step feeds (a draft head that runs a chain of
    # k steps writes its keys for k - 1 positions that are scheduled only in the next step)
    num_lookahead_tokens: int = 0


@dataclass
class CompilationConfig:
    """CUDA-graph policy.  ``cudagraph_mode``: NONE | FULL_DECODE_ONLY."""
    cudagraph_mode: str = "FULL_DECODE_ONLY"
    cudagraph_capture_sizes: Optional[List[int]] = None
    max_capture_size: int = 256

    def capture_sizes(self, max_num_seqs: int) -> List[int]:
        if self.cudagraph_mode == "NONE":
            return []
        if self.cudagraph_capture_sizes:
            return sorted(set(s for s in self.cudagraph_capture_sizes if s <= max(max_num_seqs, 1)))
        sizes, s = [], 1
        top = min(max_num_seqs, self.max_capture_size)
        while s < top:
            sizes.append(s)
            s = s * 2 if s < 8 else s + 8 if s < 64 else s + 16
        sizes.append(top)
        return sorted(set(sizes))


@dataclass
class KVTransferConfig:
    kv_connector: Optional[str] = None        # "P2PKVConnector" (alias "LLMDataDistConnector")
    kv_role: Optional[str] = None             # kv_producer | kv_consumer | kv_both
    kv_rank: int = 0
    kv_parallel_size: int = 1
    kv_ip: str = "127.0.0.1"
    kv_port: int = 14579
    kv_connector_extra_config: Dict[str, Any] = field(default_factory=dict)

    @property
    def is_producer(self) -> bool:
        return self.kv_role in ("kv_producer", "kv_both")

    @property
    def is_consumer(self) -> bool:
        return self.kv_role in ("kv_consumer", "kv_both")


@dataclass
class SpeculativeConfig:
    # who proposes draft tokens: "ngram" (prompt lookup, any model), "mtp" / "deepseek_mtp"
    # (the model's multi-token-prediction head); None = no speculation
    method: Optional[str] = None
    num_speculative_tokens: int = 0           # drafts per request and step
    prompt_lookup_max: int = 4
    prompt_lookup_min: int = 2


@dataclass
class EngineConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    cache: CacheConfig = field(default_factory=CacheConfig)
    parallel: ParallelConfig = field(default_factory=ParallelConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    compilation: CompilationConfig = field(default_factory=CompilationConfig)
    kv_transfer: Optional[KVTransferConfig] = None
    speculative: SpeculativeConfig = field(default_factory=SpeculativeConfig)
    model_path: Optional[str] = None          # HF directory with safetensors; None = random init
    load_format: str = "auto"                 # auto | dummy
    seed: int = 0
    device: str = "auto"                      # auto | cuda | cpu
    enforce_eager: bool = False
    enable_sleep_mode: bool = False
    additional_config: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        ac = self.additional_config
        self.use_rejection_sampler = bool(ac.get("use_rejection_sampler", False))
        self.use_penalty = bool(ac.get("use_penalty", True))
        self.async_pull_kv = bool(ac.get("async_pull_kv", False))
        self.enable_kv_rmsnorm_rope_cache = bool(ac.get("enable_kv_rmsnorm_rope_cache", True))
        self.fused_collectives = bool(ac.get("fused_collectives", True))
        if self.scheduler.max_model_len > self.model.max_position_embeddings:
            self.scheduler.max_model_len = self.model.max_position_embeddings
        if self.enforce_eager:
            self.compilation.cudagraph_mode = "NONE"
        if self.parallel.prefill_context_parallel_size > 1:
            if (self.parallel.pipeline_parallel_size > 1 or self.parallel.data_parallel_size > 1
                    or self.parallel.decode_context_parallel_size > 1 or self.parallel.sequence_parallel_residual):
                raise ValueError("prefill context parallelism combines with tensor and expert parallelism only")
            if self.speculative.method and self.speculative.num_speculative_tokens > 0:
                raise ValueError("speculative decoding is not supported with prefill_context_parallel_size > 1")
            if self.kv_transfer is not None:
                raise ValueError("KV transfer connectors are not supported with prefill_context_parallel_size > 1")
        if self.parallel.pipeline_parallel_size > 1:
            # stages exchange (hidden, residual) with point-to-point sends; the draft paths would
            # need the last stage's hidden states on every stage
            if self.speculative.method and self.speculative.num_speculative_tokens > 0:
                raise ValueError("speculative decoding is not supported with pipeline_parallel_size > 1")
            if self.kv_transfer is not None:
                raise ValueError("KV transfer connectors are not supported with pipeline_parallel_size > 1")

    def resolved_device(self) -> torch.device:
        if self.device == "cpu":
            return torch.device("cpu")
        if self.device in ("cuda", "auto") and torch.cuda.is_available():
            return torch.device("cuda", torch.cuda.current_device())
        if self.device == "cuda":
            raise RuntimeError("device='cuda' requested but no CUDA device is visible")
        return torch.device("cpu")

    def replace(self, **kw) -> "EngineConfig":
        return dataclasses.replace(self, **kw)
