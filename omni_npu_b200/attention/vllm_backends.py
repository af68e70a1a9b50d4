"""Attention backends in vLLM's v1 backend interface.

``B200AttentionBackend`` (name ``B200_ATTN``) serves grouped-query attention of stock vLLM
models with this package's paged kernels: the KV cache of a layer is one tensor
``[2, blocks, kv_heads, block_size, head_size]`` (head-major inside a block, so a block of one
head is a contiguous TMA box), the metadata builder keeps vLLM's device tensors (query
offsets, sequence lengths, block table, slot mapping) without any host copy, and the
implementation writes the step's keys / values into the cache and runs the prefill or
decode kernel.  ``B200MLABackend`` (``B200_MLA``) and ``B200DSABackend`` (``B200_DSA``) carry
the names, cache shapes (latent 512 + 64 rope; plus a 128-wide indexer key for sparse
attention) and builders for the MLA model classes of this package, whose attention modules
call the absorbed-MLA kernels directly.

Counterparts: ``NPUAttentionBackend`` (omni_npu/attention/backends/attention.py:53-162),
``NPUMLABackend`` (omni_npu/attention/backends/mla.py:43-180), ``NPUDSABackend``
(omni_npu/attention/backends/dsa.py:42-73).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, List, Optional, Tuple

import torch

from .. import compat, ops

if compat.vllm_available():
    from vllm.v1.attention.backend import AttentionBackend as _Backend
    from vllm.v1.attention.backend import AttentionImpl as _Impl
    from vllm.v1.attention.backend import AttentionMetadataBuilder as _Builder
else:
    class _Backend:  # type: ignore[no-redef]
        pass

    class _Impl:  # type: ignore[no-redef]
        pass

    class _Builder:  # type: ignore[no-redef]
        def __init__(self, kv_cache_spec=None, layer_names=None, vllm_config=None, device=None) -> None:
            self.kv_cache_spec, self.layer_names, self.vllm_config, self.device = \
                kv_cache_spec, layer_names, vllm_config, device


@dataclass
class B200AttentionMetadata:
    num_actual_tokens: int
    num_reqs: int
    max_query_len: int
    max_seq_len: int
    query_start_loc: torch.Tensor      # [num_reqs + 1] int32
    seq_lens: torch.Tensor             # [num_reqs] int32
    block_table: torch.Tensor          # [num_reqs, max_blocks] int32
    slot_mapping: torch.Tensor         # [num_tokens]
    is_decode: bool                    # every request has exactly one query token
    causal: bool = True


class B200AttentionMetadataBuilder(_Builder):
    # decode batches are replayed from CUDA graphs: lengths live in device tensors
    reorder_batch_threshold: ClassVar[int] = 1

    def __init__(self, kv_cache_spec=None, layer_names=None, vllm_config=None, device=None) -> None:
        # vLLM declares the base initialiser abstract: a builder that does not define its own
        # cannot be instantiated
        self.kv_cache_spec, self.layer_names = kv_cache_spec, layer_names
        self.vllm_config, self.device = vllm_config, device

    def build(self, common_prefix_len: int, common_attn_metadata, fast_build: bool = False) -> B200AttentionMetadata:
        m = common_attn_metadata
        n_tok, n_req = int(m.num_actual_tokens), int(m.num_reqs)
        return B200AttentionMetadata(
            num_actual_tokens=n_tok, num_reqs=n_req, max_query_len=int(m.max_query_len),
            max_seq_len=int(m.max_seq_len), query_start_loc=m.query_start_loc.to(torch.int32),
            seq_lens=m.seq_lens.to(torch.int32), block_table=m.block_table_tensor,
            slot_mapping=m.slot_mapping, is_decode=int(m.max_query_len) == 1, causal=bool(getattr(m, "causal", True)))

    def build_for_cudagraph_capture(self, common_attn_metadata) -> B200AttentionMetadata:
        return self.build(0, common_attn_metadata)


class B200AttentionImpl(_Impl):
    def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: Optional[int] = None,
                 alibi_slopes: Optional[List[float]] = None, sliding_window: Optional[int] = None,
                 kv_cache_dtype: str = "auto", logits_soft_cap: Optional[float] = None, attn_type: str = "decoder",
                 kv_sharing_target_layer_name: Optional[str] = None, sinks: Optional[torch.Tensor] = None,
                 **extra) -> None:
        if alibi_slopes is not None or logits_soft_cap:
            raise NotImplementedError("ALiBi and logit soft-capping are not supported by the B200 attention kernels")
        if kv_cache_dtype not in ("auto", "bfloat16"):
            raise NotImplementedError(f"KV cache dtype {kv_cache_dtype!r} is not supported")
        self.num_heads, self.head_size, self.scale = num_heads, head_size, float(scale)
        self.num_kv_heads = num_kv_heads or num_heads
        self.sliding_window = int(sliding_window or 0)
        self.sink_len = int(extra.get("sink_len", 0))
        self.kv_sharing_target_layer_name = kv_sharing_target_layer_name

    def forward(self, layer, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                attn_metadata: Optional[B200AttentionMetadata], output: Optional[torch.Tensor] = None,
                output_scale=None, output_block_scale=None) -> torch.Tensor:
        if attn_metadata is None:                      # memory-profiling run: nothing to attend to
            return output if output is not None else torch.zeros_like(query)
        md = attn_metadata
        n = md.num_actual_tokens
        q = query[:n].reshape(n, -1)
        k_cache, v_cache = kv_cache[0], kv_cache[1]
        if key is not None and self.kv_sharing_target_layer_name is None:
            ops.gqa_cache_write(key[:n].reshape(n, -1), value[:n].reshape(n, -1), k_cache, v_cache,
                                md.slot_mapping[:n].to(torch.int32))
        if md.is_decode:
            o = ops.gqa_decode(q, k_cache, v_cache, md.block_table, md.seq_lens, md.num_reqs, self.num_heads,
                               self.scale, 1, self.sliding_window, max_seq_len=md.max_seq_len, sink=self.sink_len)
        else:
            o = ops.gqa_prefill(q, k_cache, v_cache, md.block_table, md.query_start_loc, md.seq_lens, md.num_reqs,
                                md.max_query_len, self.num_heads, self.scale, md.causal, self.sliding_window,
                                sink=self.sink_len)
        if output is None:
            return o.view(n, self.num_heads * o.shape[-1] // self.num_heads)
        output[:n].reshape(n, -1).copy_(o)
        return output


class B200AttentionBackend(_Backend):
    accept_output_buffer: bool = True
    forward_includes_kv_cache_update: bool = True
    supported_dtypes: ClassVar[list] = [torch.bfloat16]

    @staticmethod
    def get_name() -> str:
        return "B200_ATTN"

    @staticmethod
    def get_impl_cls():
        return B200AttentionImpl

    @staticmethod
    def get_builder_cls():
        return B200AttentionMetadataBuilder

    @staticmethod
    def get_metadata_cls():
        return B200AttentionMetadata

    @staticmethod
    def get_supported_head_sizes() -> List[int]:
        return [64, 128]

    @staticmethod
    def get_supported_kernel_block_sizes() -> List[int]:
        return [16, 32, 64, 128]

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> Tuple[int, ...]:
        return (2, num_blocks, num_kv_heads, block_size, head_size)

    @classmethod
    def supports_sink(cls) -> bool:
        return True


class B200MLABackend(_Backend):
    """Multi-head latent attention: one 576-wide latent row per token (512 compressed KV +
    64 rotary key dims)."""
    accept_output_buffer: bool = True

    @staticmethod
    def get_name() -> str:
        return "B200_MLA"

    @staticmethod
    def get_builder_cls():
        return B200AttentionMetadataBuilder

    @staticmethod
    def get_metadata_cls():
        return B200AttentionMetadata

    @staticmethod
    def get_impl_cls():
        from .mla import MLAAttention
        return MLAAttention

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           cache_dtype_str: str = "auto") -> Tuple[int, ...]:
        return (num_blocks, block_size, head_size)      # head_size = kv_lora_rank + qk_rope_head_dim

    @classmethod
    def is_mla(cls) -> bool:
        return True


class B200DSABackend(B200MLABackend):
    """Sparse MLA: the latent cache plus a 128-wide key cache for the lightning indexer."""

    @staticmethod
    def get_name() -> str:
        return "B200_DSA"

    @staticmethod
    def get_impl_cls():
        from .dsa import SparseMLAAttention
        return SparseMLAAttention

    @staticmethod
    def get_kv_cache_shapes(num_blocks: int, block_size: int, kv_lora_rank: int = 512, rope_dim: int = 64,
                            index_dim: int = 128):
        return ((num_blocks, block_size, kv_lora_rank + rope_dim), (num_blocks, block_size, index_dim))

    @classmethod
    def is_sparse(cls) -> bool:
        return True
