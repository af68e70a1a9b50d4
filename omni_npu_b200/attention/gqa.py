"""Grouped-query attention backend over the paged KV cache.

Counterpart of ``NPUAttentionBackend`` (omni_npu/attention/backends/attention.py:114-281):
KV cache shape, metadata handling and the forward that first stores this
step's keys/values (fused with RoPE) and then runs one paged attention call.
Different K and V head sizes are allowed (needed by Pangu Pro MoE).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import ops
from .metadata import AttentionMetadata, get_forward_context


class GQABackend:
    name = "B200_GQA"

    @staticmethod
    def get_name() -> str:
        return GQABackend.name

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                           head_size_v: Optional[int] = None) -> Tuple[Tuple[int, ...], Tuple[int, ...]]:
        hv = head_size_v or head_size
        return ((num_blocks, num_kv_heads, block_size, head_size),
                (num_blocks, num_kv_heads, block_size, hv))

    @staticmethod
    def allocate_kv_cache(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                          dtype: torch.dtype, device: torch.device,
                          head_size_v: Optional[int] = None):
        ks, vs = GQABackend.get_kv_cache_shape(num_blocks, block_size, num_kv_heads, head_size, head_size_v)
        return (torch.zeros(ks, dtype=dtype, device=device), torch.zeros(vs, dtype=dtype, device=device))

    @staticmethod
    def bytes_per_block(block_size: int, num_kv_heads: int, head_size: int, dtype: torch.dtype,
                        head_size_v: Optional[int] = None) -> int:
        hv = head_size_v or head_size
        return block_size * num_kv_heads * (head_size + hv) * dtype.itemsize


class GQAAttention(torch.nn.Module):
    """One layer's attention: RoPE + cache write + paged attention."""

    # gathers the step's keys / values when the step is split over prefill-context-parallel ranks
    supports_prefill_context_parallel = True

    def __init__(self, layer_idx: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 scale: float, rot_dim: int, neox: bool = True, sliding_window: int = 0,
                 head_dim_v: Optional[int] = None) -> None:
        super().__init__()
        self.layer_idx = layer_idx
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.head_dim_v = head_dim_v or head_dim
        self.scale = scale
        self.rot_dim = rot_dim
        self.neox = neox
        self.window = sliding_window

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                cos_sin: Optional[torch.Tensor], apply_rope: bool = True) -> torch.Tensor:
        """q [T, Hq*D], k [T, Hk*D], v [T, Hk*Dv] (views into the fused QKV
        projection are fine).  Returns [T, Hq*Dv]."""
        ctx = get_forward_context()
        md: AttentionMetadata = ctx.attn_metadata
        k_cache, v_cache = ctx.kv_caches[self.layer_idx]
        pc = md.extra.get("pcp") if md.is_prefill else None
        if pc is not None:
            # prefill context parallelism: this rank holds the query rows of its token shard; the
            # keys and values of the whole step are gathered, rotated with their own positions and
            # written into the local cache, then the shard attends causally over the cache
            t = q.shape[0]
            pad = pc["pad"]

            def gathered(x):
                x = x.contiguous()
                if t < pad:
                    x = torch.cat([x, x.new_zeros(pad - t, x.shape[1])])
                return pc["group"].all_gather(x, dim=0).index_select(0, pc["gather_idx"])

            k_all, v_all = gathered(k), gathered(v)
            if apply_rope and cos_sin is not None:
                ops.rope_qk_(q, q.new_empty(t, 0), md.positions, cos_sin, self.head_dim, self.rot_dim, self.neox)
                ops.rope_qk_(k_all, k_all.new_empty(k_all.shape[0], 0), pc["positions_all"], cos_sin, self.head_dim,
                             self.rot_dim, self.neox)
            ops.gqa_cache_write(k_all, v_all, k_cache, v_cache, pc["slot_all"])
            return ops.gqa_prefill(q, k_cache, v_cache, md.block_tables, md.cu_q, md.seq_lens,
                                   md.num_seqs, md.max_q_len, self.num_heads, self.scale, True, self.window)
        if apply_rope and cos_sin is not None and md.positions.dim() == 1:
            ops.rope_cache_gqa_(q, k, v, k_cache, v_cache, md.positions, md.slot_mapping, cos_sin,
                                self.head_dim, self.rot_dim, self.neox)
        else:
            ops.gqa_cache_write(k, v, k_cache, v_cache, md.slot_mapping)
        nd = md.extra.get("num_decode_seqs", 0) if md.is_prefill else 0
        if nd:
            # mixed batch: rows [0, nd) are the single new tokens of decoding sequences
            o_dec = ops.gqa_decode(q[:nd], k_cache, v_cache, md.block_tables[:nd], md.seq_lens[:nd], nd,
                                   self.num_heads, self.scale, 1, self.window, max_seq_len=md.max_seq_len)
            o_pre = ops.gqa_prefill(q[nd:], k_cache, v_cache, md.block_tables[nd:], md.extra["cu_q_prefill"],
                                    md.seq_lens[nd:], md.num_seqs - nd, md.extra["max_q_len_prefill"],
                                    self.num_heads, self.scale, True, self.window)
            return torch.cat([o_dec, o_pre], 0)
        if md.is_prefill:
            return ops.gqa_prefill(q, k_cache, v_cache, md.block_tables, md.cu_q, md.seq_lens,
                                   md.num_seqs, md.max_q_len, self.num_heads, self.scale, True,
                                   self.window)
        return ops.gqa_decode(q, k_cache, v_cache, md.block_tables, md.seq_lens, md.num_seqs,
                              self.num_heads, self.scale, md.q_len, self.window,
                              max_seq_len=md.max_seq_len)
