"""DeepSeek sparse attention (DSA): lightning indexer + sparse MLA.

For every query token the indexer scores all cached tokens with a small
multi-head dot product,

    score_j = sum_h  w_h * relu(q_h . k_j),      h = 1..index_n_heads, dim index_head_dim

keeps the ``index_topk`` best positions (causal), and the main attention then
runs the absorbed MLA kernel over just those rows of the latent cache.  The
indexer keeps its own paged cache of 128-wide keys next to the latent cache.

Counterpart of ``Indexer`` and ``NPUDeepseekSparseAttention``
(omni_npu/v1/layers/attention/npu_dsa.py:37-142, :370-586) and of the DSA
backend's cache split 512 + 64 + 128 (omni_npu/attention/backends/dsa.py:57-73).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..layers.linear import ReplicatedLinear
from ..layers.norm import LayerNorm
from ..layers.rope import get_rope
from .metadata import AttentionMetadata, get_forward_context
from .mla import MLAAttention, kv_slots_for_sequences


class DSABackend:
    name = "B200_DSA"

    @staticmethod
    def get_name() -> str:
        return DSABackend.name

    @staticmethod
    def get_kv_cache_shape(num_blocks, block_size, kv_lora_rank, rope_dim, index_dim):
        return ((num_blocks, block_size, kv_lora_rank + rope_dim), (num_blocks, block_size, index_dim))


def indexer_topk_reference(q: torch.Tensor, w: torch.Tensor, keys: torch.Tensor, q_pos: torch.Tensor,
                           topk: int) -> torch.Tensor:
    """q [T,Hi,D], w [T,Hi], keys [L,D] (one sequence), q_pos [T] absolute positions.
    Returns int32 [T, topk] key positions, -1 padded, causal (key <= q_pos)."""
    logits = torch.einsum("thd,ld->thl", q.float(), keys.float()).relu_()
    score = (logits * w.float().unsqueeze(-1)).sum(1)                      # [T, L]
    l = keys.shape[0]
    mask = torch.arange(l, device=q.device).unsqueeze(0) > q_pos.unsqueeze(1)
    score = score.masked_fill(mask, float("-inf"))
    k = min(topk, l)
    vals, idx = score.topk(k, dim=-1)
    idx = torch.where(torch.isinf(vals), torch.full_like(idx, -1), idx)
    if k < topk:
        idx = torch.cat([idx, idx.new_full((idx.shape[0], topk - k), -1)], dim=1)
    return idx.to(torch.int32)


class Indexer(nn.Module):
    def __init__(self, cfg, layer_idx: int, device, prefix: str) -> None:
        super().__init__()
        self.layer_idx = layer_idx
        self.n_heads, self.head_dim, self.topk = cfg.index_n_heads, cfg.index_head_dim, cfg.index_topk
        self.rope_dim = cfg.qk_rope_head_dim
        dt = cfg.dtype
        q_in = cfg.q_lora_rank or cfg.hidden_size
        self.wq_b = ReplicatedLinear(q_in, self.n_heads * self.head_dim, dtype=dt, device=device,
                                     prefix=f"{prefix}.wq_b")
        self.wk = ReplicatedLinear(cfg.hidden_size, self.head_dim, dtype=dt, device=device, prefix=f"{prefix}.wk")
        self.k_norm = LayerNorm(self.head_dim, 1e-6, torch.float32, device)
        self.weights_proj = ReplicatedLinear(cfg.hidden_size, self.n_heads, dtype=dt, device=device,
                                             prefix=f"{prefix}.weights_proj")
        self.rotary = get_rope(self.rope_dim, self.rope_dim, cfg.max_position_embeddings, cfg.rope_theta,
                               True, cfg.rope_scaling, device)
        self.softmax_scale = self.head_dim ** -0.5

    def forward(self, hidden: torch.Tensor, q_latent: torch.Tensor, md: AttentionMetadata,
                index_cache: torch.Tensor) -> torch.Tensor:
        """Returns top-k key positions int32 [T, topk] (-1 = none)."""
        t = hidden.shape[0]
        q = self.wq_b(q_latent).view(t, self.n_heads, self.head_dim)
        k = self.k_norm(self.wk(hidden)).to(hidden.dtype)
        # RoPE on the leading rope_dim dims of q and k
        q_pe = q[:, :, : self.rope_dim].reshape(t, self.n_heads * self.rope_dim).contiguous()
        k_pe = k[:, : self.rope_dim].contiguous()
        ops.rope_qk_(q_pe, k_pe, md.positions, self.rotary.cos_sin_cache, self.rope_dim, self.rope_dim, True)
        q = torch.cat([q_pe.view(t, self.n_heads, self.rope_dim), q[:, :, self.rope_dim:]], dim=-1)
        k = torch.cat([k_pe, k[:, self.rope_dim:]], dim=-1).contiguous()
        pc = md.extra.get("pcp") if md.is_prefill else None
        if pc is not None:
            # prefill context parallelism: the index keys of the whole step go into the local cache
            if t < pc["pad"]:
                k = torch.cat([k, k.new_zeros(pc["pad"] - t, k.shape[1])])
            ops.paged_scatter_rows(index_cache, pc["group"].all_gather(k, dim=0).index_select(0, pc["gather_idx"]),
                                   pc["slot_all"])
        else:
            ops.paged_scatter_rows(index_cache, k, md.slot_mapping)
        w = self.weights_proj(hidden).float() * (self.n_heads ** -0.5) * self.softmax_scale
        return self._topk(q, w, md, index_cache)

    def _topk(self, q, w, md: AttentionMetadata, index_cache) -> torch.Tensor:
        """Scores on the tensor cores and a radix select per query token (one score kernel and one
        select kernel for the whole batch, no host synchronisation, so the step stays graph
        capturable).  Index shapes the kernel does not cover (head dim != 128, heads not a
        multiple of 16, pages that do not tile 128 keys) take the dense torch path below."""
        bs = index_cache.shape[1]
        kernel_ok = (not q.is_cuda) or (self.head_dim == 128 and self.n_heads % 16 == 0 and self.n_heads <= 256 and
                                        bs % 8 == 0 and (bs % 128 == 0 if bs >= 128 else 128 % bs == 0))
        if not kernel_ok:
            return self._topk_dense(q, w, md, index_cache)
        if md.is_prefill:
            return ops.dsa_indexer_topk(q, w, index_cache, md.block_tables, md.positions, md.num_seqs, self.topk,
                                        cu_q=md.cu_q, max_ctx=int(md.max_seq_len or 0), max_q=int(md.max_q_len or 0))
        q_len = max(1, md.q_len)
        return ops.dsa_indexer_topk(q, w, index_cache, md.block_tables, md.positions, md.num_seqs, self.topk,
                                    q_len=q_len, max_ctx=int(md.max_seq_len or 0), max_q=q_len)

    def _topk_dense(self, q, w, md: AttentionMetadata, index_cache) -> torch.Tensor:
        """Per-sequence dense scores + ``torch.topk``.  Decode steps touch no host value (a fixed
        window over the whole block table, keys beyond a token's position masked), so they can
        be captured in a CUDA graph; prefill steps read the lengths on the host."""
        bs = index_cache.shape[1]
        t = q.shape[0]
        out = torch.full((t, self.topk), -1, dtype=torch.int32, device=q.device)
        flat = index_cache.view(-1, index_cache.shape[-1])
        if md.is_prefill:
            cu = md.cu_q[: md.num_seqs + 1].tolist()
            lens = md.seq_lens[: md.num_seqs].tolist()
        else:
            cu = [i * md.q_len for i in range(md.num_seqs + 1)]
            lens = None
        for b in range(md.num_seqs):
            qs, qe = cu[b], cu[b + 1]
            if qe <= qs:
                continue
            n = lens[b] if lens is not None else md.block_tables.shape[1] * bs
            pos = torch.arange(n, device=q.device)
            rows = md.block_tables[b][pos // bs].long() * bs + pos % bs
            out[qs:qe] = indexer_topk_reference(q[qs:qe], w[qs:qe], flat[rows], md.positions[qs:qe].long(), self.topk)
        return out


class SparseMLAAttention(MLAAttention):
    """MLA whose keys are restricted to the indexer's top-k selection."""

    def __init__(self, cfg, layer_idx: int, device, prefix: str, quant_factory=None) -> None:
        super().__init__(cfg, layer_idx, device, prefix, quant_factory)
        self.indexer = Indexer(cfg, layer_idx, device, f"{prefix}.indexer")

    def forward(self, hidden: torch.Tensor, reduce: bool = True, topk_indices=None) -> torch.Tensor:
        ctx = get_forward_context()
        md: AttentionMetadata = ctx.attn_metadata
        lat_cache, idx_cache = ctx.kv_caches[self.layer_idx]
        q_latent = self.q_a_layernorm(self.q_a_proj(hidden)) if self.q_lora_rank else hidden
        sel = self.indexer(hidden, q_latent, md, idx_cache)
        return super().forward(hidden, reduce=reduce, topk_indices=sel)
