"""Multi-head latent attention (DeepSeek V2 / V3 family) over a paged latent cache.

Cache row per token: ``[RMSNorm(c_kv) (kv_lora_rank) | RoPE(k_pe) (qk_rope_head_dim)]``
written by one fused kernel.  Two compute paths, as in the reference
(omni_npu/attention/backends/mla.py:452-616 prefill, :695-804 decode;
omni_npu/v1/layers/attention/npu_mla.py:169-348):

* prefill  (non-absorbed): the latent rows of every sequence (cached context
  included, so chunked prefill needs no separate merge pass) are up-projected
  with ``kv_b_proj`` to per-head K (nope|rope, 192) and V (128) and run through
  the variable-length attention kernel.
* decode   (absorbed): q_nope is folded through W_UK into the latent space, one
  MQA pass over the latent cache yields [N, 512] per token, W_UV maps it back.

``MLABackend`` carries the cache-shape bookkeeping the model runner needs.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..layers.linear import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear
from ..layers.norm import RMSNorm
from ..layers.rope import get_rope, yarn_get_mscale
from ..parallel import state as pstate
from .metadata import AttentionMetadata, get_forward_context


class MLABackend:
    name = "B200_MLA"

    @staticmethod
    def get_name() -> str:
        return MLABackend.name

    @staticmethod
    def get_kv_cache_shape(num_blocks: int, block_size: int, kv_lora_rank: int, rope_dim: int):
        return (num_blocks, block_size, kv_lora_rank + rope_dim)

    @staticmethod
    def allocate_kv_cache(num_blocks, block_size, kv_lora_rank, rope_dim, dtype, device):
        return torch.zeros(MLABackend.get_kv_cache_shape(num_blocks, block_size, kv_lora_rank, rope_dim),
                           dtype=dtype, device=device)

    @staticmethod
    def bytes_per_block(block_size, kv_lora_rank, rope_dim, dtype) -> int:
        return block_size * (kv_lora_rank + rope_dim) * dtype.itemsize


def kv_slots_for_sequences(md: AttentionMetadata, block_size: int, total_kv: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """For a prefill step: cache slot of every kv token of every sequence, laid out
    sequence after sequence, plus (seq id, position) of each.  Device-side only."""
    dev = md.seq_lens.device
    lens = md.seq_lens[: md.num_seqs].long()
    seq_id = torch.repeat_interleave(torch.arange(md.num_seqs, device=dev), lens, output_size=total_kv)
    starts = torch.cumsum(lens, 0) - lens
    pos = torch.arange(total_kv, device=dev) - starts[seq_id]
    blk = md.block_tables[seq_id, pos // block_size].long()
    return blk * block_size + pos % block_size, seq_id, pos


class MLAAttention(nn.Module):
    """Attention block of a DeepSeek-style layer: projections, cache write, attention, o_proj."""

    # gathers the step's compressed keys when the step is split over prefill-context-parallel ranks
    supports_prefill_context_parallel = True

    def __init__(self, cfg, layer_idx: int, device, prefix: str, quant_factory=None) -> None:
        super().__init__()
        self.layer_idx = layer_idx
        self.hidden = cfg.hidden_size
        tp = pstate.get_tp_group()
        self.tp_size = tp.world_size
        assert cfg.num_heads % self.tp_size == 0
        self.num_heads = cfg.num_heads // self.tp_size
        self.q_lora_rank, self.kv_lora_rank = cfg.q_lora_rank, cfg.kv_lora_rank
        self.nope, self.rope_dim, self.v_dim = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        self.qk_dim = self.nope + self.rope_dim
        qm = quant_factory or (lambda: None)
        dt = cfg.dtype
        if self.q_lora_rank:
            self.q_a_proj = ReplicatedLinear(self.hidden, self.q_lora_rank, dtype=dt, device=device,
                                             quant_method=qm(), prefix=f"{prefix}.q_a_proj")
            self.q_a_layernorm = RMSNorm(self.q_lora_rank, cfg.rms_norm_eps, dt, device)
            self.q_b_proj = ColumnParallelLinear(self.q_lora_rank, cfg.num_heads * self.qk_dim, dtype=dt,
                                                 device=device, quant_method=qm(), prefix=f"{prefix}.q_b_proj")
        else:
            self.q_proj = ColumnParallelLinear(self.hidden, cfg.num_heads * self.qk_dim, dtype=dt,
                                               device=device, quant_method=qm(), prefix=f"{prefix}.q_proj")
        self.kv_a_proj_with_mqa = ReplicatedLinear(self.hidden, self.kv_lora_rank + self.rope_dim, dtype=dt,
                                                   device=device, quant_method=qm(),
                                                   prefix=f"{prefix}.kv_a_proj_with_mqa")
        self.kv_a_layernorm = RMSNorm(self.kv_lora_rank, cfg.rms_norm_eps, dt, device)
        self.kv_b_proj = ColumnParallelLinear(self.kv_lora_rank, cfg.num_heads * (self.nope + self.v_dim),
                                              dtype=dt, device=device, prefix=f"{prefix}.kv_b_proj")
        self.o_proj = RowParallelLinear(cfg.num_heads * self.v_dim, self.hidden, dtype=dt, device=device,
                                        quant_method=qm(), prefix=f"{prefix}.o_proj")
        self.rotary = get_rope(self.rope_dim, self.rope_dim, cfg.max_position_embeddings, cfg.rope_theta,
                               False, cfg.rope_scaling, device)
        self.scale = self.qk_dim ** -0.5
        rs = cfg.rope_scaling or {}
        if rs.get("rope_type", rs.get("type")) in ("yarn", "deepseek_yarn") and rs.get("mscale_all_dim"):
            m = yarn_get_mscale(rs["factor"], rs["mscale_all_dim"])
            self.scale *= m * m
        # decode context parallelism (the latent cache sharded by tokens over the tensor-parallel group)
        # (set by the decoder layer from ParallelConfig.decode_context_parallel_size)
        self.cp_group = None
        self.w_uk: Optional[torch.Tensor] = None    # [N, 512, 128]: rows = latent dims  (q_nope @ W_UK)
        self.w_uv: Optional[torch.Tensor] = None    # [N, 128, 512]: rows = v dims       (o_lat @ W_UV^T)

    def process_weights_after_loading(self) -> None:
        """Split kv_b_proj into the absorbed-path matrices."""
        w = self.kv_b_proj.weight.data
        if w.dtype == torch.float8_e4m3fn:
            return
        n, l = self.num_heads, self.kv_lora_rank
        w = w.view(n, self.nope + self.v_dim, l)
        # q_lat[n, t, l] = sum_p q_nope[n,t,p] * W[n,p,l]  ->  GEMM weight rows are output dims: [l, p]
        self.w_uk = w[:, : self.nope, :].transpose(1, 2).contiguous()
        # v[n, t, d] = sum_l o_lat[n,t,l] * W[n, nope+d, l] ->  weight rows [d, l]
        self.w_uv = w[:, self.nope:, :].contiguous()

    # ------------------------------------------------------------------ forward
    def _project_q(self, hidden: torch.Tensor) -> torch.Tensor:
        if self.q_lora_rank:
            return self.q_b_proj(self.q_a_layernorm(self.q_a_proj(hidden)))
        return self.q_proj(hidden)

    def forward(self, hidden: torch.Tensor, reduce: bool = True,
                topk_indices: Optional[torch.Tensor] = None) -> torch.Tensor:
        ctx = get_forward_context()
        md: AttentionMetadata = ctx.attn_metadata
        cache = ctx.kv_caches[self.layer_idx]
        cache = cache[0] if isinstance(cache, (tuple, list)) else cache
        t = hidden.shape[0]
        n = self.num_heads
        q = self._project_q(hidden).view(t, n, self.qk_dim)
        kv_a = self.kv_a_proj_with_mqa(hidden)
        pc = md.extra.get("pcp") if md.is_prefill else None
        if pc is not None:
            # prefill context parallelism: this rank holds a token shard of the step; the compressed
            # keys of the WHOLE step are gathered and written into the local cache with their own
            # positions, so the prefill below (which reads every key from the cache) sees the tokens
            # of the other shards that precede its query rows
            x = kv_a.contiguous()
            if t < pc["pad"]:
                x = torch.cat([x, x.new_zeros(pc["pad"] - t, x.shape[1])])
            kv_all = pc["group"].all_gather(x, dim=0).index_select(0, pc["gather_idx"])
            ops.mla_kv_rmsnorm_rope_cache(kv_all[:, : self.kv_lora_rank], kv_all[:, self.kv_lora_rank:],
                                          self.kv_a_layernorm.weight, cache, pc["positions_all"], pc["slot_all"],
                                          self.rotary.cos_sin_cache, self.kv_a_layernorm.eps, False)
        else:
            # fused: RMSNorm(c_kv), RoPE(k_pe), write [c_kv | k_pe] into the paged cache
            ops.mla_kv_rmsnorm_rope_cache(kv_a[:, : self.kv_lora_rank], kv_a[:, self.kv_lora_rank:],
                                          self.kv_a_layernorm.weight, cache, md.positions, md.slot_mapping,
                                          self.rotary.cos_sin_cache, self.kv_a_layernorm.eps, False)
        # RoPE on the rope part of q (k_pe is handled by the cache kernel)
        q_pe = q[:, :, self.nope:].reshape(t, n * self.rope_dim).contiguous()
        dummy_k = q_pe.new_empty(t, 0)
        ops.rope_qk_(q_pe, dummy_k, md.positions, self.rotary.cos_sin_cache, self.rope_dim, self.rope_dim, False)
        q_pe = q_pe.view(t, n, self.rope_dim)
        nd = md.extra.get("num_decode_seqs", 0) if md.is_prefill and topk_indices is None else 0
        if nd and "md_decode" in md.extra:
            # mixed batch: rows [0, nd) are the single new tokens of decoding sequences: they take the
            # absorbed latent-space path, the prompt rows behind them the non-absorbed prefill
            o = torch.cat([self._decode(q[:nd], q_pe[:nd], cache, md.extra["md_decode"], None),
                           self._prefill(q[nd:], q_pe[nd:], cache, md.extra["md_prefill"])], 0)
        elif md.is_prefill and topk_indices is None:
            o = self._prefill(q, q_pe, cache, md)
        else:
            o = self._decode(q, q_pe, cache, md, topk_indices)
        return self.o_proj(o, reduce=reduce)

    def _prefill(self, q, q_pe, cache, md: AttentionMetadata) -> torch.Tensor:
        """Non-absorbed attention of this step's queries over every key of their sequences (cached
        context included).  The latent blocks of the sequences are gathered block-wise, up-projected
        with ``kv_b_proj`` and handed to the variable-length kernel as a temporary paged K / V whose
        block table is the identity; lengths and block counts come from the host copy of the step
        (no device-to-host read).  With decode context parallelism every rank gathers its token
        shard of the same blocks, the shards are all-gathered, and (block, offset, rank) read in
        that order IS the global token order, so the gathered tensor is the same paged latent with
        ``block_size * world`` tokens per block
        (reference: prefill omni_npu/attention/backends/mla.py:452-616, context gather under
        context parallelism :317-375)."""
        t, n = q.shape[0], self.num_heads
        bs = cache.shape[1]
        dev = q.device
        lens_h = md.extra.get("seq_lens_host")
        if lens_h is None:                   # a caller outside the model runner: one host read
            lens_h = md.seq_lens[: md.num_seqs].tolist()
        cp = self.cp_group
        w = cp.world_size if cp is not None else 1
        gbs = bs * w                                            # tokens per block id
        nblk = [(int(l) + gbs - 1) // gbs for l in lens_h]
        max_blocks = max(1, max(nblk))
        total_blocks = sum(nblk)
        seq_of_blk = [i for i, c in enumerate(nblk) for _ in range(c)]
        j_of_blk = [j for c in nblk for j in range(c)]
        starts, acc = [], 0
        for c in nblk:
            starts.append(acc)
            acc += c
        idx = torch.tensor([seq_of_blk, j_of_blk], dtype=torch.long).to(dev, non_blocking=True)
        blk_ids = md.block_tables[idx[0], idx[1]].long()
        lat = cache.index_select(0, blk_ids)                                     # [blocks, bs, 576]
        if w > 1:
            lat = cp.all_gather(lat.unsqueeze(2).contiguous(), dim=2)            # [blocks, bs, w, 576]
            lat = lat.reshape(total_blocks, gbs, lat.shape[-1])
        l = self.kv_lora_rank
        kv = self.kv_b_proj(lat[..., :l].reshape(total_blocks * gbs, l).contiguous())
        kv = kv.view(total_blocks, gbs, n, self.nope + self.v_dim)
        k_pe = lat[..., l:].unsqueeze(2).expand(total_blocks, gbs, n, self.rope_dim)
        k_paged = torch.cat([kv[..., : self.nope], k_pe], dim=-1).permute(0, 2, 1, 3).contiguous()
        v_paged = kv[..., self.nope:].permute(0, 2, 1, 3).contiguous()
        bt = torch.tensor([[s0 + min(j, max(c - 1, 0)) for j in range(max_blocks)] for s0, c in zip(starts, nblk)],
                          dtype=torch.int32).to(dev, non_blocking=True)
        qf = torch.cat([q[:, :, : self.nope], q_pe], dim=-1).reshape(t, n * self.qk_dim)
        return ops.gqa_prefill(qf, k_paged, v_paged, bt, md.cu_q, md.seq_lens, md.num_seqs, md.max_q_len, n,
                               self.scale, True, 0)

    def _absorb_q(self, q, q_pe):
        """q_lat[h] = q_nope[h] @ W_UK[h] (heads act as the groups of a grouped GEMM); returns the
        [t, n * 576] query of the latent-space kernel and the group offsets."""
        t, n, l = q.shape[0], self.num_heads, self.kv_lora_rank
        if self.w_uk is None:
            self.process_weights_after_loading()
        q_nope = q[:, :, : self.nope].transpose(0, 1).reshape(n * t, self.nope).contiguous()
        offs = torch.arange(0, (n + 1) * t, t, dtype=torch.int32, device=q.device)
        q_lat = ops.grouped_gemm(q_nope, self.w_uk, offs).view(n, t, l).transpose(0, 1)
        qf = torch.cat([q_lat, q_pe], dim=-1).reshape(t, n * (l + self.rope_dim)).contiguous()
        return qf, offs

    def _unabsorb_o(self, o_lat, offs):
        """v[h] = o_lat[h] @ W_UV[h]^T -> [t, n * v_dim]."""
        t, n, l = o_lat.shape[0], self.num_heads, self.kv_lora_rank
        o_lat = o_lat.view(t, n, l).transpose(0, 1).reshape(n * t, l).contiguous()
        o = ops.grouped_gemm(o_lat, self.w_uv, offs).view(n, t, self.v_dim).transpose(0, 1)
        return o.reshape(t, n * self.v_dim).contiguous()

    @staticmethod
    def _rows_per_token(md: AttentionMetadata, t: int, device):
        """Block table and causal length for every query token taken as a one-token sequence
        (prefill steps through the latent-space kernel, per-token key selections)."""
        if md.is_prefill:
            seq_of_tok = torch.repeat_interleave(torch.arange(md.num_seqs, device=device),
                                                 (md.cu_q[1: md.num_seqs + 1] - md.cu_q[: md.num_seqs]).long(),
                                                 output_size=t)
        else:
            seq_of_tok = torch.arange(md.num_seqs, device=device).repeat_interleave(md.q_len)
        return seq_of_tok

    def _decode(self, q, q_pe, cache, md: AttentionMetadata, topk_indices) -> torch.Tensor:
        t, n = q.shape[0], self.num_heads
        qf, offs = self._absorb_q(q, q_pe)
        if md.is_prefill:
            # sparse prefill: every query token is its own "sequence" row for the kernel
            seq_of_tok = self._rows_per_token(md, t, q.device)
            bt = md.block_tables[seq_of_tok]
            sl = md.seq_lens[seq_of_tok]
            o_lat = ops.mla_decode(qf, cache, bt.contiguous(), sl.contiguous(), t, n, self.scale, 1, topk_indices)
        elif self.cp_group is not None:
            # the cache holds this rank's token shard: attention of all heads over it, then the
            # partial results are exchanged by head and merged by their log-sum-exp
            if topk_indices is not None or md.q_len != 1:
                raise NotImplementedError("decode context parallelism: plain one-token decode steps only")
            from .dcp import dcp_mla_decode
            o_lat = dcp_mla_decode(qf, cache, md.block_tables, md.seq_lens, md.num_seqs, n, self.scale,
                                   self.cp_group)
        else:
            o_lat = ops.mla_decode(qf, cache, md.block_tables, md.seq_lens, md.num_seqs, n, self.scale, md.q_len,
                                   topk_indices, max_seq_len=md.max_seq_len)
        return self._unabsorb_o(o_lat, offs)


class StaticSinkMLAAttention(MLAAttention):
    """Latent attention with learned static sink tokens and an optional sliding window.

    ``sink_len`` learned (latent | rope-key) rows are visible to every query of every sequence;
    real keys are limited to the last ``sliding_window`` positions (0 = all).  Both prefill and
    decode run in the latent space as two partial attentions over disjoint key sets, merged by
    their log-sum-exp:

    * the window: the sparse mode of the latent-cache kernel with per-token indices
      ``pos - W + 1 .. pos`` (holes before the sequence start), so a long context costs W keys
      per token and the cache needs no sink blocks;
    * the sinks: one small GEMM of the absorbed queries against the ``sink_len`` x 576 table.

    The sink rows go through the KV norm once after loading; their rope part is used as stored
    (position-free).  Counterpart of the sink / sliding-window branches of the reference's MLA
    backend (omni_npu/attention/backends/mla.py:495-560,724-760: two attention calls + LSE
    update) and of ``StaticSinkMLAAttention`` / ``update_sink_kv``
    (omni_npu/vllm_patches/patches/models/pangu_sink_swa_mla/patch_static_sink_attention.py:257-349,
    patch_mla.py:18-78)."""

    supports_prefill_context_parallel = False     # the sink / window composition reads per-token rows it built itself

    def __init__(self, cfg, layer_idx: int, device, prefix: str, quant_factory=None,
                 sink_len: int = 0, sliding_window: int = 0) -> None:
        super().__init__(cfg, layer_idx, device, prefix, quant_factory)
        self.sink_len, self.window = int(sink_len), int(sliding_window or 0)
        if self.sink_len:
            self.param_sink_kv = nn.Parameter(torch.zeros(self.sink_len, self.kv_lora_rank + self.rope_dim,
                                                          dtype=cfg.dtype, device=device), requires_grad=False)
        self.sink_latent: Optional[torch.Tensor] = None     # [sink_len, 576] normed latent | rope key

    def process_weights_after_loading(self) -> None:
        super().process_weights_after_loading()
        if self.sink_len:
            raw = self.param_sink_kv.data
            l = self.kv_lora_rank
            self.sink_latent = torch.cat([self.kv_a_layernorm(raw[:, :l].contiguous()), raw[:, l:]], dim=-1)

    def update_sink_kv(self, sink_k_pe: torch.Tensor, sink_compressed_kv: torch.Tensor) -> None:
        """Install sink rows prepared by the caller (already normed / rotated as it wants them)."""
        self.sink_latent = torch.cat([sink_compressed_kv, sink_k_pe], dim=-1).to(self.kv_b_proj.weight.device)
        self.sink_len = self.sink_latent.shape[0]

    def _prefill(self, q, q_pe, cache, md: AttentionMetadata) -> torch.Tensor:
        return self._sink_window(q, q_pe, cache, md)

    def _decode(self, q, q_pe, cache, md: AttentionMetadata, topk_indices) -> torch.Tensor:
        if topk_indices is not None:
            raise NotImplementedError("static sinks are not combined with indexer-selected keys")
        return self._sink_window(q, q_pe, cache, md)

    def _sink_window(self, q, q_pe, cache, md: AttentionMetadata) -> torch.Tensor:
        t, n, l = q.shape[0], self.num_heads, self.kv_lora_rank
        qf, offs = self._absorb_q(q, q_pe)
        pos = md.positions.reshape(-1)[:t].to(torch.int32)
        seq_of_tok = self._rows_per_token(md, t, q.device)
        bt = md.block_tables[seq_of_tok].contiguous()
        sl = (pos + 1).contiguous()                     # causal length of each token's own row
        idx = None
        if self.window:
            w = self.window
            idx = pos.unsqueeze(1) - (w - 1) + torch.arange(w, dtype=torch.int32, device=q.device).unsqueeze(0)
            idx = torch.where(idx < 0, torch.full_like(idx, -1), idx).contiguous()
        o_win, lse_win = ops.mla_decode(qf, cache, bt, sl, t, n, self.scale, 1, idx,
                                        max_seq_len=md.max_seq_len, return_lse=True)
        if not self.sink_len:
            return self._unabsorb_o(o_win, offs)
        if self.sink_latent is None:
            self.process_weights_after_loading()
        sink = self.sink_latent.to(qf.dtype)                                              # [S, 576]
        sc = (qf.view(t * n, l + self.rope_dim) @ sink.t()).float() * self.scale          # [t*n, S]
        lse_s = torch.logsumexp(sc, dim=-1).view(t, n)
        o_s = (torch.softmax(sc, dim=-1).to(qf.dtype) @ sink[:, :l]).view(t, n, l)
        o_lat, _ = ops.merge_attn_states(torch.stack([o_win.view(t, n, l), o_s]),
                                         torch.stack([lse_win.view(t, n).float(), lse_s]))
        return self._unabsorb_o(o_lat.reshape(t, n * l).to(qf.dtype), offs)
