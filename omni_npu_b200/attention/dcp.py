"""Decode context parallelism for multi-head latent attention.

With plain tensor parallelism every rank keeps the whole latent KV cache (MLA has one
shared KV "head") and only the query heads are split.  Decode context parallelism splits
the *tokens* of the cache across the ranks instead: token ``p`` of a sequence lives on rank
``p % world`` (interleave 1) at local position ``p // world``, so every rank stores and
streams ``1 / world`` of the context.  A decode step then is

  1. all-gather the queries of all heads,
  2. local absorbed attention of ALL heads over the local token shard, with its
     log-sum-exp,
  3. all-to-all: head chunk j of (output, lse) goes to rank j,
  4. N-way log-sum-exp merge of the partials of this rank's heads.

Same scheme as the reference's MLA backend (slot selection
omni_npu/attention/backends/mla.py:174-180; decode path :618-700; merge
omni_npu/attention/ops.py:109-141).
"""
from __future__ import annotations

from typing import Tuple

import torch

from .. import ops


def local_seq_lens(seq_lens: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """How many of the first ``seq_len`` tokens live on ``rank`` (tokens rank, rank + world, ...)."""
    return torch.clamp((seq_lens - rank + world - 1) // world, min=0).to(seq_lens.dtype)


def local_slot_mapping(positions: torch.Tensor, slot_mapping: torch.Tensor, block_tables_of_token: torch.Tensor,
                       block_size: int, world: int, rank: int) -> torch.Tensor:
    """Slot of each new token in the LOCAL cache, -1 for tokens owned by another rank.
    ``block_tables_of_token`` [T, max_blocks] is the block-table row of the token's sequence."""
    mine = (positions % world) == rank
    lp = (positions // world).long()
    blk = block_tables_of_token.gather(1, (lp // block_size).unsqueeze(1)).squeeze(1).long()
    slot = blk * block_size + lp % block_size
    return torch.where(mine, slot, torch.full_like(slot, -1)).to(slot_mapping.dtype)


def dcp_mla_decode(q_local: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor,
                   num_seqs: int, heads_local: int, scale: float, group) -> torch.Tensor:
    """q_local [T, heads_local*576] (this rank's heads), cache: this rank's token shard,
    ``seq_lens``: GLOBAL lengths.  Returns [T, heads_local*512]."""
    world, rank = group.world_size, group.rank_in_group
    if world == 1:
        return ops.mla_decode(q_local, cache, block_tables, seq_lens, num_seqs, heads_local, scale)
    t = q_local.shape[0]
    q_all = group.all_gather(q_local.view(t, heads_local, 576), dim=1)               # [T, H, 576]
    h = heads_local * world
    lens = local_seq_lens(seq_lens, world, rank)
    out, lse = ops.mla_decode(q_all.reshape(t, h * 576).contiguous(), cache, block_tables, lens, num_seqs, h, scale,
                              return_lse=True)
    out = out.view(t, world, heads_local, 512)
    lse = lse.view(t, world, heads_local)
    # head chunk j goes to rank j; what comes back are the world partials of my heads
    packed = torch.cat([out.float(), lse.unsqueeze(-1).float()], dim=-1)              # [T, W, hl, 513]
    send = packed.permute(1, 0, 2, 3).contiguous()                                   # [W, T, hl, 513]
    recv = group.all_to_all_single(send.view(world * t, heads_local * 513)).view(world, t, heads_local, 513)
    outs = recv[..., :512].to(q_local.dtype).contiguous()
    lses = recv[..., 512].contiguous()
    merged, _ = ops.merge_attn_states(outs, lses)
    return merged.reshape(t, heads_local * 512)
