"""Helpers of the KV connectors: option lookup, producer-rank selection and KV
re-sharding between instances with different tensor-parallel sizes."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple


def get_config_from_dict_or_env(cfg: Optional[Dict[str, Any]], key: str, env: str, default: Any = None) -> Any:
    """Option lookup order: explicit dict entry, environment variable, default
    (omni_npu/connector/utils.py:239-255)."""
    if cfg and cfg.get(key) is not None:
        return cfg[key]
    v = os.environ.get(env)
    return v if v is not None else default


def get_p_start_rank(p_tp_size: int, d_tp_size: int, d_rank: int, p_dp_size: int = 1, d_dp_rank: int = 0) -> int:
    """Which producer rank a consumer rank pulls from.

    Equal TP sizes map rank i to rank i.  A consumer with a larger TP degree
    (KV heads split finer, or replicated latent caches) maps several of its ranks
    onto one producer rank; a smaller degree maps each consumer rank to the first
    of the producer ranks that jointly hold its heads (the others are fetched by
    ``TPConvertor``).  (omni_npu/connector/utils.py:182-237)"""
    if p_tp_size == d_tp_size:
        return d_rank
    if d_tp_size > p_tp_size:
        return d_rank * p_tp_size // d_tp_size
    return d_rank * (p_tp_size // d_tp_size)


@dataclass
class ReshardPlan:
    """For one consumer rank: the producer ranks to pull from and, for each, which
    slice of the KV-head dimension of the producer block lands in which slice of
    the consumer block."""
    sources: List[Tuple[int, Tuple[int, int], Tuple[int, int]]]   # (p_rank, (src_lo, src_hi), (dst_lo, dst_hi))


class TPConvertor:
    """KV re-sharding when producer and consumer use different TP degrees.

    KV heads are split evenly over TP ranks (MLA latent caches are replicated, so
    any producer rank serves).  The plan is expressed in KV-head indices of the
    per-rank blocks; block ids map one to one.  (omni_npu/connector/utils.py:13-180
    solves the same problem for token-interleaved decode context parallelism.)"""

    def __init__(self, num_kv_heads: int, p_tp: int, d_tp: int, replicated: bool = False) -> None:
        self.num_kv_heads, self.p_tp, self.d_tp, self.replicated = num_kv_heads, p_tp, d_tp, replicated
        if not replicated and (num_kv_heads % p_tp or num_kv_heads % d_tp) and \
                not (p_tp % num_kv_heads == 0 or d_tp % num_kv_heads == 0):
            raise ValueError("KV heads must divide (or be divided by) both TP sizes")

    def heads_of(self, tp: int, rank: int) -> Tuple[int, int]:
        """Global KV-head range [lo, hi) held by ``rank`` at TP degree ``tp``."""
        if tp >= self.num_kv_heads:
            h = rank * self.num_kv_heads // tp
            return h, h + 1
        per = self.num_kv_heads // tp
        return rank * per, (rank + 1) * per

    def plan(self, d_rank: int) -> ReshardPlan:
        if self.replicated:
            return ReshardPlan([(get_p_start_rank(self.p_tp, self.d_tp, d_rank), (0, 1), (0, 1))])
        d_lo, d_hi = self.heads_of(self.d_tp, d_rank)
        out = []
        seen = set()
        for p_rank in range(self.p_tp):
            p_lo, p_hi = self.heads_of(self.p_tp, p_rank)
            lo, hi = max(d_lo, p_lo), min(d_hi, p_hi)
            if lo >= hi or (p_lo, p_hi) in seen:
                continue
            seen.add((p_lo, p_hi))     # replicas of the same head range: take the first
            out.append((p_rank, (lo - p_lo, hi - p_lo), (lo - d_lo, hi - d_lo)))
        return ReshardPlan(out)

    def remap_blocks(self, remote_block_ids: Sequence[int], num_tokens: int, block_size: int) -> List[int]:
        """Blocks that actually hold tokens (the tail of the producer's list may be unused)."""
        n = (num_tokens + block_size - 1) // block_size
        return list(remote_block_ids[:n])


# ------------------------------------------------------------------------------------------------
# Token-interleaved caches (decode context parallelism): token p of a sequence lives on rank
# p % world at local index p // world.  When the decode instance shards over more ranks than the
# prefill instance (d_world = stride x p_world) a consumer rank needs every stride-th token of ONE
# producer rank.  The reference pulls whole blocks at a block stride and then evens out the tail
# block's tokens with an all-to-all among the consumer ranks (omni_npu/connector/utils.py:27-74,
# 126-180); with per-token interleaving the same result is a strided gather out of the pulled
# blocks, with no exchange between consumer ranks.
@dataclass
class DcpReshardPlan:
    src_rank: int                 # producer rank this consumer rank pulls from
    num_tokens: int               # tokens this consumer rank ends up holding
    src_blocks: List[int]         # indices into the producer rank's block list that must be pulled
    src_local: List[int]          # producer-local token index of each token, in consumer-local order


def plan_dcp_reshard(num_tokens: int, p_world: int, d_world: int, d_rank: int, block_size: int) -> DcpReshardPlan:
    """Which of the producer's tokens consumer rank ``d_rank`` takes, and from which blocks."""
    if d_world % p_world != 0:
        raise ValueError(f"consumer world {d_world} must be a multiple of the producer world {p_world}")
    stride = d_world // p_world
    a, b = divmod(d_rank, p_world)                       # token p = (k * stride + a) * p_world + b
    n = max(0, -(-(num_tokens - d_rank) // d_world))     # tokens with p % d_world == d_rank
    src_local = [k * stride + a for k in range(n)]
    blocks = sorted({i // block_size for i in src_local})
    return DcpReshardPlan(b, n, blocks, src_local)


def apply_dcp_reshard(dst_cache, dst_block_ids: Sequence[int], pulled, plan: DcpReshardPlan, block_size: int) -> None:
    """Move the planned tokens from ``pulled`` (the producer blocks named by ``plan.src_blocks``, in
    that order, shape [len(src_blocks), block_size, ...]) into ``dst_cache`` ([num_blocks,
    block_size, ...]) at this rank's blocks ``dst_block_ids``: consumer-local token k goes to block
    ``dst_block_ids[k // block_size]``, offset ``k % block_size``."""
    import torch
    if plan.num_tokens == 0:
        return
    where = {blk: i for i, blk in enumerate(plan.src_blocks)}
    dev = dst_cache.device
    src_b = torch.tensor([where[i // block_size] for i in plan.src_local], dtype=torch.long, device=dev)
    src_o = torch.tensor([i % block_size for i in plan.src_local], dtype=torch.long, device=dev)
    k = torch.arange(plan.num_tokens, device=dev)
    dst_b = torch.tensor(list(dst_block_ids), dtype=torch.long, device=dev)[k // block_size]
    dst_cache[dst_b, k % block_size] = pulled[src_b, src_o]
