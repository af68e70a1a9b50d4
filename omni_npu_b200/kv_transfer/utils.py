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
