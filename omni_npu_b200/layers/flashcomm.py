"""Sequence-parallel residual stream inside a tensor-parallel group ("FlashComm-1").

With plain tensor parallelism every rank holds the full ``[T, H]`` residual stream and
each row-parallel projection ends in an all-reduce.  Here the stream is sharded by
tokens instead: rank r keeps rows ``[r*T/tp, (r+1)*T/tp)``.  Around each block

    full  = all_gather(norm(shard))         # before QKV / gate_up (column-parallel GEMMs)
    part  = block(full)                      # row-parallel output, still a partial sum
    shard = shard + reduce_scatter(part)     # instead of all-reduce + replicated add

so the residual adds and RMSNorms run on ``T/tp`` rows, and the bytes on NVLink are the
same as one all-reduce (reduce-scatter + all-gather).  Over peer-mapped memory both
collectives are single kernels (``parallel/symm_mem.py``).  ``T`` is padded to a multiple
of the group size; the padding rows are dropped at the end.

Same pattern as the reference's v0 Qwen3-MoE (slice after embedding, all-gather before
QKV, reduce-scatter after o_proj, all-gather at the final norm:
omni_npu/v0/models/qwen/qwen3_moe.py:216,258,405-413,443,464) and the
``x_transform`` / ``y_transform`` hooks of its v1 linears (omni_npu/v1/layers/linear.py:39-53).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


class ShardedRows:
    """A token-sharded activation on its way into a column-parallel projection.  The projection
    either consumes the shard directly (all-gather fused into its GEMM over peer memory) or
    asks for the gathered rows."""

    def __init__(self, shard: torch.Tensor, stream: "SequenceParallelStream") -> None:
        self.shard = shard
        self.stream = stream
        self._full: Optional[torch.Tensor] = None

    @property
    def num_tokens(self) -> int:
        return self.stream.num_tokens

    @property
    def shape(self):
        return (self.stream.num_tokens,) + tuple(self.shard.shape[1:])

    def full(self) -> torch.Tensor:
        if self._full is None:
            self._full = self.stream.gather(self.shard)[: self.stream.num_tokens]
        return self._full


class SequenceParallelStream:
    def __init__(self, group) -> None:
        self.group = group
        self.world = group.world_size
        self.rank = group.rank_in_group
        self.num_tokens = 0
        self.padded = 0
        self.fused_gather = False     # True: blocks get ShardedRows; their first projection fuses the gather

    @property
    def enabled(self) -> bool:
        return self.world > 1

    # ------------------------------------------------------------- enter / leave
    def scatter(self, x: torch.Tensor) -> torch.Tensor:
        """Full ``[T, H]`` (identical on every rank) -> this rank's token shard."""
        self.num_tokens = x.shape[0]
        per = (self.num_tokens + self.world - 1) // self.world
        self.padded = per * self.world
        if self.padded != self.num_tokens:
            x = torch.cat([x, x.new_zeros(self.padded - self.num_tokens, *x.shape[1:])], dim=0)
        return x[self.rank * per: (self.rank + 1) * per].contiguous()

    def gather(self, shard: torch.Tensor, trim: bool = False) -> torch.Tensor:
        """Token shard -> full rows (padded unless ``trim``)."""
        comm = self.group.comm
        symm = getattr(comm, "symm", None)
        if symm is not None and shard.is_cuda and symm._ok(shard) and \
                shard.numel() * 2 * self.world <= symm.half_bytes:
            full = symm.all_gather(shard)
        else:
            full = self.group.all_gather(shard, dim=0)
        return full[: self.num_tokens] if trim else full

    def reduce_scatter(self, partial: torch.Tensor) -> torch.Tensor:
        """Partial sums over the full (padded) rows -> reduced shard of this rank."""
        if partial.shape[0] != self.padded:
            partial = torch.cat([partial, partial.new_zeros(self.padded - partial.shape[0], *partial.shape[1:])], 0)
        comm = self.group.comm
        symm = getattr(comm, "symm", None)
        if symm is not None and partial.is_cuda and symm._ok(partial) and \
                partial.numel() * 2 <= symm.half_bytes:
            return symm.reduce_scatter(partial)
        return self.group.reduce_scatter(partial, dim=0)

    # ----------------------------------------------------------------- blocks
    def block(self, norm, shard_hidden: Optional[torch.Tensor], shard_residual: torch.Tensor,
              fn) -> Tuple[torch.Tensor, torch.Tensor]:
        """One pre-norm block on the sharded stream.  ``shard_hidden`` is the previous block's
        reduced output shard (None at the very first block, where ``shard_residual`` is the
        embedding shard).  ``fn(full_rows) -> partial sums``.  Returns (output shard, residual)."""
        if shard_hidden is None:
            normed = norm(shard_residual)
        else:
            normed, shard_residual = norm(shard_hidden, shard_residual)
        symm = getattr(self.group.comm, "symm", None)
        if self.fused_gather and symm is not None and normed.is_cuda and normed.shape[0] % 128 == 0:
            # the block's first projection reads the shards from their owners inside its GEMM
            return self._reduced(fn(ShardedRows(normed, self))), shard_residual
        full = self.gather(normed)[: self.num_tokens]
        return self._reduced(fn(full)), shard_residual

    def _reduced(self, out) -> torch.Tensor:
        """Block output -> reduced shard: already reduced inside the block's last GEMM
        (``layers.linear.ReducedShard``) or a partial sum that still needs the reduce-scatter."""
        if isinstance(out, torch.Tensor):
            return self.reduce_scatter(out)
        return out.tensor

    @property
    def scatter_mode(self):
        """What a block passes as ``reduce=`` to its row-parallel projection."""
        return "scatter" if (self.fused_gather and self.padded == self.num_tokens) else False
