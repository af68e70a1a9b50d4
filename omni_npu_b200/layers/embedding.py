"""Vocabulary-parallel embedding and LM head.

The vocabulary is split across the tensor-parallel group.  Lookup masks
tokens owned by other ranks and all-reduces (or reduce-scatters, when the
residual stream is token-sharded) the partial embeddings; the LM head
computes a vocabulary shard of the logits and all-gathers it
(reference: omni_npu/v1/layers/vocab_parallel_embedding.py:161-265).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from .. import ops
from ..parallel import state as pstate


def pad_vocab(vocab: int, multiple: int = 64) -> int:
    return (vocab + multiple - 1) // multiple * multiple


class VocabParallelEmbedding(nn.Module):
    def __init__(self, vocab_size: int, hidden_size: int, dtype=torch.bfloat16, device=None,
                 group=None) -> None:
        super().__init__()
        self.group = group or pstate.get_tp_group()
        tp = self.group.world_size
        self.vocab_size = vocab_size
        self.padded_vocab = pad_vocab(vocab_size, 64 * tp)
        self.per_rank = self.padded_vocab // tp
        self.start = self.group.rank_in_group * self.per_rank
        self.end = self.start + self.per_rank
        self.weight = nn.Parameter(torch.zeros(self.per_rank, hidden_size, dtype=dtype, device=device),
                                   requires_grad=False)

    def forward(self, ids: torch.Tensor, reduce: str = "AllReduce") -> torch.Tensor:
        ids = ids.long()
        if self.group.world_size == 1:
            return self.weight[ids]
        mask = (ids >= self.start) & (ids < self.end)
        local = torch.where(mask, ids - self.start, torch.zeros_like(ids))
        out = self.weight[local] * mask.unsqueeze(-1).to(self.weight.dtype)
        if reduce == "ReduceScatter":
            return self.group.reduce_scatter(out, dim=0)
        return self.group.all_reduce(out)

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        n = min(self.end, loaded.shape[0]) - self.start
        if n > 0:
            param.data[:n].copy_(loaded[self.start:self.start + n].to(param.dtype))


class ParallelLMHead(VocabParallelEmbedding):
    def compute_logits(self, hidden: torch.Tensor, embedding_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """hidden [B,H] -> logits [B, vocab] in fp32."""
        logits = ops.gemm(hidden, self.weight, out_dtype=torch.float32)
        if self.group.world_size > 1:
            logits = self.group.all_gather(logits, dim=-1)
        logits = logits[:, : self.vocab_size]
        if embedding_bias is not None:
            logits = logits + embedding_bias
        return logits
