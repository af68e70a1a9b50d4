"""Group-scoped communication helpers for model code.

Thin functions over the named groups of ``parallel/state.py``: every helper is a no-op on
a group of one rank, takes either a group object or the key of a per-layer group, and
works on any dimension.  They are what layer code calls instead of touching
``torch.distributed`` (the reference's ``communication_op_ext``:
omni_npu/v1/distributed/communication_op_ext.py:37-181).

The reference's v0 tree also has *hierarchical* collectives for multi-node Ascend
clusters: two-stage (node-local then cross-node), near/far pipelined and round-robin
variants (omni_npu/v0/distributed/communication_op.py:40-292).  Inside one NVSwitch
domain every peer is one hop away at full bandwidth, so here those entry points exist with
the same names but run the single-stage collective; the local-world group is kept for
code that shards the LM head over the GPUs of one box.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch

from . import state as pstate
from .state import GroupCoordinator

GroupLike = Union[GroupCoordinator, str, None]


def _group(group: GroupLike) -> GroupCoordinator:
    if group is None:
        return pstate.get_tp_group()
    if isinstance(group, str):
        g = pstate.get_layer_group(group)
        return g if g is not None else pstate.get_tp_group()
    return group


def get_world_size(group: GroupLike = None) -> int:
    return _group(group).world_size


def get_rank(group: GroupLike = None) -> int:
    return _group(group).rank_in_group


# ------------------------------------------------------------ single stage
def all_reduce(x: torch.Tensor, group: GroupLike = None) -> torch.Tensor:
    g = _group(group)
    return x if g.world_size == 1 else g.all_reduce(x)


def all_gather(x: torch.Tensor, dim: int = -1, group: GroupLike = None) -> torch.Tensor:
    g = _group(group)
    return x if g.world_size == 1 else g.all_gather(x, dim)


def reduce_scatter(x: torch.Tensor, dim: int = 0, group: GroupLike = None) -> torch.Tensor:
    g = _group(group)
    return x if g.world_size == 1 else g.reduce_scatter(x, dim)


def all_gatherv(x: torch.Tensor, sizes: Sequence[int], dim: int = 0, group: GroupLike = None) -> torch.Tensor:
    g = _group(group)
    return x if g.world_size == 1 else g.all_gatherv(x, dim, list(sizes))


def reduce_scatterv(x: torch.Tensor, sizes: Sequence[int], dim: int = 0, group: GroupLike = None) -> torch.Tensor:
    g = _group(group)
    return x if g.world_size == 1 else g.reduce_scatterv(x, dim, list(sizes))


def all_to_all(x: torch.Tensor, scatter_dim: int = 0, gather_dim: int = -1, group: GroupLike = None,
               scatter_sizes: Optional[List[int]] = None, gather_sizes: Optional[List[int]] = None) -> torch.Tensor:
    g = _group(group)
    if g.world_size == 1:
        return x
    return g.comm.all_to_all(x, scatter_dim, gather_dim, scatter_sizes, gather_sizes)


def broadcast(x: torch.Tensor, src: int = 0, group: GroupLike = None) -> torch.Tensor:
    g = _group(group)
    return x if g.world_size == 1 else g.broadcast(x, src)


def sequence_parallel_chunk(x: torch.Tensor, group: GroupLike = None) -> torch.Tensor:
    """This rank's slice of the rows of ``x`` (zero-padded to a multiple of the group size)."""
    g = _group(group)
    if g.world_size == 1:
        return x
    per = (x.shape[0] + g.world_size - 1) // g.world_size
    pad = per * g.world_size - x.shape[0]
    if pad:
        x = torch.cat([x, x.new_zeros(pad, *x.shape[1:])], dim=0)
    return x[g.rank_in_group * per: (g.rank_in_group + 1) * per]


# -------------------------------------------------- hierarchical entry points
def all_reduce_two_stage(x: torch.Tensor, group: GroupLike = None) -> torch.Tensor:
    """Node-local reduce-scatter + cross-node all-reduce + node-local all-gather on a
    multi-node cluster; one NVSwitch domain needs a single stage."""
    return all_reduce(x, group)


def all_gather_two_stage(x: torch.Tensor, dim: int = 0, group: GroupLike = None) -> torch.Tensor:
    return all_gather(x, dim, group)


def reduce_scatter_two_stage(x: torch.Tensor, dim: int = 0, group: GroupLike = None) -> torch.Tensor:
    return reduce_scatter(x, dim, group)


def all_gather_pipeline(x: torch.Tensor, dim: int = 0, group: GroupLike = None) -> torch.Tensor:
    """Near/far pipelined gather of the reference: nothing to pipeline between uniform peers."""
    return all_gather(x, dim, group)


def all_gather_round_pipeline(x: torch.Tensor, dim: int = 0, group: GroupLike = None) -> torch.Tensor:
    return all_gather(x, dim, group)


def all_gather_local(x: torch.Tensor, dim: int = 0) -> torch.Tensor:
    """Gather over the GPUs of this box (the group the LM head is sharded over)."""
    return all_gather(x, dim, pstate.get_local_world_group())


def all_to_all_local(x: torch.Tensor, scatter_dim: int = 0, gather_dim: int = -1) -> torch.Tensor:
    return all_to_all(x, scatter_dim, gather_dim, pstate.get_local_world_group())
