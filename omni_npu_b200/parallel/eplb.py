"""Expert-parallel load balancing (EPLB): load statistics, redundant-expert placement and the
logical -> physical expert remap applied to the router's choice every step.

A MoE layer with ``E`` logical experts may own ``P >= E`` physical expert slots spread over
the expert-parallel ranks (``P / ep_size`` per rank).  The extra ``P - E`` slots hold copies
of the most loaded experts, so the tokens of a hot expert are shared between its replicas
and the per-rank work evens out.  Three pieces:

* ``EplbState.record`` / ``remap`` run inside the step, on the device, with static shapes
  (a scatter-add histogram and two gathers), so they are CUDA-graph capturable.
* ``plan_placement`` turns a load vector into a physical -> logical map: replicas are
  handed out one by one to the expert with the largest load per replica, then the
  physical experts are packed onto ranks largest-first into the least loaded rank that
  still has a free slot.
* ``rearrange_expert_weights`` moves expert weights between ranks after a re-plan
  (one broadcast per physical slot whose content changes; slots that keep their expert
  are untouched).

Fills the role of the external planner the reference hooks in
(omni_npu/distributed/eplb_state.py:14-69: initial map ``[0..E) + [i % E]``, ``step()`` calls
``place_experts``) and of its MoE-layer remap hook
(omni_npu/layers/quantization/compressed_tensors/compressed_tensors_moe.py:47-65,225-235).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch


def initial_physical_to_logical(num_logical: int, num_redundant: int) -> List[int]:
    """Slots ``[0, E)`` hold the experts in order, redundant slot i holds expert ``i % E``."""
    return list(range(num_logical)) + [i % num_logical for i in range(num_redundant)]


def plan_placement(load: Sequence[float], num_physical: int, num_ranks: int) -> List[int]:
    """physical -> logical map (length ``num_physical``, rank r owns the contiguous slots
    ``[r * P/R, (r+1) * P/R)``) that balances ``load`` over the ranks."""
    e = len(load)
    if num_physical < e or num_physical % num_ranks != 0:
        raise ValueError("num_physical must be >= the number of experts and divisible by the rank count")
    load = [max(float(x), 0.0) for x in load]
    replicas = [1] * e
    for _ in range(num_physical - e):
        hot = max(range(e), key=lambda i: (load[i] / replicas[i], -i))
        replicas[hot] += 1
    items = sorted(((load[i] / replicas[i], i) for i in range(e) for _ in range(replicas[i])),
                   key=lambda t: (-t[0], t[1]))
    per_rank = num_physical // num_ranks
    rank_load = [0.0] * num_ranks
    rank_slots: List[List[int]] = [[] for _ in range(num_ranks)]
    for w, i in items:
        # least loaded rank with a free slot; prefer one that does not hold this expert yet
        cands = [r for r in range(num_ranks) if len(rank_slots[r]) < per_rank]
        fresh = [r for r in cands if i not in rank_slots[r]] or cands
        r = min(fresh, key=lambda q: (rank_load[q], q))
        rank_slots[r].append(i)
        rank_load[r] += w
    return [i for r in range(num_ranks) for i in sorted(rank_slots[r])]


def logical_to_physical(phy2log: Sequence[int], num_logical: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(map int32 [E, max_replicas] padded with the first replica, replica counts int32 [E])."""
    slots: List[List[int]] = [[] for _ in range(num_logical)]
    for p, l in enumerate(phy2log):
        slots[l].append(p)
    if any(len(s) == 0 for s in slots):
        raise ValueError("every logical expert needs at least one physical slot")
    width = max(len(s) for s in slots)
    table = torch.tensor([s + [s[0]] * (width - len(s)) for s in slots], dtype=torch.int32)
    return table, torch.tensor([len(s) for s in slots], dtype=torch.int32)


class EplbState:
    """Per-layer EPLB state.  All tensors live on ``device`` and keep their shapes for the
    life of the layer, so a captured graph sees placement changes through their contents."""

    def __init__(self, num_logical: int, num_redundant: int, ep_size: int, device=None) -> None:
        self.num_logical = num_logical
        self.num_physical = num_logical + num_redundant
        if self.num_physical % ep_size != 0:
            raise ValueError("logical + redundant experts must divide evenly over the expert-parallel ranks")
        self.ep_size = ep_size
        self.device = device
        self.max_replicas = 1 + num_redundant          # worst case: every spare slot copies one expert
        self.load = torch.zeros(num_logical, dtype=torch.float32, device=device)
        self.phy2log = torch.zeros(self.num_physical, dtype=torch.int32, device=device)
        self.log2phy = torch.zeros(num_logical, self.max_replicas, dtype=torch.int32, device=device)
        self.replicas = torch.ones(num_logical, dtype=torch.int32, device=device)
        self.steps = 0
        self.set_placement(initial_physical_to_logical(num_logical, num_redundant))

    # ------------------------------------------------------------- placement
    def set_placement(self, phy2log: Sequence[int]) -> None:
        table, counts = logical_to_physical(phy2log, self.num_logical)
        full = table[:, :1].repeat(1, self.max_replicas)
        full[:, : table.shape[1]] = table
        self.phy2log.copy_(torch.tensor(list(phy2log), dtype=torch.int32))
        self.log2phy.copy_(full)
        self.replicas.copy_(counts)

    def placement(self) -> List[int]:
        return self.phy2log.tolist()

    def local_slots(self, rank: int) -> range:
        per = self.num_physical // self.ep_size
        return range(rank * per, (rank + 1) * per)

    def local_logical_ids(self, rank: int) -> List[int]:
        p = self.placement()
        return [p[s] for s in self.local_slots(rank)]

    # ------------------------------------------------------------ step hooks
    def record(self, ids: torch.Tensor) -> None:
        """Add this step's routed tokens to the load histogram (``ids`` int [T, k], -1 = none)."""
        flat = ids.reshape(-1).long()
        valid = (flat >= 0).to(self.load.dtype)
        self.load.index_add_(0, flat.clamp_min(0), valid)
        self.steps += 1

    def remap(self, ids: torch.Tensor) -> torch.Tensor:
        """Logical expert ids [T, k] -> physical ids; the replicas of an expert are used round
        robin over the token index, so their shares are equal for any batch."""
        t, k = ids.shape
        safe = ids.clamp_min(0).long()
        n = self.replicas[safe].long()
        tok = torch.arange(t, device=ids.device).unsqueeze(1).expand(t, k)
        phys = self.log2phy[safe, tok % n]
        return torch.where(ids >= 0, phys.to(ids.dtype), ids)

    # ------------------------------------------------------------- re-planning
    def global_load(self, group=None) -> torch.Tensor:
        load = self.load.clone()
        if group is not None and group.world_size > 1:
            load = group.all_reduce(load)
        return load

    def replan(self, group=None, decay: float = 0.0) -> Tuple[List[int], List[int]]:
        """New placement from the (group-wide) load seen so far.  Returns (old, new) physical ->
        logical maps; the statistics are decayed (0 = reset).  The caller moves the weights
        (``rearrange_expert_weights``) and then calls ``set_placement(new)``."""
        load = self.global_load(group).tolist()
        old = self.placement()
        new = plan_placement(load, self.num_physical, self.ep_size)
        new = _keep_in_place(old, new, self.num_physical // self.ep_size)
        self.load.mul_(decay)
        return old, new

    def imbalance(self, group=None) -> float:
        """max / mean of the per-rank load under the current placement (1.0 = perfect)."""
        load = self.global_load(group)
        per_phys = (load / self.replicas.to(load.dtype))[self.phy2log.long()]
        per_rank = per_phys.view(self.ep_size, -1).sum(1)
        mean = per_rank.mean().clamp_min(1e-9)
        return float(per_rank.max() / mean)


def _keep_in_place(old: Sequence[int], new: Sequence[int], per_rank: int) -> List[int]:
    """Reorder the slots of each rank in ``new`` so that experts the rank already holds stay in
    the slot they occupy: fewer weights to move."""
    out: List[int] = []
    for r in range(len(new) // per_rank):
        o = list(old[r * per_rank: (r + 1) * per_rank])
        n = list(new[r * per_rank: (r + 1) * per_rank])
        slots: List[Optional[int]] = [None] * per_rank
        for i, e in enumerate(o):
            if e in n:
                slots[i] = e
                n.remove(e)
        for i in range(per_rank):
            if slots[i] is None:
                slots[i] = n.pop(0)
        out.extend(slots)          # type: ignore[arg-type]
    return out


def rearrange_expert_weights(params: Iterable[torch.Tensor], old: Sequence[int], new: Sequence[int], group,
                             ) -> int:
    """Make the physical slots hold the experts of ``new``.  ``params``: this rank's expert
    tensors ``[local_slots, ...]``.  For every slot whose expert changes, a rank that held that
    expert under ``old`` broadcasts it to the slot's owner.  Returns the number of moved slots.
    Collective over ``group`` (every rank passes the same ``old`` / ``new``)."""
    world = group.world_size if group is not None else 1
    rank = group.rank_in_group if group is not None else 0
    per = len(new) // world
    params = list(params)
    holders: Dict[int, int] = {}
    for p, e in enumerate(old):
        holders.setdefault(e, p)
    # read every source before any slot is overwritten
    staged: Dict[int, List[torch.Tensor]] = {}
    moves = [(p, new[p], holders[new[p]]) for p in range(len(new)) if new[p] != old[p]]
    for dst, _, src in moves:
        if src // per == rank:
            staged[dst] = [t[src % per].clone() for t in params]
    for dst, _, src in moves:
        src_rank, dst_rank = src // per, dst // per
        if src_rank == dst_rank:
            if rank == dst_rank:
                for t, s in zip(params, staged[dst]):
                    t[dst % per].copy_(s)
            continue
        for i, t in enumerate(params):
            if rank == src_rank:
                buf = staged[dst][i]
            elif rank == dst_rank:
                buf = torch.empty_like(t[dst % per])
            else:
                buf = torch.empty_like(t[0])
            buf = group.broadcast(buf, src=src_rank)
            if rank == dst_rank:
                t[dst % per].copy_(buf)
    return len(moves)
