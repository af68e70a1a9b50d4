"""Process-group state: world, tensor / pipeline / data / expert parallel groups,
a node-local group, and named per-layer groups.

Rank layout (outermost to innermost): DP x PP x TP, the same order vLLM uses,
so rank = dp * (pp * tp) + pp_rank * tp + tp_rank.  The expert-parallel group
spans DP x TP of one pipeline stage.  Every group owns a device process group
(NCCL on GPUs, gloo on CPU), a gloo CPU group for host-side barriers and object
exchange, and a :class:`B200Communicator`.

Per-layer groups (the reference's "layer parallel" JSON,
omni_npu/v1/distributed/parallel_state_ext.py:123-193,380-545) let single
linears run with a TP degree or rank list different from the model-wide one.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Union

import torch
import torch.distributed as dist

from ..logger import logger

from .communicator import B200Communicator


class GroupCoordinator:
    def __init__(self, ranks: Sequence[int], device: torch.device, backend: str, name: str,
                 all_rank_lists: Optional[Sequence[Sequence[int]]] = None) -> None:
        self.name = name
        self.ranks = list(ranks)
        self.world_size = len(self.ranks)
        self.device = device
        my = dist.get_rank() if dist.is_initialized() else 0
        self.rank_in_group = self.ranks.index(my) if my in self.ranks else 0
        self.device_group = None
        self.cpu_group = None
        if dist.is_initialized() and dist.get_world_size() > 1:
            # new_group is collective over the default group: every rank must
            # create every subgroup, in the same order.
            for rl in (all_rank_lists or [self.ranks]):
                dg = dist.new_group(list(rl), backend=backend)
                cg = dg if backend == "gloo" else dist.new_group(list(rl), backend="gloo")
                if my in rl:
                    self.device_group, self.cpu_group = dg, cg
        self.comm = B200Communicator(self.cpu_group, device, self.device_group, unique_name=name)

    @property
    def is_first_rank(self) -> bool:
        return self.rank_in_group == 0

    @property
    def is_last_rank(self) -> bool:
        return self.rank_in_group == self.world_size - 1

    # thin forwards so call sites read like the usual group API
    def all_reduce(self, x):
        return self.comm.all_reduce(x)

    def all_gather(self, x, dim=-1):
        return self.comm.all_gather(x, dim)

    def reduce_scatter(self, x, dim=-1):
        return self.comm.reduce_scatter(x, dim)

    def all_reduce_async(self, x):
        return self.comm.all_reduce_async(x)

    def all_gather_async(self, x, dim=0):
        return self.comm.all_gather_async(x, dim)

    def reduce_scatter_async(self, x, dim=0):
        return self.comm.reduce_scatter_async(x, dim)

    def all_gatherv(self, x, dim=0, sizes=None):
        return self.comm.all_gatherv(x, dim, sizes)

    def reduce_scatterv(self, x, dim=0, sizes=None):
        return self.comm.reduce_scatterv(x, dim, sizes)

    def all_to_all_single(self, x, output_split_sizes=None, input_split_sizes=None):
        return self.comm.all_to_all_single(x, output_split_sizes, input_split_sizes)

    def swap(self, x):
        """Exchange ``x`` with the other rank of a two-rank group (each side receives the peer's
        tensor of the same shape); the 2-rank shortcut the reference's v0 coordinator offers
        for DP<->TP hand-overs (omni_npu/v0/distributed/parallel_state.py:52-208)."""
        if self.world_size == 1:
            return x
        if self.world_size != 2:
            raise ValueError("swap() is defined for groups of exactly two ranks")
        both = self.all_gather(x.unsqueeze(0), dim=0)
        return both[1 - self.rank_in_group].contiguous()

    def broadcast(self, x, src=0):
        return self.comm.broadcast(x, src)

    def broadcast_object(self, obj, src: int = 0):
        if self.world_size == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=self.ranks[src], group=self.cpu_group)
        return box[0]

    def all_gather_object(self, obj) -> list:
        if self.world_size == 1:
            return [obj]
        out = [None] * self.world_size
        dist.all_gather_object(out, obj, group=self.cpu_group)
        return out

    def barrier(self):
        self.comm.barrier()

    def send(self, x, dst=None):
        self.comm.send(x, dst)

    def recv(self, size, dtype, src=None):
        return self.comm.recv(size, dtype, src)

    def destroy(self):
        self.comm.destroy()


@dataclass
class _State:
    world: Optional[GroupCoordinator] = None
    tp: Optional[GroupCoordinator] = None
    pp: Optional[GroupCoordinator] = None
    dp: Optional[GroupCoordinator] = None
    ep: Optional[GroupCoordinator] = None
    pcp: Optional[GroupCoordinator] = None
    local: Optional[GroupCoordinator] = None
    layer_groups: Optional[Dict[str, GroupCoordinator]] = None
    layer_transforms: Optional[Dict[str, tuple]] = None
    backend: str = "gloo"
    device: Optional[torch.device] = None
    initialized: bool = False


_S = _State()


def init_distributed(device: torch.device, backend: Optional[str] = None,
                     init_method: Optional[str] = None, world_size: Optional[int] = None,
                     rank: Optional[int] = None, timeout_s: float = 600.0) -> None:
    """Join the default process group (env:// by default).  A single process
    without RANK/WORLD_SIZE in the environment stays un-initialised: every
    group then has world size 1 and every collective is the identity."""
    import datetime
    world_size = int(os.environ.get("WORLD_SIZE", "1")) if world_size is None else world_size
    rank = int(os.environ.get("RANK", "0")) if rank is None else rank
    backend = backend or ("nccl" if device.type == "cuda" else "gloo")
    _S.backend, _S.device = backend, device
    if world_size > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        kw = {}
        if device.type == "cuda":
            kw["device_id"] = device
        dist.init_process_group(backend=backend, init_method=init_method or "env://",
                                world_size=world_size, rank=rank,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)


def init_model_parallel(tp: int = 1, pp: int = 1, dp: int = 1, device: Optional[torch.device] = None,
                        backend: Optional[str] = None, pcp: int = 1) -> None:
    """Rank grid [dp, pp, pcp, tp], tp fastest.  ``pcp`` is the prefill-context-parallel dimension:
    its ranks hold different tokens of the same prompts.  The expert-parallel group spans dp x pcp x
    tp of one pipeline stage, so a MoE layer fed with a rank's own token shard needs nothing around
    it: dispatch sends each shard's rows to the experts' owners and combine brings them back
    (the reference all-gathers hidden states and router logits over the PCP group before its MoE and
    reduce-scatters after it: omni_npu/vllm_patches/patches/models/pangu72b-vl/patch_fusedmoe.py:148-159,216-220)."""
    device = device or _S.device or torch.device("cpu")
    backend = backend or _S.backend or ("nccl" if device.type == "cuda" else "gloo")
    _S.device, _S.backend = device, backend
    world = dist.get_world_size() if dist.is_initialized() else 1
    if world != tp * pp * dp * pcp:
        raise ValueError(f"world size {world} != tp {tp} * pp {pp} * dp {dp} * pcp {pcp}")
    rank = dist.get_rank() if dist.is_initialized() else 0
    grid = torch.arange(world).view(dp, pp, pcp, tp)

    def make(name: str, lists: List[List[int]]) -> GroupCoordinator:
        mine = next(l for l in lists if rank in l)
        return GroupCoordinator(mine, device, backend, name, all_rank_lists=lists)

    _S.world = make("world", [list(range(world))])
    _S.tp = make("tp", grid.reshape(-1, tp).tolist())
    _S.pp = make("pp", grid.permute(0, 2, 3, 1).reshape(-1, pp).tolist())
    _S.dp = make("dp", grid.permute(1, 2, 3, 0).reshape(-1, dp).tolist())
    _S.ep = make("ep", grid.permute(1, 0, 2, 3).reshape(pp, dp * pcp * tp).tolist())
    _S.pcp = make("pcp", grid.permute(0, 1, 3, 2).reshape(-1, pcp).tolist())
    _S.local = _S.world
    _S.layer_groups = {}
    _S.layer_transforms = {}
    _S.initialized = True


def model_parallel_is_initialized() -> bool:
    return _S.initialized


def ensure_initialized(device: Optional[torch.device] = None) -> None:
    if not _S.initialized:
        init_model_parallel(1, 1, 1, device or torch.device("cpu"))


def _get(name: str) -> GroupCoordinator:
    ensure_initialized()
    return getattr(_S, name)


def get_world_group() -> GroupCoordinator:
    return _get("world")


def get_tp_group() -> GroupCoordinator:
    return _get("tp")


def get_pp_group() -> GroupCoordinator:
    return _get("pp")


def get_dp_group() -> GroupCoordinator:
    return _get("dp")


def get_ep_group() -> GroupCoordinator:
    return _get("ep")


def get_pcp_group() -> GroupCoordinator:
    return _get("pcp")


def get_local_world_group() -> GroupCoordinator:
    return _get("local")


def tp_world_size() -> int:
    return get_tp_group().world_size


def tp_rank() -> int:
    return get_tp_group().rank_in_group


# ------------------------------------------------------------ per-layer groups
def register_layer_group(key: str, tp_size_or_ranks: Union[int, Sequence[Sequence[int]]]) -> GroupCoordinator:
    """Create (collectively) a named group.  An int n partitions the world into
    consecutive groups of n ranks; a list of rank lists is used as given."""
    ensure_initialized()
    world = _S.world.world_size
    if isinstance(tp_size_or_ranks, int):
        n = tp_size_or_ranks
        if world % n != 0:
            raise ValueError(f"layer group size {n} does not divide world size {world}")
        lists = [list(range(i, i + n)) for i in range(0, world, n)]
    else:
        lists = [list(l) for l in tp_size_or_ranks]
        flat = sorted(r for l in lists for r in l)
        if flat != list(range(world)):
            raise ValueError("layer group rank lists must partition the world")
    rank = dist.get_rank() if dist.is_initialized() else 0
    mine = next(l for l in lists if rank in l)
    g = GroupCoordinator(mine, _S.device, _S.backend, f"layer:{key}", all_rank_lists=lists)
    _S.layer_groups[key] = g
    return g


def get_layer_group(key: str) -> Optional[GroupCoordinator]:
    ensure_initialized()
    return _S.layer_groups.get(key)


_TRANSFORM_NAMES = {"none": None, "noop": None, "allreduce": "AllReduce", "allgather": "AllGather",
                    "reducescatter": "ReduceScatter", "all2all": "ALL2ALL", "alltoall": "ALL2ALL"}


def _transform_name(spec) -> Optional[str]:
    if spec is None:
        return None
    kind = spec.get("type") if isinstance(spec, dict) else spec
    key = str(kind).replace("_", "").lower()
    if key not in _TRANSFORM_NAMES:
        raise ValueError(f"unknown transform type {kind!r}")
    return _TRANSFORM_NAMES[key]


def apply_layer_parallel_config(layer_parallel_config: Dict[str, dict]) -> Dict[str, GroupCoordinator]:
    """Create the per-layer groups and record the input / output transforms a
    deployment plan asks for.  ``layer_parallel_config`` maps a layer key (the last
    two components of the module name, e.g. ``"mlp.down_proj"``) to
    ``{"tp_size_or_ranks": int | [[ranks]...], "x_transform": {"type": ...},
    "y_transform": {"type": ...}}``.  Every rank must call this with the same
    dictionary (group creation is collective).  Same role as
    ``init_layer_parallel_groups`` in omni_npu/v1/distributed/parallel_state_ext.py:380-545."""
    ensure_initialized()
    made = {}
    for key in sorted(layer_parallel_config):
        spec = layer_parallel_config[key] or {}
        size = spec.get("tp_size_or_ranks", None)
        if size is not None:
            made[key] = register_layer_group(key, size)
        _S.layer_transforms[key] = (_transform_name(spec.get("x_transform")),
                                    _transform_name(spec.get("y_transform")))
    return made


def get_layer_transforms(key: str) -> tuple:
    """(x_transform, y_transform) recorded for a layer key, (None, None) if none."""
    ensure_initialized()
    return (_S.layer_transforms or {}).get(key, (None, None))


def destroy_model_parallel() -> None:
    for g in (_S.tp, _S.pp, _S.dp, _S.ep, _S.pcp, _S.world):
        if g is not None:
            g.destroy()
    for g in (_S.layer_groups or {}).values():
        g.destroy()
    _S.world = _S.tp = _S.pp = _S.dp = _S.ep = _S.pcp = _S.local = None
    _S.layer_groups = None
    _S.layer_transforms = None
    _S.initialized = False


def destroy_distributed() -> None:
    destroy_model_parallel()
    if dist.is_initialized():
        dist.destroy_process_group()


def _all_groups() -> List[GroupCoordinator]:
    gs = [g for g in (_S.world, _S.tp, _S.pp, _S.dp, _S.ep, _S.pcp, _S.local) if g is not None]
    gs += list((_S.layer_groups or {}).values())
    seen, out = set(), []
    for g in gs:
        if id(g) not in seen:
            seen.add(id(g))
            out.append(g)
    return out


def abort_communicators() -> int:
    """Abort the device communicators of every group so that collectives blocked on a
    failed peer return (used by token recovery).  Returns how many were aborted."""
    n = 0
    for g in _all_groups():
        pg = getattr(g, "device_group", None)
        if pg is None:
            continue
        try:
            backend = pg._get_backend(torch.device("cuda")) if _S.backend == "nccl" else None
            abort = getattr(backend, "abort", None) or getattr(backend, "_abort", None)
            if abort is not None:
                abort()
                n += 1
        except Exception as e:        # best effort: a communicator that never started has nothing to abort
            logger.debug("abort of %s: %s", getattr(g, "name", "?"), e)
    return n


def reinit_communicators() -> None:
    """Bring the groups' communicators back after ``abort_communicators`` and drop
    peer-mapped buffers whose signal state may be mid-flight (they are rebuilt lazily)."""
    for g in _all_groups():
        comm = getattr(g, "comm", None)
        symm = getattr(comm, "symm", None)
        if symm is not None:
            try:
                symm.close()
            except Exception:
                pass
            comm.symm = None
    if dist.is_initialized() and dist.get_world_size() > 1:
        world = getattr(_S, "world", None)
        (world.barrier if world is not None else dist.barrier)()     # host-side rendezvous of the survivors


def finish_process(engine=None, code: int = 0, deadline_s: float = 30.0) -> None:
    """End a rank of a multi-process program: barrier, release peer-mapped memory and
    CUDA graphs (``engine.shutdown()``), leave the process groups, then ``os._exit``.

    A watchdog ends the process after ``deadline_s`` even if a library finaliser
    blocks: communicator tear-down has been seen to wait for minutes when peers
    unmap shared buffers in a different order."""
    import os
    import sys
    import threading

    def _now():
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(code)

    timer = threading.Timer(deadline_s, _now)
    timer.daemon = True
    timer.start()
    try:
        if dist.is_initialized() and dist.get_world_size() > 1:
            world = getattr(_S, "world", None)
            world.barrier() if world is not None else dist.barrier()   # host-side (gloo) when set up
        if engine is not None:
            engine.shutdown()
        destroy_distributed()
    except Exception as e:  # best effort: the process ends either way
        print(f"finish_process: {type(e).__name__}: {e}", file=sys.stderr)
    _now()
