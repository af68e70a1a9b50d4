"""KV connector whose blocks travel through a host-memory pool.

The prefill instance does not keep finished prompts parked in its GPU cache until the
decode instance has fetched them.  Instead it copies the request's KV blocks into a pool
in host memory (a file in ``/dev/shm`` mapped by both instances and, with a GPU, pinned so
that the copies are DMA transfers), frees its GPU blocks at once and hands the decode
instance the pool slots.  The decode instance maps the same file and copies the slots into
its own cache; its ack lets the prefill instance recycle the slots.

    producer                                   consumer
    request_finished -> D2H blocks -> slots    get_num_new_matched_tokens / alloc
    kv_transfer_params {pool, slots, ...}  ->  start_load_kv: H2D slots -> local blocks
    take_released_requests <- "pulled" ack <-  notify_pulled
    slots back on the free list

Pool layout: ``[num_slots][layer tensors of one block, back to back]``; a slot holds one KV
block of every cache tensor (K and V, or the latent and index caches).  Slot allocation is
done by the producer only, so no cross-process locking is needed; the control channel is the
one the GPU-to-GPU connector uses (``control_plane.py``).

Counterpart of the reference's host-pool connector and its transfer daemon
(omni_npu/connector/omni_cache_connector_v1.py:193-235 scheduler half, :503-541 daemon
launch, :788-823 worker half, :934-1078 transfer threads).  The external daemon has no
equivalent here: on one machine the mapped file plus ``cudaMemcpyAsync`` is the transport.
"""
from __future__ import annotations

import mmap
import os
import threading
import time
from typing import Any, Dict, List, Optional, Sequence, Set, Tuple

import torch

from ..config import EngineConfig
from ..logger import logger
from .connector import ConnectorMetadata, P2PKVConnector, ReqMeta
from .control_plane import ControlServer
from .manager import flatten_kv_caches

POOL_DIR = os.environ.get("OMNI_B200_KV_POOL_DIR", "/dev/shm")


class HostKVPool:
    """A slot array in a shared, memory-mapped file.  ``create=True`` sizes the file; the
    other side opens it by name with the same geometry."""

    def __init__(self, name: str, num_slots: int, tensor_block_bytes: Sequence[int], create: bool,
                 pin: bool = False) -> None:
        self.name = name
        self.path = os.path.join(POOL_DIR, name)
        self.num_slots = int(num_slots)
        self.tensor_block_bytes = [int(b) for b in tensor_block_bytes]
        self.offsets = [0]
        for b in self.tensor_block_bytes:
            self.offsets.append(self.offsets[-1] + b)
        self.slot_bytes = self.offsets[-1]
        total = self.slot_bytes * self.num_slots
        flags = os.O_RDWR | (os.O_CREAT if create else 0)
        fd = os.open(self.path, flags, 0o600)
        try:
            if create:
                os.ftruncate(fd, total)
            elif os.fstat(fd).st_size < total:
                raise ValueError(f"KV pool {name}: file is smaller than {total} bytes")
            self.map = mmap.mmap(fd, total)
        finally:
            os.close(fd)
        self.created = create
        self.buf = torch.frombuffer(self.map, dtype=torch.uint8).view(self.num_slots, self.slot_bytes)
        self.pinned = False
        if pin and torch.cuda.is_available():
            rc = torch.cuda.cudart().cudaHostRegister(self.buf.data_ptr(), total, 0)
            self.pinned = int(rc) == 0
            if not self.pinned:
                # the runtime keeps the failure as its "last error": read it off, or the next
                # unrelated CUDA call that checks for errors reports it
                try:
                    import ctypes
                    from pathlib import Path
                    ctypes.CDLL(str(Path(__file__).resolve().parent.parent / "_C.so")).b200_cuda_take_last_error()
                except OSError:
                    pass
                logger.warning("KV pool %s: cudaHostRegister failed (%s); copies will be pageable", name, rc)
        self._free = list(range(self.num_slots - 1, -1, -1)) if create else []
        self._lock = threading.Lock()

    def geometry(self) -> Dict[str, Any]:
        return {"pool": self.name, "num_slots": self.num_slots, "tensor_block_bytes": self.tensor_block_bytes}

    def slots_view(self, tensor_index: int) -> torch.Tensor:
        """uint8 [num_slots, block_bytes of tensor] view of one cache tensor's part of every slot."""
        return self.buf[:, self.offsets[tensor_index]: self.offsets[tensor_index + 1]]

    # -------------------------------------------------------------- allocation
    def alloc(self, n: int) -> Optional[List[int]]:
        with self._lock:
            if len(self._free) < n:
                return None
            out = [self._free.pop() for _ in range(n)]
        return out

    def free(self, slots: Sequence[int]) -> None:
        with self._lock:
            self._free.extend(slots)

    @property
    def num_free(self) -> int:
        with self._lock:
            return len(self._free)

    def close(self) -> None:
        if self.pinned:
            torch.cuda.cudart().cudaHostUnregister(self.buf.data_ptr())
            self.pinned = False
        self.buf = None
        try:
            self.map.close()
        except BufferError:
            pass
        if self.created:
            try:
                os.unlink(self.path)
            except OSError:
                pass


def _as_block_bytes(t: torch.Tensor) -> torch.Tensor:
    """[num_blocks, ...] cache tensor -> uint8 [num_blocks, block_bytes] view."""
    return t.view(t.shape[0], -1).view(torch.uint8)


class HostPoolKVConnector(P2PKVConnector):
    """Same scheduler / worker interface as the GPU-to-GPU connector; the data path is the
    host pool.  Extra config: ``kv_pool_slots`` (default 4096), ``kv_pool_name``."""

    def __init__(self, config: EngineConfig, device: Optional[torch.device] = None) -> None:
        super().__init__(config, device)
        extra = self.kt.kv_connector_extra_config or {}
        self.pool_slots = int(extra.get("kv_pool_slots", 4096))
        self.pool_name = str(extra.get("kv_pool_name", f"omni_b200_kv_{self.port}_{self.rank}"))
        self.pool: Optional[HostKVPool] = None
        self._remote_pools: Dict[str, HostKVPool] = {}
        self._caches: List[torch.Tensor] = []
        self._slots_of: Dict[str, List[int]] = {}
        self._saved_at: Dict[str, float] = {}
        self._copy_stream = None

    # =================================================================== worker
    def register_kv_caches(self, kv_caches) -> None:
        self._caches = flatten_kv_caches(kv_caches)
        sizes = [_as_block_bytes(t).shape[1] for t in self._caches]
        cuda = self.device.type == "cuda"
        if cuda:
            self._copy_stream = torch.cuda.Stream(self.device)
        if self.kt.is_producer and self.pool is None:
            self.pool = HostKVPool(self.pool_name, self.pool_slots, sizes, create=True, pin=cuda)
            self.server = ControlServer(self.host_ip, self.port + self.rank, self.pool.geometry, self._on_consumer_lost)
            logger.info("KV host pool %s: %d slots of %d bytes, control endpoint %s", self.pool.path,
                        self.pool.num_slots, self.pool.slot_bytes, self.server.endpoint)

    # ---- producer: blocks -> slots
    def save_blocks(self, block_ids: Sequence[int]) -> Optional[List[int]]:
        """Copy the given cache blocks into freshly allocated pool slots (None: pool full)."""
        slots = self.pool.alloc(len(block_ids))
        if slots is None:
            return None
        idx = torch.tensor(list(block_ids), dtype=torch.long, device=self.device)
        slot_idx = torch.tensor(slots, dtype=torch.long)
        cuda = self.device.type == "cuda"
        staged = []
        if cuda:
            self._copy_stream.wait_stream(torch.cuda.current_stream(self.device))
        for i, cache in enumerate(self._caches):
            rows = _as_block_bytes(cache)
            if cuda:
                with torch.cuda.stream(self._copy_stream):
                    gathered = rows.index_select(0, idx)                       # contiguous on the GPU
                    host = torch.empty(gathered.shape, dtype=torch.uint8, pin_memory=True)
                    host.copy_(gathered, non_blocking=True)
                staged.append((i, host))
            else:
                self.pool.slots_view(i)[slot_idx] = rows.index_select(0, idx)
        if cuda:
            self._copy_stream.synchronize()
            for i, host in staged:
                self.pool.slots_view(i)[slot_idx] = host
        return slots

    def request_finished(self, request, block_ids: List[int]) -> Tuple[Optional[float], Optional[Dict[str, Any]]]:
        from ..engine.request import RequestStatus
        if not self.kt.is_producer or request.status != RequestStatus.FINISHED_LENGTH_CAPPED or not block_ids:
            return None, None
        if self.pool is None:
            raise RuntimeError("HostPoolKVConnector: register_kv_caches has not run")
        slots = self.save_blocks(block_ids)
        if slots is None:
            logger.warning("KV host pool full (%d free): request %s keeps no KV for the decode instance",
                           self.pool.num_free, request.request_id)
            return None, None
        with self._lock:
            self._slots_of[request.request_id] = slots
            self._saved_at[request.request_id] = time.monotonic()
        params = dict(remote_block_ids=slots, remote_cluster_id=self.cluster_id,
                      remote_host_ip=f"tcp://{self.host_ip}:{self.port}", kv_pool=self.pool.geometry(),
                      spec_token_ids=list(getattr(request, "spec_token_ids", []) or []),
                      remote_dp_rank=self.dp_rank, remote_request_id=request.request_id)
        # the GPU blocks are free at once: the KV now lives in the pool
        return None, params

    def take_released_requests(self) -> List[str]:
        """Requests whose slots were fetched (or that waited too long): recycle their slots."""
        from .connector import BLOCK_RELEASE_DELAY_S
        done = self.server.take_pulled() if self.server is not None else []
        now = time.monotonic()
        with self._lock:
            late = [rid for rid, t in self._saved_at.items() if now - t > BLOCK_RELEASE_DELAY_S]
            for rid in set(done) | set(late):
                slots = self._slots_of.pop(rid, None)
                self._saved_at.pop(rid, None)
                if slots:
                    self.pool.free(slots)
        return []          # nothing is parked in the GPU cache

    # ---- consumer: slots -> blocks
    def _pool_for(self, geometry: Dict[str, Any]) -> HostKVPool:
        name = geometry["pool"]
        pool = self._remote_pools.get(name)
        if pool is None:
            pool = HostKVPool(name, geometry["num_slots"], geometry["tensor_block_bytes"], create=False,
                              pin=self.device.type == "cuda")
            self._remote_pools[name] = pool
        return pool

    def update_state_after_alloc(self, request, block_ids: List[int], num_external_tokens: int) -> None:
        super().update_state_after_alloc(request, block_ids, num_external_tokens)
        with self._lock:
            meta = self._pending_loads.get(request.request_id)
            if meta is not None:
                meta.pool_geometry = request.kv_transfer_params.get("kv_pool")      # type: ignore[attr-defined]

    def _load_one(self, rid: str, meta: ReqMeta) -> None:
        try:
            geometry = getattr(meta, "pool_geometry", None)
            if geometry is None:
                raise ValueError("kv_transfer_params carry no host-pool description")
            pool = self._pool_for(geometry)
            sizes = [_as_block_bytes(t).shape[1] for t in self._caches]
            if sizes != pool.tensor_block_bytes:
                raise ValueError(f"KV layout mismatch: pool {pool.tensor_block_bytes} vs local cache {sizes}")
            slot_idx = torch.tensor(meta.remote_block_ids, dtype=torch.long)
            dst = torch.tensor(meta.local_block_ids, dtype=torch.long, device=self.device)
            cuda = self.device.type == "cuda"
            ev = None
            if cuda:
                torch.cuda.set_device(self.device)
                with torch.cuda.stream(self._copy_stream):
                    for i, cache in enumerate(self._caches):
                        host = pool.slots_view(i)[slot_idx].pin_memory()
                        _as_block_bytes(cache).index_copy_(0, dst, host.to(self.device, non_blocking=True))
                    ev = torch.cuda.Event()
                    ev.record(self._copy_stream)
            else:
                for i, cache in enumerate(self._caches):
                    _as_block_bytes(cache).index_copy_(0, dst, pool.slots_view(i)[slot_idx])
            client = self._client_for(meta, 0)
            with self._lock:
                self._events[rid] = (ev, client, meta)
            if ev is None:
                self._poll_events()
        except Exception as e:
            logger.error("KV load of %s from the host pool failed: %s", rid, e)
            with self._lock:
                self._failed.add(rid)

    def close(self) -> None:
        super().close()
        for pool in self._remote_pools.values():
            pool.close()
        if self.pool is not None:
            self.pool.close()
