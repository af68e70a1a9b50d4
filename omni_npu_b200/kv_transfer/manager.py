"""KV link manager: registers this instance's KV-cache tensors, exports them to
other instances on the same machine and pulls blocks from remote exports.

GPU: every cache tensor is exported through CUDA IPC (torch's storage sharing,
which handles sub-allocations of the caching allocator); the consumer maps the
producer's tensors lazily on first use ("link"), pulls blocks with the one-launch
copy kernel ``kv_p2p_copy`` on a side stream, and drops the mapping when the
producer is declared dead ("force_unlink").  CPU (tests, gloo runs): exports are
kept in an in-process registry and a pull is a tensor copy.

Counterpart of ``LLMDataDistManager`` (omni_npu/connector/llmdatadist_manager_v1.py:175-555):
``register_memory`` (:415-442), lazy ``register_link`` / ``close_link`` /
``force_unlink`` (:251-301), ``pull_kv`` with retry and link refresh (:303-361).
The cluster id packs ip, port and TP size like the reference (:538-555).
"""
from __future__ import annotations

import ipaddress
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..logger import logger

PULL_RETRIES = 2
RETRY_WAIT_S = 1.0

# in-process registry for CPU exports: cluster id -> list of tensors
_LOCAL_EXPORTS: Dict[str, List[torch.Tensor]] = {}


def make_cluster_id(ip: str, port: int, tp_size: int) -> str:
    """ip << 32 | port << 16 | tp_size, printed as a decimal string."""
    try:
        ip_int = int(ipaddress.ip_address(ip))
    except ValueError:
        ip_int = 0x7F000001
    return str((ip_int << 32) | ((port & 0xFFFF) << 16) | (tp_size & 0xFFFF))


def parse_cluster_id(cid: str) -> Tuple[str, int, int]:
    v = int(cid)
    return str(ipaddress.ip_address(v >> 32)), (v >> 16) & 0xFFFF, v & 0xFFFF


def flatten_kv_caches(kv_caches: Sequence) -> List[torch.Tensor]:
    """Per-layer caches may be tensors or tuples of tensors (K, V / latent, index key)."""
    flat: List[torch.Tensor] = []
    for c in kv_caches:
        if isinstance(c, (tuple, list)):
            flat.extend(c)
        else:
            flat.append(c)
    return flat


@dataclass
class KVExport:
    """Picklable description of one instance-rank's KV cache."""
    cluster_id: str
    rank: int
    device_type: str
    shapes: List[Tuple[int, ...]]
    dtype: str
    ipc: Optional[List[Any]] = None        # per tensor: torch storage sharing info + offset


@dataclass
class _Link:
    tensors: List[torch.Tensor]
    created: float = field(default_factory=time.monotonic)
    mappings: List[Any] = field(default_factory=list)     # IPC mappings this link opened (CUDA)


class _RemoteView:
    """A tensor-like handle on memory of another GPU mapped into this process: just what the
    copy kernel and the layout checks need (address, shape, dtype)."""

    def __init__(self, ptr: int, shape, dtype: torch.dtype) -> None:
        self._ptr, self.shape, self.dtype = ptr, torch.Size(shape), dtype

    def data_ptr(self) -> int:
        return self._ptr

    def element_size(self) -> int:
        return self.dtype.itemsize


def _raw_ipc_handle(blob: bytes) -> bytes:
    """The 64-byte cudaIpcMemHandle_t inside torch's shareable handle.  Newer torch versions
    prefix it with a format version and a type tag ('c' = plain cudaMalloc allocation,
    'e' = expandable segment, which cannot be opened with cudaIpcOpenMemHandle)."""
    if len(blob) == 64:
        return blob
    if len(blob) > 64:
        tag = blob[len(blob) - 65: len(blob) - 64]
        if tag == b"e":
            raise ConnectionError("the producer's KV cache lives in an expandable allocator segment; "
                                  "disable expandable_segments for the KV cache to share it")
        return blob[-64:]
    raise ConnectionError(f"unexpected IPC handle of {len(blob)} bytes")


def _open_ipc_exports(ipc, shapes, dtype: torch.dtype):
    """Map a producer's cache tensors on THIS rank's current device.  The handles come from
    torch's storage sharing (handle of the allocation + byte offset of the storage in it); they
    are opened with cudaIpcOpenMemHandle + lazy peer access in the current context, so kernels
    of this GPU may dereference the addresses (a mapping made in the producer device's context
    is not accessible from another GPU without peer access enabled).  One allocation is opened
    once even when several tensors live in it."""
    import ctypes

    from ..parallel.symm_mem import _lib
    lib = _lib()
    opened: Dict[bytes, int] = {}
    mappings: List[Any] = []
    views: List[_RemoteView] = []
    try:
        for (info, offset_elems, stride), shape in zip(ipc, shapes):
            handle, storage_off = _raw_ipc_handle(bytes(info[1])), int(info[3])
            want = tuple(int(x) for x in stride)
            dense = tuple(torch.empty(shape, device="meta").stride())
            if want != dense:
                raise ValueError(f"remote cache tensor is not contiguous (strides {want})")
            base = opened.get(handle)
            if base is None:
                p = ctypes.c_void_p()
                rc = lib.b200_symm_open(handle, ctypes.byref(p))
                if rc != 0:
                    raise ConnectionError(f"cudaIpcOpenMemHandle failed ({rc}); peer access between the "
                                          "two GPUs is required")
                base = p.value
                opened[handle] = base
                mappings.append(p)
            views.append(_RemoteView(base + storage_off + int(offset_elems) * dtype.itemsize, shape, dtype))
    except Exception:
        for p in mappings:
            lib.b200_symm_close(p)
        raise
    return views, mappings


class KVLinkManager:
    def __init__(self, cluster_id: str, rank: int, device: torch.device) -> None:
        self.cluster_id, self.rank, self.device = cluster_id, rank, device
        self.local: List[torch.Tensor] = []
        self.links: Dict[str, _Link] = {}
        self._lock = threading.Lock()
        self._stream: Optional[torch.cuda.Stream] = None
        self._desc_cache: Dict[str, torch.Tensor] = {}
        self.stats = {"pulls": 0, "blocks": 0, "bytes": 0, "retries": 0, "seconds": 0.0}

    # ----------------------------------------------------------------- export
    def register_memory(self, kv_caches: Sequence) -> KVExport:
        self.local = flatten_kv_caches(kv_caches)
        if not self.local:
            raise ValueError("no KV cache tensors to register")
        shapes = [tuple(t.shape) for t in self.local]
        dtype = str(self.local[0].dtype)
        if self.device.type == "cuda":
            self._stream = torch.cuda.Stream(self.device)
            ipc = []
            for t in self.local:
                st = t.untyped_storage()
                ipc.append((st._share_cuda_(), t.storage_offset(), tuple(t.stride())))
            self.export = KVExport(self.cluster_id, self.rank, "cuda", shapes, dtype, ipc)
        else:
            _LOCAL_EXPORTS[f"{self.cluster_id}/{self.rank}"] = self.local
            self.export = KVExport(self.cluster_id, self.rank, "cpu", shapes, dtype, None)
        return self.export

    # ------------------------------------------------------------------ links
    def register_link(self, export: KVExport) -> None:
        key = f"{export.cluster_id}/{export.rank}"
        with self._lock:
            if key in self.links:
                return
            if len(export.shapes) != len(self.local):
                raise ValueError(f"remote instance has {len(export.shapes)} cache tensors, local has "
                                 f"{len(self.local)}: layouts do not match")
            mappings: List[Any] = []
            if export.device_type == "cpu":
                tensors = _LOCAL_EXPORTS.get(key)
                if tensors is None:
                    raise ConnectionError(f"no export registered for {key}")
            else:
                dtype = getattr(torch, export.dtype.replace("torch.", ""))
                tensors, mappings = _open_ipc_exports(export.ipc, export.shapes, dtype)
            for mine, theirs in zip(self.local, tensors):
                if mine.shape[1:] != theirs.shape[1:] or mine.dtype != theirs.dtype:
                    raise ValueError("KV block layout differs between the two instances: "
                                     f"{tuple(mine.shape[1:])} vs {tuple(theirs.shape[1:])}")
            self.links[key] = _Link(tensors, mappings=mappings)
            self._desc_cache.pop(key, None)
            logger.info("KV link up: %s -> %s", f"{self.cluster_id}/{self.rank}", key)

    def close_link(self, cluster_id: str, rank: Optional[int] = None) -> None:
        with self._lock:
            for key in [k for k in self.links if k.split("/")[0] == cluster_id and
                        (rank is None or k.endswith(f"/{rank}"))]:
                link = self.links.pop(key)
                self._desc_cache.pop(key, None)
                if link.mappings:
                    if self._stream is not None:
                        self._stream.synchronize()           # no copy may still read the mapping
                    from ..parallel.symm_mem import _lib
                    for p in link.mappings:
                        _lib().b200_symm_close(p)
                logger.info("KV link closed: %s", key)

    def force_unlink(self, cluster_id: str) -> None:
        """Drop every mapping of a producer that stopped answering."""
        if self.device.type == "cuda" and self._stream is not None:
            self._stream.synchronize()
        self.close_link(cluster_id)

    def is_linked(self, cluster_id: str, rank: int) -> bool:
        return f"{cluster_id}/{rank}" in self.links

    # ------------------------------------------------------------------- pull
    def pull_kv(self, cluster_id: str, rank: int, remote_blocks: Sequence[int], local_blocks: Sequence[int],
                refresh: Optional[Callable[[], KVExport]] = None):
        """Copy remote blocks into local blocks for every cache tensor.  Returns a CUDA
        event (GPU) or None (CPU) that marks completion.  On failure the link is
        refreshed (``refresh()`` returns a new export) and the pull retried."""
        n = min(len(remote_blocks), len(local_blocks))
        if n == 0:
            return None
        key = f"{cluster_id}/{rank}"
        last: Optional[Exception] = None
        for attempt in range(PULL_RETRIES + 1):
            try:
                if key not in self.links:
                    if refresh is None:
                        raise ConnectionError(f"not linked to {key}")
                    self.register_link(refresh())
                return self._pull_once(key, list(remote_blocks[:n]), list(local_blocks[:n]))
            except Exception as e:   # broken mapping, layout change, producer restart
                last = e
                self.stats["retries"] += 1
                self.close_link(cluster_id, rank)
                if attempt < PULL_RETRIES:
                    time.sleep(RETRY_WAIT_S if self.device.type == "cuda" else 0.0)
        raise ConnectionError(f"pulling KV from {key} failed after {PULL_RETRIES + 1} attempts: {last}")

    def _pull_once(self, key: str, remote_blocks: List[int], local_blocks: List[int]):
        link = self.links[key]
        t0 = time.monotonic()
        nbytes = 0
        if self.device.type != "cuda":
            src = torch.tensor(remote_blocks, dtype=torch.long)
            dst = torch.tensor(local_blocks, dtype=torch.long)
            for mine, theirs in zip(self.local, link.tensors):
                mine[dst] = theirs[src]
                nbytes += mine[0].numel() * mine.element_size() * len(local_blocks)
            event = None
        else:
            from .. import ops
            desc = self._desc_cache.get(key)
            if desc is None:
                rows = [[theirs.data_ptr(), mine.data_ptr(), mine[0].numel() * mine.element_size()]
                        for mine, theirs in zip(self.local, link.tensors)]
                desc = torch.tensor(rows, dtype=torch.int64, device=self.device)
                self._desc_cache[key] = desc
            max_bytes = max(t[0].numel() * t.element_size() for t in self.local)
            nbytes = sum(t[0].numel() * t.element_size() for t in self.local) * len(local_blocks)
            src = torch.tensor(remote_blocks, dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
            dst = torch.tensor(local_blocks, dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
            self._stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._stream):
                ops.kv_p2p_copy(desc, src, dst, max_bytes)
                event = torch.cuda.Event()
                event.record(self._stream)
            src.record_stream(self._stream)
            dst.record_stream(self._stream)
        self.stats["pulls"] += 1
        self.stats["blocks"] += len(local_blocks)
        self.stats["bytes"] += nbytes
        self.stats["seconds"] += time.monotonic() - t0
        return event

    def close(self) -> None:
        for cid in {k.split("/")[0] for k in self.links}:
            self.force_unlink(cid)
        _LOCAL_EXPORTS.pop(f"{self.cluster_id}/{self.rank}", None)
