"""KV connector for prefill/decode-disaggregated serving on one machine.

Life cycle (the same one the reference drives through vLLM's scheduler,
omni_npu/connector/llmdatadist_connector_v1.py:110-231):

producer (``kv_role=kv_producer``, runs the prompt with max_tokens=1)
  * ``request_finished``: a length-capped request keeps its blocks ("parked") and
    returns ``kv_transfer_params`` = {remote_block_ids, remote_cluster_id,
    remote_host_ip, spec_token_ids, remote_dp_rank, remote_request_id};
  * the control server collects "pulled" acks; ``take_released_requests`` hands
    them to the scheduler, which frees the parked blocks (or after
    ``BLOCK_RELEASE_DELAY`` seconds at the latest).

consumer (``kv_role=kv_consumer``)
  * ``get_num_new_matched_tokens``: a request that carries kv_transfer_params gets
    its whole prompt from the producer (block granular) and loads asynchronously;
  * ``update_state_after_alloc`` remembers the local blocks;
    ``build_connector_meta`` ships (local, remote) block lists to the worker half;
  * worker half ``start_load_kv``: lazily links to the producer rank, pulls the
    blocks GPU-to-GPU on a side stream, then acks to the producer;
  * ``is_load_finished`` / ``get_finished`` report completed loads.

Both halves of one engine process share a single connector object.
"""
from __future__ import annotations

import os
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Set, Tuple

import torch

from ..config import EngineConfig, KVTransferConfig
from ..logger import logger
from .control_plane import ControlClient, ControlServer, HeartbeatMonitor, HeartbeatThread
from .manager import KVExport, KVLinkManager, make_cluster_id
from .utils import get_config_from_dict_or_env, get_p_start_rank

BLOCK_RELEASE_DELAY_S = float(os.environ.get("BLOCK_RELEASE_DELAY", 600))


@dataclass
class ReqMeta:
    local_block_ids: List[int]
    remote_block_ids: List[int]
    remote_host: str
    remote_cluster_id: str
    remote_request_id: Optional[str]
    remote_dp_rank: int = 0
    spec_token_ids: Optional[List[int]] = None
    token_num: int = 0


@dataclass
class ConnectorMetadata:
    requests: Dict[str, ReqMeta] = field(default_factory=dict)            # consumer: loads to start
    finished_producer: Dict[str, float] = field(default_factory=dict)     # producer: finish times


class P2PKVConnector:
    def __init__(self, config: EngineConfig, device: Optional[torch.device] = None) -> None:
        kt: KVTransferConfig = config.kv_transfer
        self.config, self.kt = config, kt
        self.block_size = config.cache.block_size
        self.device = device or torch.device("cpu")
        extra = kt.kv_connector_extra_config or {}
        self.host_ip = get_config_from_dict_or_env(extra, "kv_ip", "OMNI_B200_KV_IP", kt.kv_ip)
        self.port = int(get_config_from_dict_or_env(extra, "kv_port", "OMNI_B200_KV_PORT", kt.kv_port))
        self.tp_size = config.parallel.tensor_parallel_size
        self.rank = int(os.environ.get("RANK", "0")) % max(1, self.tp_size)
        self.dp_rank = int(extra.get("dp_rank", 0))
        self.cluster_id = make_cluster_id(self.host_ip, self.port, self.tp_size)
        self.producer_tp_size = int(extra.get("kv_producer_tp_size", self.tp_size))
        self.async_pull = bool(config.additional_config.get("async_pull_kv", True))
        self.manager = KVLinkManager(self.cluster_id, self.rank, self.device)
        self._lock = threading.Lock()
        # scheduler-side state
        self._pending_loads: Dict[str, ReqMeta] = {}
        self._new_loads: Dict[str, ReqMeta] = {}
        self._finish_times: Dict[str, float] = {}
        # worker-side state
        self._events: Dict[str, Any] = {}
        self._loaded: Set[str] = set()
        self._failed: Set[str] = set()
        self._clients: Dict[str, ControlClient] = {}
        self._exports: Dict[str, Dict[int, KVExport]] = {}
        self._pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="kv-pull")
        self.server: Optional[ControlServer] = None
        self.heartbeat: Optional[HeartbeatThread] = None
        self._export: Optional[KVExport] = None

    # ================================================================ scheduler
    def get_num_new_matched_tokens(self, request, num_computed_tokens: int) -> Tuple[int, bool]:
        if not self.kt.is_consumer or not request.kv_transfer_params:
            return 0, False
        p = request.kv_transfer_params
        if not p.get("remote_block_ids"):
            return 0, False
        n_remote = len(p["remote_block_ids"]) * self.block_size
        ext = min(request.num_prompt_tokens, n_remote) - num_computed_tokens
        return max(0, ext), True

    def update_state_after_alloc(self, request, block_ids: List[int], num_external_tokens: int) -> None:
        if num_external_tokens <= 0:
            return
        p = request.kv_transfer_params
        nblk = (num_external_tokens + self.block_size - 1) // self.block_size
        meta = ReqMeta(local_block_ids=list(block_ids[:nblk]), remote_block_ids=list(p["remote_block_ids"][:nblk]),
                       remote_host=p["remote_host_ip"], remote_cluster_id=p["remote_cluster_id"],
                       remote_request_id=p.get("remote_request_id"), remote_dp_rank=p.get("remote_dp_rank", 0),
                       spec_token_ids=p.get("spec_token_ids"), token_num=num_external_tokens)
        with self._lock:
            self._new_loads[request.request_id] = meta
            self._pending_loads[request.request_id] = meta

    def build_connector_meta(self, scheduler_output) -> ConnectorMetadata:
        md = ConnectorMetadata()
        with self._lock:
            md.requests, self._new_loads = self._new_loads, {}
            md.finished_producer, self._finish_times = self._finish_times, {}
        if self.async_pull and md.requests:
            # start pulling right away instead of waiting for the next model step
            self.start_load_kv(md)
            md.requests = {}
        return md

    def request_finished(self, request, block_ids: List[int]) -> Tuple[Optional[float], Optional[Dict[str, Any]]]:
        """Returns (seconds to keep the blocks parked or None, kv_transfer_params or None)."""
        # compared by name: under vLLM the request carries vLLM's own status enum
        status = getattr(request.status, "name", str(request.status))
        if not self.kt.is_producer or status != "FINISHED_LENGTH_CAPPED" or not block_ids:
            return None, None
        with self._lock:
            self._finish_times[request.request_id] = time.monotonic()
        params = dict(remote_block_ids=list(block_ids), remote_cluster_id=self.cluster_id,
                      remote_host_ip=f"tcp://{self.host_ip}:{self.port}",
                      spec_token_ids=list(getattr(request, "spec_token_ids", []) or []),
                      remote_dp_rank=self.dp_rank, remote_request_id=request.request_id)
        return BLOCK_RELEASE_DELAY_S, params

    def take_released_requests(self) -> List[str]:
        return self.server.take_pulled() if self.server is not None else []

    def is_load_finished(self, request) -> bool:
        rid = request.request_id
        self._poll_events()
        with self._lock:
            if rid in self._failed:
                # a per-request event: forget the load so the caller's fallback (local recompute)
                # or a retry does not meet the same error again
                self._failed.discard(rid)
                self._pending_loads.pop(rid, None)
                self._new_loads.pop(rid, None)
                raise ConnectionError(f"KV load for request {rid} failed")
            if rid in self._loaded:
                self._loaded.discard(rid)
                self._pending_loads.pop(rid, None)
                return True
        return False

    # =================================================================== worker
    def register_kv_caches(self, kv_caches) -> None:
        self._export = self.manager.register_memory(kv_caches)
        if self.kt.is_producer and self.server is None and self.rank == 0 or \
                (self.kt.is_producer and self.server is None):
            port = self.port + self.rank
            self.server = ControlServer(self.host_ip, port, lambda: self._export, self._on_consumer_lost)
            logger.info("KV producer control endpoint %s (cluster %s)", self.server.endpoint, self.cluster_id)
        if self.kt.is_consumer and self.heartbeat is None:
            self.heartbeat = HeartbeatThread(lambda: dict(self._clients), self._on_producer_lost)
            self.heartbeat.start()

    def _client_for(self, meta: ReqMeta, remote_rank: int) -> ControlClient:
        base = meta.remote_host
        host, port = base.rsplit(":", 1)
        endpoint = f"{host}:{int(port) + remote_rank}"
        c = self._clients.get(endpoint)
        if c is None:
            c = ControlClient(endpoint, self.cluster_id)
            self._clients[endpoint] = c
        return c

    def start_load_kv(self, md: ConnectorMetadata) -> None:
        for rid, meta in md.requests.items():
            if self.async_pull:
                self._pool.submit(self._load_one, rid, meta)
            else:
                self._load_one(rid, meta)

    def _load_one(self, rid: str, meta: ReqMeta) -> None:
        try:
            remote_rank = get_p_start_rank(self.producer_tp_size, self.tp_size, self.rank)
            client = self._client_for(meta, remote_rank)

            def refresh() -> KVExport:
                return client.get_meta()

            if self.device.type == "cuda":
                torch.cuda.set_device(self.device)
            ev = self.manager.pull_kv(meta.remote_cluster_id, remote_rank, meta.remote_block_ids,
                                      meta.local_block_ids, refresh)
            with self._lock:
                self._events[rid] = (ev, client, meta)
            if ev is None:
                self._poll_events()
        except Exception as e:
            logger.error("KV load for %s failed: %s", rid, e)
            with self._lock:
                self._failed.add(rid)

    def _poll_events(self) -> None:
        done = []
        with self._lock:
            for rid, (ev, client, meta) in list(self._events.items()):
                if ev is None or ev.query():
                    done.append((rid, client, meta))
                    del self._events[rid]
        for rid, client, meta in done:
            # every rank of a TP group finishes its own pull; rank 0 acks for the request
            try:
                if meta.remote_request_id is not None:
                    client.notify_pulled([meta.remote_request_id])
            except Exception as e:
                logger.warning("could not ack pull of %s: %s", rid, e)
            with self._lock:
                self._loaded.add(rid)

    def get_finished(self) -> Tuple[Set[str], Set[str]]:
        """(finished sending, finished receiving) request ids since the last call."""
        self._poll_events()
        sent = set(self.take_released_requests())
        with self._lock:
            recv = set(self._loaded)
        return sent, recv

    def wait_for_layer_load(self, layer_name: str) -> None:
        """Loads are whole-request copies finished before the request is scheduled."""

    def save_kv_layer(self, layer_name: str, kv_layer, attn_metadata=None) -> None:
        """The producer's KV already lives in its cache; consumers pull it."""

    def wait_for_save(self) -> None:
        pass

    # ================================================================ liveness
    def _on_consumer_lost(self, cluster: str) -> None:
        logger.warning("KV consumer %s stopped sending heartbeats", cluster)

    def _on_producer_lost(self, endpoint: str) -> None:
        logger.warning("KV producer at %s stopped answering: dropping its links", endpoint)
        client = self._clients.pop(endpoint, None)
        if client is not None:
            client.close()
        with self._lock:
            lost = [rid for rid, m in self._pending_loads.items() if endpoint.startswith(m.remote_host.rsplit(":", 1)[0])]
            self._failed.update(lost)
        for cid in list({k.split("/")[0] for k in self.manager.links}):
            self.manager.force_unlink(cid)

    def close(self) -> None:
        if self.heartbeat is not None:
            self.heartbeat.close()
        if self.server is not None:
            self.server.close()
        self._pool.shutdown(wait=False)
        for c in self._clients.values():
            c.close()
        self.manager.close()


_INSTANCES: Dict[Tuple[int, int], P2PKVConnector] = {}
# connector names that select the host-memory pool data path (kv_transfer/host_pool.py)
HOST_POOL_NAMES = ("HostPoolKVConnector", "OmniCacheConnector")


def create_connector(config: EngineConfig, role: str, device: Optional[torch.device] = None) -> P2PKVConnector:
    """One connector per engine process, shared by its scheduler and worker halves."""
    key = (os.getpid(), id(config))
    inst = _INSTANCES.get(key)
    if inst is None:
        name = config.kv_transfer.kv_connector if config.kv_transfer is not None else None
        if name in HOST_POOL_NAMES:
            from .host_pool import HostPoolKVConnector
            inst = HostPoolKVConnector(config, device)
        else:
            inst = P2PKVConnector(config, device)
        _INSTANCES[key] = inst
    elif device is not None and inst.device.type == "cpu" and device.type == "cuda":
        inst.device = device
        inst.manager.device = device
    return inst
