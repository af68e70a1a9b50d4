"""Control plane of prefill/decode disaggregation: who pulled what, and who is alive.

Producer (prefill instance) side: a ``ControlServer`` thread on a ZMQ ROUTER
socket answers

    {"type": "get_meta"}                       -> the producer's KV-cache export (IPC descriptors)
    {"type": "pulled", "request_ids": [...]}   -> blocks of these requests may be freed
    {"type": "abort",  "request_ids": [...]}   -> the consumer gave up on these requests
    {"type": "heartbeat", "cluster": id}       -> consumer is alive; reply carries the producer's beat

Consumer (decode instance) side: ``ControlClient`` (DEALER) sends those messages.
``HeartbeatMonitor`` tracks the last beat per peer with an injectable clock, so
expiry logic is testable without sleeping.  Intervals follow the reference
(5 s beats, 60 s link timeout: omni_npu/connector/llmdatadist_connector_v1.py:48-51,
heartbeat threads :335-382,:631-678).
"""
from __future__ import annotations

import pickle
import threading
import time
from typing import Any, Callable, Dict, List, Optional, Set

HEARTBEAT_INTERVAL_S = 5.0
PEER_TIMEOUT_S = 60.0


class HeartbeatMonitor:
    def __init__(self, timeout_s: float = PEER_TIMEOUT_S, clock: Callable[[], float] = time.monotonic) -> None:
        self.timeout_s = timeout_s
        self.clock = clock
        self._last: Dict[str, float] = {}
        self._lock = threading.Lock()

    def beat(self, peer: str) -> None:
        with self._lock:
            self._last[peer] = self.clock()

    def alive(self, peer: str) -> bool:
        with self._lock:
            t = self._last.get(peer)
        return t is not None and self.clock() - t <= self.timeout_s

    def expired(self) -> List[str]:
        now = self.clock()
        with self._lock:
            dead = [p for p, t in self._last.items() if now - t > self.timeout_s]
            for p in dead:
                del self._last[p]
        return dead

    def peers(self) -> List[str]:
        with self._lock:
            return list(self._last)


class ControlServer:
    """Producer-side endpoint.  ``meta_provider()`` returns the picklable KV export."""

    def __init__(self, host: str, port: int, meta_provider: Callable[[], Any],
                 on_peer_lost: Optional[Callable[[str], None]] = None,
                 monitor: Optional[HeartbeatMonitor] = None) -> None:
        import zmq
        self._zmq = zmq
        self.ctx = zmq.Context.instance()
        self.sock = self.ctx.socket(zmq.ROUTER)
        self.sock.setsockopt(zmq.LINGER, 0)
        self.port = port if port else None
        if port:
            self.sock.bind(f"tcp://{host}:{port}")
        else:
            self.port = self.sock.bind_to_random_port(f"tcp://{host}")
        self.endpoint = f"tcp://{host}:{self.port}"
        self.meta_provider = meta_provider
        self.on_peer_lost = on_peer_lost
        self.monitor = monitor or HeartbeatMonitor()
        self._pulled: Set[str] = set()
        self._aborted: Set[str] = set()
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self.thread = threading.Thread(target=self._run, name="kv-control-server", daemon=True)
        self.thread.start()

    def _run(self) -> None:
        zmq = self._zmq
        poller = zmq.Poller()
        poller.register(self.sock, zmq.POLLIN)
        while not self._stop.is_set():
            if poller.poll(200):
                try:
                    ident, payload = self.sock.recv_multipart()
                    msg = pickle.loads(payload)
                    reply = self.handle(msg)
                    self.sock.send_multipart([ident, pickle.dumps(reply)])
                except Exception as e:  # pragma: no cover - keep the server alive
                    try:
                        self.sock.send_multipart([ident, pickle.dumps({"ok": False, "error": str(e)})])
                    except Exception:
                        pass
            for peer in self.monitor.expired():
                if self.on_peer_lost is not None:
                    self.on_peer_lost(peer)

    def handle(self, msg: Dict[str, Any]) -> Dict[str, Any]:
        kind = msg.get("type")
        if kind == "get_meta":
            return {"ok": True, "meta": self.meta_provider()}
        if kind == "pulled":
            with self._lock:
                self._pulled.update(msg.get("request_ids", []))
            return {"ok": True}
        if kind == "abort":
            with self._lock:
                self._aborted.update(msg.get("request_ids", []))
                self._pulled.update(msg.get("request_ids", []))   # their blocks can go as well
            return {"ok": True}
        if kind == "heartbeat":
            self.monitor.beat(str(msg.get("cluster")))
            return {"ok": True, "beat": time.time()}
        return {"ok": False, "error": f"unknown message type {kind!r}"}

    def take_pulled(self) -> List[str]:
        with self._lock:
            out, self._pulled = list(self._pulled), set()
        return out

    def close(self) -> None:
        self._stop.set()
        self.thread.join(timeout=2)
        self.sock.close(0)


class ControlClient:
    """Consumer-side endpoint towards one producer."""

    def __init__(self, endpoint: str, cluster_id: str, timeout_ms: int = 5000) -> None:
        import zmq
        self._zmq = zmq
        self.endpoint, self.cluster_id, self.timeout_ms = endpoint, cluster_id, timeout_ms
        self.ctx = zmq.Context.instance()
        self._lock = threading.Lock()
        self._connect()

    def _connect(self) -> None:
        zmq = self._zmq
        self.sock = self.ctx.socket(zmq.DEALER)
        self.sock.setsockopt(zmq.LINGER, 0)
        self.sock.connect(self.endpoint)

    def request(self, msg: Dict[str, Any], retries: int = 1) -> Dict[str, Any]:
        zmq = self._zmq
        with self._lock:
            for attempt in range(retries + 1):
                self.sock.send(pickle.dumps(msg))
                if self.sock.poll(self.timeout_ms, zmq.POLLIN):
                    return pickle.loads(self.sock.recv())
                # no answer: drop the socket (a late reply must not be taken for the next one)
                self.sock.close(0)
                self._connect()
            raise TimeoutError(f"no reply from {self.endpoint} to {msg.get('type')}")

    def get_meta(self) -> Any:
        return self.request({"type": "get_meta"})["meta"]

    def notify_pulled(self, request_ids: List[str]) -> None:
        self.request({"type": "pulled", "request_ids": list(request_ids)})

    def notify_abort(self, request_ids: List[str]) -> None:
        self.request({"type": "abort", "request_ids": list(request_ids)})

    def heartbeat(self) -> bool:
        try:
            return bool(self.request({"type": "heartbeat", "cluster": self.cluster_id}, retries=0).get("ok"))
        except TimeoutError:
            return False

    def close(self) -> None:
        self.sock.close(0)


class HeartbeatThread:
    """Consumer-side beat sender: pings every producer it is linked to and reports
    the ones that stopped answering for longer than the timeout."""

    def __init__(self, clients: Callable[[], Dict[str, ControlClient]], on_producer_lost: Callable[[str], None],
                 interval_s: float = HEARTBEAT_INTERVAL_S, timeout_s: float = PEER_TIMEOUT_S,
                 clock: Callable[[], float] = time.monotonic) -> None:
        self.clients, self.on_lost = clients, on_producer_lost
        self.interval_s = interval_s
        self.monitor = HeartbeatMonitor(timeout_s, clock)
        self._stop = threading.Event()
        self.thread = threading.Thread(target=self._run, name="kv-heartbeat", daemon=True)

    def start(self) -> None:
        self.thread.start()

    def tick(self) -> None:
        for name, client in list(self.clients().items()):
            if name not in self.monitor.peers():
                self.monitor.beat(name)          # start the clock at first sight
            if client.heartbeat():
                self.monitor.beat(name)
        for name in self.monitor.expired():
            self.on_lost(name)

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            self.tick()

    def close(self) -> None:
        self._stop.set()
