"""Coordinator of token recovery: collects fault reports and drives all workers through
stop -> recover -> continue.

Endpoints (JSON over HTTP): ``/report_failure``, ``/worker_status``,
``/report_worker_server_info``, ``/ha_msg``.  ``HAProcessor`` runs in a thread: when a new
faulty step is known it (1) pokes every worker (``/stop_device``) so that healthy ranks
leave their collectives too, (2) waits until all report ``device_force_stopped``, (3)
sends ``do_recovery``, (4) waits for ``device_restarted``, (5) sends ``keep_run`` with the
option (recompute / abort bad blocks / exit).  Timeouts turn into ``exit_retry``.

Counterpart of omni_npu/v0/token_recovery/ha_server.py:40-103 and ha_processor.py:41-211;
stdlib HTTP only (no web framework in the workers' critical path).
"""
from __future__ import annotations

import json
import threading
import time
import urllib.request
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Callable, Dict, List, Optional, Tuple

from ..logger import logger
from . import common as C


def post_json(url: str, body: dict, timeout: float = 5.0) -> Optional[dict]:
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=timeout) as r:
            data = r.read()
            return json.loads(data) if data else {}
    except Exception as e:                                  # a dead worker must not stop the coordinator
        logger.warning("POST %s failed: %s", url, e)
        return None


class JsonServer:
    """Tiny threaded HTTP server dispatching POST/GET paths to callables(dict) -> dict."""

    def __init__(self, host: str, port: int, routes: Dict[str, Callable[[dict], dict]]) -> None:
        outer = self

        class Handler(BaseHTTPRequestHandler):
            def _reply(self, code: int, obj: dict) -> None:
                data = json.dumps(obj).encode()
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)

            def _dispatch(self, body: dict) -> None:
                fn = outer.routes.get(self.path)
                if fn is None:
                    return self._reply(404, {"error": "unknown path"})
                try:
                    self._reply(200, fn(body) or {})
                except Exception as e:
                    self._reply(500, {"error": str(e)})

            def do_POST(self) -> None:   # noqa: N802
                n = int(self.headers.get("Content-Length", "0") or 0)
                raw = self.rfile.read(n) if n else b"{}"
                try:
                    body = json.loads(raw or b"{}")
                except json.JSONDecodeError:
                    return self._reply(400, {"error": "bad json"})
                self._dispatch(body)

            def do_GET(self) -> None:    # noqa: N802
                self._dispatch({})

            def log_message(self, *a) -> None:
                pass

        self.routes = routes
        self.httpd = ThreadingHTTPServer((host, port), Handler)
        self.port = self.httpd.server_address[1]
        self.thread = threading.Thread(target=self.httpd.serve_forever, daemon=True)

    def start(self) -> "JsonServer":
        self.thread.start()
        return self

    def stop(self) -> None:
        self.httpd.shutdown()
        self.httpd.server_close()


class HAProcessor:
    def __init__(self, stats: C.FaultStatistics, worker_status: Dict[str, C.WorkerStatus],
                 wait_stop_s: float = C.WORKER_WAITING_STOP_TIME,
                 wait_recovery_s: float = C.WORKER_WAITING_RECOVERY_TIME, poll_s: float = 0.05,
                 post: Callable[[str, dict], Optional[dict]] = post_json) -> None:
        self.stats = stats
        self.worker_status = worker_status
        self.worker_servers: List[str] = []
        self.wait_stop_s, self.wait_recovery_s, self.poll_s = wait_stop_s, wait_recovery_s, poll_s
        self.post = post
        self.running = False
        self.thread: Optional[threading.Thread] = None
        self.history: List[Tuple[int, str]] = []           # (step, outcome)

    def start(self) -> None:
        if self.running:
            return
        self.running = True
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def stop(self) -> None:
        self.running = False
        if self.thread is not None:
            self.thread.join(timeout=5)

    # ------------------------------------------------------------------ loop
    def _loop(self) -> None:
        while self.running:
            if not self.stats.has_new_step_fault():
                time.sleep(self.poll_s)
                continue
            step = self.stats.largest_fault_step
            try:
                outcome = self.process_fault_step(step)
            except Exception as e:       # keep serving later faults
                logger.error("token recovery of step %d failed: %s", step, e)
                outcome = "error"
            self.history.append((step, outcome))
            self.stats.update_largest_processed_step(step)

    def _broadcast(self, path: str, body: dict) -> None:
        threads = [threading.Thread(target=self.post, args=(f"http://{w}{path}", body), daemon=True)
                   for w in self.worker_servers]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=6)

    def _wait_all(self, status: str, since: float, limit: float) -> Tuple[bool, List[str]]:
        workers = list(self.worker_servers)
        missing = workers
        while time.time() - since < limit:
            have = {v.worker_server_ip for v in self.worker_status.values()
                    if v.status == status and v.timestamp >= since - limit}
            missing = [w for w in workers if w not in have]
            if not missing:
                return True, []
            time.sleep(self.poll_s)
        return False, missing

    def keep_run_option(self) -> Tuple[str, List[int]]:
        stopped = [v for v in self.worker_status.values() if v.status == C.WORKER_STATUS_DEVICE_FORCE_STOPPED]
        codes = {v.err_code for v in stopped if v.err_code}
        bad = set()
        bad_memory = False
        for v in stopped:
            bad_memory |= bool(v.bad_memory)
            bad.update(v.bad_blocks or [])
        if bad_memory:
            if -1 in bad:
                return C.OPT_EXIT, sorted(bad)          # weights (or unknown memory) are damaged
            return C.OPT_ABORT, sorted(bad)             # only these KV blocks are lost
        if codes and codes <= C.RECOMPUTABLE:
            return C.OPT_RECOMPUTE, []
        return C.OPT_EXIT, sorted(bad)

    def process_fault_step(self, step: int) -> str:
        t0 = time.time()
        logger.info("token recovery: step %d, waking %d workers", step, len(self.worker_servers))
        self._broadcast("/stop_device", {"cmd": C.HA_CMD_KEEP_RUN})
        ok, missing = self._wait_all(C.WORKER_STATUS_DEVICE_FORCE_STOPPED, t0, self.wait_stop_s)
        opt, bad = self.keep_run_option()
        self._broadcast("/update_ha_cmd", {"cmd": C.HA_CMD_RECOVERY if ok else C.HA_CMD_EXIT_RETRY,
                                           "opt": opt, "bad_blocks": bad})
        if not ok:
            logger.error("workers %s did not stop; giving up on step %d", missing, step)
            return "stop_timeout"
        t1 = time.time()
        ok, missing = self._wait_all(C.WORKER_STATUS_DEVICE_RESTARTED, t1, self.wait_recovery_s)
        self._broadcast("/update_ha_cmd", {"cmd": C.HA_CMD_KEEP_RUN if ok else C.HA_CMD_EXIT_RETRY,
                                           "opt": opt, "bad_blocks": bad})
        if not ok:
            logger.error("workers %s did not recover; giving up on step %d", missing, step)
            return "recovery_timeout"
        logger.info("token recovery of step %d finished in %.2f s (%s)", step, time.time() - t0, opt)
        return opt


class HAServer:
    """The coordinator process' state + HTTP front."""

    def __init__(self, host: str = "127.0.0.1", port: int = 4999, **processor_kw) -> None:
        self.stats = C.FaultStatistics()
        self.worker_status: Dict[str, C.WorkerStatus] = {}
        self.failures: List[C.FailureInfo] = []
        self.ha_msg: Optional[dict] = None
        self.processor = HAProcessor(self.stats, self.worker_status, **processor_kw)
        self.http = JsonServer(host, port, {
            "/report_failure": self._report_failure, "/worker_status": self._worker_status,
            "/report_worker_server_info": self._worker_info, "/ha_msg": lambda b: self.ha_msg or {},
        })
        self.port = self.http.port

    def start(self) -> "HAServer":
        self.http.start()
        self.processor.start()
        return self

    def stop(self) -> None:
        self.processor.stop()
        self.http.stop()

    def _report_failure(self, body: dict) -> dict:
        info = C.FailureInfo(**{k: v for k, v in body.items() if k in C.FailureInfo.__dataclass_fields__})
        self.failures.append(info)
        self.stats.update_by_fault(info)
        return {"ok": True}

    def _worker_status(self, body: dict) -> dict:
        st = C.WorkerStatus(**{k: v for k, v in body.items() if k in C.WorkerStatus.__dataclass_fields__})
        self.worker_status[f"{st.worker_server_ip}"] = st
        return {"ok": True}

    def _worker_info(self, body: dict) -> dict:
        addr = body.get("worker_server_ip")
        if addr and addr not in self.processor.worker_servers:
            self.processor.worker_servers.append(addr)
        return {"ok": True, "workers": len(self.processor.worker_servers)}
