"""Worker side of token recovery.

``HAWorkerAgent`` owns the worker's command endpoint (``/update_ha_cmd``,
``/stop_device``) and the client calls to the coordinator.  ``token_recover_wrapper``
wraps a worker's ``execute_model``: when the step raises an exception whose message
carries a target error code, the worker reports the fault, stops its device work
(``worker.stop_device()``), waits for ``do_recovery``, rebuilds its communicators
(``worker.restart_device()`` + ``worker.reinit_process_group()``), reports
``device_restarted``, waits for ``keep_run`` and returns ``{"opt": ..., "abort_reqs":
[...]}`` in place of the step's tokens; the engine then recomputes the step or aborts the
requests that used damaged KV blocks.  Two faults in a row are not survived.

Failures are detected on the host (an exception from the step); nothing here makes a
device fault on purpose.  Counterpart of omni_npu/v0/token_recovery/ha_monitor.py:52-279,
ha_worker_server.py:30-89 and ha_patches.py:25-90.
"""
from __future__ import annotations

import functools
import threading
import time
from typing import Callable, List, Optional

from ..logger import logger
from . import common as C
from .server import JsonServer, post_json


class HAWorkerAgent:
    def __init__(self, env: C.HAEnv, rank: int, local_rank: int = 0, host: str = "127.0.0.1", port: int = 0,
                 post: Callable[[str, dict], Optional[dict]] = post_json) -> None:
        self.env, self.rank, self.local_rank = env, rank, local_rank
        self.post = post
        self.cmd: Optional[str] = None
        self.opt: str = C.OPT_RECOMPUTE
        self.bad_blocks: List[int] = []
        self.event = threading.Event()
        self.stop_requested = threading.Event()
        self.recompute_pending = False
        self.step = 0
        self.http = JsonServer(host, port, {"/update_ha_cmd": self._update_cmd, "/stop_device": self._stop_device})
        self.address = f"{host}:{self.http.port}"

    # ---------------------------------------------------------------- server
    def start(self) -> "HAWorkerAgent":
        self.http.start()
        self.post(self._url("/report_worker_server_info"), {"worker_server_ip": self.address})
        return self

    def stop(self) -> None:
        self.http.stop()

    def _update_cmd(self, body: dict) -> dict:
        self.cmd, self.opt = body.get("cmd"), body.get("opt", C.OPT_RECOMPUTE)
        self.bad_blocks = list(body.get("bad_blocks") or [])
        self.event.set()
        return {"ok": True}

    def _stop_device(self, body: dict) -> dict:
        # a healthy rank is told that a peer failed: it must leave its collective too
        self.stop_requested.set()
        return {"ok": True}

    # ---------------------------------------------------------------- client
    def _url(self, path: str) -> str:
        return f"http://{self.env.ha_server_ip}:{self.env.ha_port}{path}"

    def report_fault(self, code: str, msg: str) -> None:
        self.post(self._url("/report_failure"), C.FailureInfo(
            error_code=code, error_msg=msg[:2000], actor_name=f"worker-{self.rank}", rank=self.rank,
            local_rank=self.local_rank, node_ip=self.address.split(":")[0], step_count=self.step).to_json())

    def report_status(self, status: str, code: Optional[str] = None, bad_memory: Optional[bool] = None,
                      bad_blocks: Optional[List[int]] = None) -> None:
        self.post(self._url("/worker_status"), C.WorkerStatus(
            worker_server_ip=self.address, rank=self.rank, local_rank=self.local_rank, status=status,
            err_code=code, bad_memory=bad_memory, bad_blocks=bad_blocks).to_json())

    def wait_cmd(self, timeout: float) -> Optional[str]:
        if self.event.wait(timeout):
            self.event.clear()
            return self.cmd
        return None


def matching_error_code(msg: str) -> Optional[str]:
    for code in C.TARGET_ERROR_CODES:
        if code in msg:
            return code
    return None


def bad_kv_blocks(worker, code: str):
    """(memory damaged?, KV blocks affected).  Only an uncorrectable-memory error can lose
    data; the worker may implement ``find_bad_kv_blocks()`` (address ranges from the driver's
    error records against its KV tensors); without it the damage is treated as unknown."""
    if code != C.ERR_UNCORRECTABLE_MEMORY:
        return False, []
    finder = getattr(worker, "find_bad_kv_blocks", None)
    if finder is None:
        return True, [-1]
    blocks = list(finder())
    return True, blocks if blocks else [-1]


def token_recover_wrapper(func):
    """Decorator for ``Worker.execute_model(self, scheduler_output)``; ``self.ha_agent`` is
    the worker's :class:`HAWorkerAgent` (None / absent = feature off)."""

    @functools.wraps(func)
    def wrapper(self, *args, **kwargs):
        agent: Optional[HAWorkerAgent] = getattr(self, "ha_agent", None)
        if agent is None or not agent.env.use_ha:
            return func(self, *args, **kwargs)
        try:
            if agent.stop_requested.is_set():
                agent.stop_requested.clear()
                raise RuntimeError("collective operation timeout: a peer rank reported a fault")
            result = func(self, *args, **kwargs)
            agent.recompute_pending = False
            return result
        except Exception as origin:
            msg = str(origin)
            code = matching_error_code(msg)
            if code is None:
                raise
            if agent.recompute_pending:
                logger.error("rank %d: a second fault while recomputing is not survivable", agent.rank)
                raise
            agent.step += 1
            try:
                agent.report_fault(code, msg)
                self.stop_device()
                bad_mem, blocks = bad_kv_blocks(self, code)
                agent.report_status(C.WORKER_STATUS_DEVICE_FORCE_STOPPED, code, bad_mem, blocks)
                if agent.wait_cmd(C.WORKER_WAITING_STOP_TIME) != C.HA_CMD_RECOVERY:
                    raise origin
                t0 = time.time()
                self.restart_device()
                self.reinit_process_group()
                logger.info("rank %d: local recovery took %.2f s", agent.rank, time.time() - t0)
                agent.report_status(C.WORKER_STATUS_DEVICE_RESTARTED)
                if agent.wait_cmd(C.WORKER_WAITING_RECOVERY_TIME) != C.HA_CMD_KEEP_RUN:
                    raise origin
                if agent.opt == C.OPT_EXIT:
                    raise origin
                if agent.opt == C.OPT_RECOMPUTE:
                    agent.recompute_pending = True
                agent.stop_requested.clear()     # the poke that accompanied this fault is spent
                return {"opt": agent.opt, "bad_blocks": list(agent.bad_blocks)}
            except Exception as new:
                if new is not origin:
                    logger.error("rank %d: recovery failed: %s", agent.rank, new)
                raise origin
            finally:
                agent.cmd = None

    return wrapper
