"""Shared types of the token-recovery (high-availability) subsystem.

A *fault* is an exception in a worker's model step whose message carries one of the
target error codes.  Workers report faults and their recovery state to one coordinator
over HTTP/JSON; the coordinator decides, per faulty step, whether the job recomputes the
step, aborts the requests that touched bad KV blocks, or exits.

Same records and constants as omni_npu/v0/token_recovery/common.py:20-74 and the
environment switches of omni_npu/v0/token_recovery/envs.py:3-9.
"""
from __future__ import annotations

import os
import time
from dataclasses import asdict, dataclass, field
from typing import List, Optional

# commands the coordinator sends to workers
HA_CMD_KEEP_RUN = "keep_run"
HA_CMD_EXIT_RETRY = "exit_retry"
HA_CMD_RECOVERY = "do_recovery"

# worker states
WORKER_STATUS_RUNNING = "running"
WORKER_STATUS_DEVICE_FORCE_STOPPED = "device_force_stopped"
WORKER_STATUS_DEVICE_RESTARTED = "device_restarted"

# what to do with the faulty step
OPT_RECOMPUTE = "recompute"
OPT_ABORT = "abort"
OPT_EXIT = "exit"

# error codes (substrings of exception messages) that start a recovery; the ones in
# RECOMPUTABLE leave device memory intact, so the step can simply be run again
ERR_UNCORRECTABLE_MEMORY = "uncorrectable ECC error"
TARGET_ERROR_CODES = ("CUDA error: unspecified launch failure", "NCCL error", "NCCL communicator was aborted",
                      "collective operation timeout", ERR_UNCORRECTABLE_MEMORY, "device-side wait expired")
RECOMPUTABLE = {"NCCL error", "NCCL communicator was aborted", "collective operation timeout",
                "device-side wait expired"}

WORKER_WAITING_STOP_TIME = float(os.environ.get("HA_WAIT_STOP_S", "100"))
WORKER_WAITING_RECOVERY_TIME = float(os.environ.get("HA_WAIT_RECOVERY_S", "10"))


@dataclass
class HAEnv:
    use_ha: bool = False
    ha_server_ip: str = "127.0.0.1"
    ha_port: int = 4999

    @classmethod
    def from_environ(cls, env=None) -> "HAEnv":
        env = os.environ if env is None else env
        return cls(env.get("USE_HA", "0") == "1",
                   env.get("HA_SERVER_IP", env.get("VLLM_DP_MASTER_IP", "127.0.0.1")),
                   int(env.get("HA_PORT", "4999")))


@dataclass
class FailureInfo:
    error_code: Optional[str] = None
    error_msg: Optional[str] = None
    actor_name: Optional[str] = None
    rank: Optional[int] = None
    local_rank: Optional[int] = None
    node_ip: Optional[str] = None
    step_count: Optional[int] = None
    timestamp: float = field(default_factory=time.time)

    def to_json(self) -> dict:
        return asdict(self)


@dataclass
class WorkerStatus:
    worker_server_ip: Optional[str] = None      # "ip:port" of the worker's command endpoint
    rank: Optional[int] = None
    local_rank: Optional[int] = None
    status: Optional[str] = None
    err_code: Optional[str] = None
    bad_memory: Optional[bool] = None           # an uncorrectable memory error was seen
    bad_blocks: Optional[List[int]] = None      # KV blocks it hit; [-1] = weights / unknown
    timestamp: float = field(default_factory=time.time)

    def to_json(self) -> dict:
        return asdict(self)


class FaultStatistics:
    """Which faulty steps have been seen and which have been dealt with."""

    def __init__(self) -> None:
        self.largest_fault_step = -1
        self.largest_processed_step = -1

    def update_by_fault(self, info: FailureInfo) -> None:
        if info and info.step_count is not None and info.step_count > self.largest_fault_step:
            self.largest_fault_step = info.step_count

    def update_largest_processed_step(self, step: int) -> None:
        self.largest_processed_step = step

    def has_new_step_fault(self) -> bool:
        return self.largest_fault_step - self.largest_processed_step >= 1

    def __str__(self) -> str:
        return f"fault step {self.largest_fault_step}, processed {self.largest_processed_step}"
