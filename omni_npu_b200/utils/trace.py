"""Tracing helpers: NVTX ranges, wall/device timers and request life-cycle log lines.

``timer`` / ``marker`` / ``nvtx_range`` wrap functions or code blocks; they cost nothing
when tracing is off (``OMNI_B200_TRACE=0``, the default).  ``RequestTracer`` writes one
line per life-cycle event of a request (arrive, scheduled, first token, finished, KV pulled)
in a fixed ``key=value`` format that log scrapers can join across prefill and decode
instances.  The reference gets the same from its external ``omni_trace`` package through
patches (omni_npu/vllm_patches/patches/common/patch_trace.py:60-209).
"""
from __future__ import annotations

import contextlib
import functools
import os
import threading
import time
from collections import defaultdict
from typing import Callable, Dict, Optional

import torch

from ..logger import logger

_ENABLED = os.environ.get("OMNI_B200_TRACE", "0") == "1"
_stats: Dict[str, list] = defaultdict(lambda: [0, 0.0])
_lock = threading.Lock()


def enabled() -> bool:
    return _ENABLED


def enable(on: bool = True) -> None:
    global _ENABLED
    _ENABLED = bool(on)


@contextlib.contextmanager
def nvtx_range(name: str):
    """An NVTX range (visible to profilers) around a block; no-op off-GPU or when disabled."""
    if _ENABLED and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def timer(name: Optional[str] = None, sync: bool = False) -> Callable:
    """Decorator: accumulate wall time per name (optionally after a device sync)."""

    def deco(fn):
        label = name or fn.__qualname__

        @functools.wraps(fn)
        def wrapper(*a, **k):
            if not _ENABLED:
                return fn(*a, **k)
            t0 = time.perf_counter()
            with nvtx_range(label):
                out = fn(*a, **k)
            if sync and torch.cuda.is_available():
                torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            with _lock:
                s = _stats[label]
                s[0] += 1
                s[1] += dt
            return out

        return wrapper

    return deco


def marker(message: str) -> None:
    if _ENABLED:
        if torch.cuda.is_available():
            torch.cuda.nvtx.mark(message)
        logger.info("trace marker: %s", message)


def timer_report(reset: bool = False) -> Dict[str, Dict[str, float]]:
    with _lock:
        out = {k: {"calls": v[0], "total_s": v[1], "mean_ms": 1e3 * v[1] / max(v[0], 1)} for k, v in _stats.items()}
        if reset:
            _stats.clear()
    return out


class RequestTracer:
    """``trace(event, request_id, **fields)`` -> one log line ``<<<Action: ...>>>``-free,
    plain ``key=value`` format with a monotonic timestamp and the role of this instance."""

    def __init__(self, role: Optional[str] = None, sink: Optional[Callable[[str], None]] = None) -> None:
        self.role = role or os.environ.get("ROLE", "hybrid")
        self.sink = sink or (lambda line: logger.info("%s", line))

    def trace(self, event: str, request_id: str, **fields) -> str:
        parts = [f"event={event}", f"request_id={request_id}", f"role={self.role}", f"ts={time.time():.6f}"]
        parts += [f"{k}={v}" for k, v in fields.items()]
        line = " ".join(parts)
        if _ENABLED:
            self.sink(line)
        return line
