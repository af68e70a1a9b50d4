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


# ------------------------------------------------------------ dynamic wrapping by name list
_WRAPPERS = ("timer", "nvtx", "marker")


def _wrap(fn: Callable, kind: str, label: str) -> Callable:
    if kind == "timer":
        return timer(label)(fn)
    if kind == "nvtx":
        @functools.wraps(fn)
        def ranged(*a, **k):
            with nvtx_range(label):
                return fn(*a, **k)
        return ranged
    if kind == "marker":
        @functools.wraps(fn)
        def marked(*a, **k):
            marker(f"enter {label}")
            try:
                return fn(*a, **k)
            finally:
                marker(f"exit {label}")
        return marked
    raise ValueError(f"unknown trace wrapper {kind!r} (one of {_WRAPPERS})")


def apply_namelist(path: Optional[str] = None) -> int:
    """Wrap the functions named in a YAML list with a tracing wrapper, without touching their
    source.  The file (``PROFILING_NAMELIST`` when ``path`` is not given) looks like

        type: timer                  # default wrapper: timer | nvtx | marker
        targets:
          - module: omni_npu_b200.engine.scheduler:Scheduler     # module[:Class]
            function_name: schedule
          - module: omni_npu_b200.ops
            function_name: [gemm, gqa_decode]
            type: nvtx

    Returns the number of functions wrapped.  Same mechanism as the reference's name-list driven
    tracing (omni_npu/vllm_patches/patches/common/patch_trace.py:26-163)."""
    import importlib

    import yaml
    path = path or os.environ.get("PROFILING_NAMELIST")
    if not path:
        return 0
    with open(path) as f:
        spec = yaml.safe_load(f) or {}
    default = spec.get("type", "timer")
    count = 0
    for target in spec.get("targets", []):
        mod_name, _, cls_name = str(target["module"]).partition(":")
        owner = importlib.import_module(mod_name)
        if cls_name:
            owner = getattr(owner, cls_name)
        names = target["function_name"]
        for fn_name in names if isinstance(names, (list, tuple)) else [names]:
            fn = getattr(owner, fn_name)
            if getattr(fn, "_omni_traced", False):
                continue
            label = f"{mod_name}{':' + cls_name if cls_name else ''}.{fn_name}"
            wrapped = _wrap(fn, target.get("type", default), label)
            wrapped._omni_traced = True
            setattr(owner, fn_name, wrapped)
            count += 1
    if count:
        logger.info("tracing: wrapped %d functions from %s", count, path)
    return count
