"""CUDA-graph capture and replay of a whole decode step.

``CUDAGraphRunner`` captures a zero-argument callable whose inputs live in
persistent device buffers, and replays it.  ``CUDAGraphWrapper`` is the
per-batch-descriptor cache used as the platform's static-graph wrapper: it
captures on first use of a descriptor and replays afterwards, runs eagerly
for anything that must not be captured (prefill, graph mode NONE), checks in
debug mode that input addresses did not move, and keeps only weak references
to outputs.  It is the counterpart of ``ACLGraphWrapper``
(omni_npu/compilation/acl_graph.py:69-270) without its post-replay patching
of host-side arguments: lengths live in device memory here.
"""
from __future__ import annotations

import dataclasses
import os
import weakref
from typing import Any, Callable, Dict, Hashable, Optional

import torch

from .. import ops


class CUDAGraphRunner:
    def __init__(self, fn: Callable[[], Any], device: torch.device, pool=None) -> None:
        self.fn = fn
        self.device = device
        self.pool = pool
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.output = None
        self.num_kernels = 0

    def capture(self, warmup: int = 1) -> None:
        stream = torch.cuda.Stream(self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                self.fn()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        torch.cuda.synchronize(self.device)
        self.graph = torch.cuda.CUDAGraph()
        with ops.count_capture() as cc:
            with torch.cuda.graph(self.graph, pool=self.pool):
                self.output = self.fn()
        self.num_kernels = cc.kernels
        if self.pool is None:
            self.pool = self.graph.pool()

    def replay(self):
        self.graph.replay()
        ops.add_launches(self.num_kernels)
        return self.output


@dataclasses.dataclass(frozen=True)
class BatchDescriptor:
    num_tokens: int
    uniform_decode: bool = True


@dataclasses.dataclass
class _Entry:
    runner: Optional[CUDAGraphRunner] = None
    input_addresses: Optional[list] = None
    output_ref: Any = None


class CUDAGraphWrapper:
    """Callable wrapper: ``wrapper(descriptor, *args)`` captures/replays per descriptor."""

    def __init__(self, runnable: Callable, device: torch.device, runtime_mode: str = "FULL",
                 debug: Optional[bool] = None) -> None:
        self.runnable = runnable
        self.device = device
        self.runtime_mode = runtime_mode
        self.entries: Dict[Hashable, _Entry] = {}
        self.pool = None
        self.debug = bool(int(os.environ.get("OMNI_B200_GRAPH_DEBUG", "0"))) if debug is None else debug

    def __getattr__(self, name):
        # transparent access to the wrapped module's attributes
        return getattr(self.__dict__["runnable"], name)

    def __call__(self, descriptor: Optional[BatchDescriptor], *args, mode: Optional[str] = None, **kw):
        mode = mode or self.runtime_mode
        if descriptor is None or mode == "NONE" or self.device.type != "cuda":
            return self.runnable(*args, **kw)
        entry = self.entries.get(descriptor)
        if entry is None:
            entry = _Entry()
            self.entries[descriptor] = entry
        if entry.runner is None:
            runner = CUDAGraphRunner(lambda: self.runnable(*args, **kw), self.device, self.pool)
            runner.capture(warmup=1)
            self.pool = runner.pool
            entry.runner = runner
            entry.input_addresses = [a.data_ptr() for a in args if isinstance(a, torch.Tensor)]
            out = runner.output
            try:
                entry.output_ref = weakref.ref(out)
            except TypeError:
                entry.output_ref = lambda o=out: o
            return out
        if self.debug:
            now = [a.data_ptr() for a in args if isinstance(a, torch.Tensor)]
            if now != entry.input_addresses:
                raise RuntimeError(f"CUDA graph inputs moved for {descriptor}: "
                                   f"{entry.input_addresses} -> {now}")
        return entry.runner.replay()
