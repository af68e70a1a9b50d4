"""Decorators that choose between the captured and the eager path of a model.

``support_graph_replay(cls)`` wraps ``cls.__call__`` so that a step runs through the
per-batch-size CUDA graph only when it is a uniform decode step and graphs are on; any
batch that contains prefill tokens, and everything in mode NONE, calls ``forward``
directly.  Same decision as ``_bypass_prefill`` in omni_npu/compilation/decorators.py:49-101
(where it guards a torch.compile'd callable; here the graph path is a CUDA-graph replay).
"""
from __future__ import annotations

import functools
from typing import Callable, Optional

from ..attention.metadata import get_forward_context
from .cuda_graph import BatchDescriptor, CUDAGraphWrapper


def step_is_capturable(md, mode: str) -> bool:
    return (mode != "NONE" and md is not None and not md.is_prefill
            and md.num_actual_tokens <= md.num_tokens)


def support_graph_replay(cls=None, *, mode_attr: str = "cudagraph_mode"):
    """Class decorator.  The instance needs ``device`` and (optionally) ``cudagraph_mode``."""

    def wrap(klass):
        orig_call: Callable = klass.__call__

        @functools.wraps(orig_call)
        def __call__(self, *args, **kwargs):
            try:
                md = get_forward_context().attn_metadata
            except RuntimeError:
                md = None
            mode = getattr(self, mode_attr, "FULL_DECODE_ONLY")
            if not step_is_capturable(md, mode):
                return self.forward(*args, **kwargs)            # prefill / eager mode bypass
            wrapper: Optional[CUDAGraphWrapper] = getattr(self, "_graph_wrapper", None)
            if wrapper is None:
                wrapper = CUDAGraphWrapper(lambda *a, **k: self.forward(*a, **k), self.device, "FULL")
                self._graph_wrapper = wrapper
            return wrapper(BatchDescriptor(md.num_tokens, True), *args, **kwargs)

        klass.__call__ = __call__
        klass._graph_bypass_installed = True
        return klass

    return wrap(cls) if cls is not None else wrap
