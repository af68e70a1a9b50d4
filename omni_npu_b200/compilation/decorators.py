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


# ------------------------------------------------------------------ under vLLM
def _vllm_step_has_prefill(ctx) -> bool:
    """vLLM's forward context carries per-layer attention metadata (a dict) or a single object;
    no metadata (profile run) counts as prefill."""
    md = getattr(ctx, "attn_metadata", None)
    if md is None:
        return True
    if isinstance(md, dict):
        if not md:
            return True
        md = next(iter(md.values()))
    return int(getattr(md, "num_prefills", 0) or 0) > 0


def _wrap_compiled_call(original_call: Callable, get_ctx: Callable, full_mode) -> Callable:
    @functools.wraps(original_call)
    def call(self, *args, **kwargs):
        ctx = get_ctx()
        if _vllm_step_has_prefill(ctx) or getattr(ctx, "cudagraph_runtime_mode", None) != full_mode:
            return self.forward(*args, **kwargs)                 # eager: never traced, never captured piecewise
        out = original_call(self, *args, **kwargs)
        # a compiled callable may hand back ([tensor],) instead of the tensor
        if isinstance(out, (tuple, list)) and len(out) == 1:
            inner = out[0]
            if isinstance(inner, list) and len(inner) == 1 and hasattr(inner[0], "shape"):
                inner = inner[0]
            return inner
        return out

    call._omni_prefill_bypass = True
    return call


def patch_compile_decorators(dec_module=None, get_ctx: Optional[Callable] = None, full_mode=None) -> bool:
    """Make every model class that vLLM prepares for compilation run its plain ``forward`` for
    steps that contain prefill tokens or whose graph mode is not FULL: their MoE exchange and
    variable shapes belong neither in a traced graph nor in a captured one, and on this platform
    only whole decode steps are replayed.  Wraps ``vllm.compilation.decorators.
    _support_torch_compile`` once (idempotent); returns whether a wrapper is installed.  The
    arguments exist for tests.  (reference: omni_npu/compilation/decorators.py:49-101)"""
    if dec_module is None:
        try:
            import vllm.compilation.decorators as dec_module
            from vllm.config import CUDAGraphMode
            from vllm.forward_context import get_forward_context as vllm_ctx
        except Exception:
            return False
        get_ctx = get_ctx or vllm_ctx
        full_mode = full_mode if full_mode is not None else CUDAGraphMode.FULL
    original = getattr(dec_module, "_support_torch_compile", None)
    if original is None:
        return False
    if getattr(original, "_omni_prefill_bypass", False):
        return True

    @functools.wraps(original)
    def patched(cls, *args, **kwargs):
        cls = original(cls, *args, **kwargs)
        if not getattr(cls.__call__, "_omni_prefill_bypass", False):
            cls.__call__ = _wrap_compiled_call(cls.__call__, get_ctx, full_mode)
        return cls

    patched._omni_prefill_bypass = True
    patched._omni_original = original
    dec_module._support_torch_compile = patched
    return True


def unpatch_compile_decorators(dec_module=None) -> None:
    if dec_module is None:
        try:
            import vllm.compilation.decorators as dec_module
        except Exception:
            return
    cur = getattr(dec_module, "_support_torch_compile", None)
    if getattr(cur, "_omni_prefill_bypass", False):
        dec_module._support_torch_compile = cur._omni_original
