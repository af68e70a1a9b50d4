"""Weight / KV prefetch into L2 ahead of use.

A decoder layer knows which weights the *next* kernels will stream from HBM.
``Prefetcher`` issues L2 prefetch hints for them (``csrc/mem/l2_prefetch.cu``) on a
side stream while the current kernel runs, bounded by a per-call budget in MiB (the
126 MB L2 also has to keep the running kernel's working set).  Budgets come from the
deployment plan (``KernelPlan.*_prefetch``); a budget of 0 disables that hint.

Inside CUDA-graph capture the side stream is forked from and joined to the capturing
stream, so the hint becomes a parallel branch of the graph.

Same interface as ``PrefetcherBase`` (omni_npu/v1/layers/prefetch.py:9-77): weights,
MoE expert weights, attention projections, KV-cache blocks.
"""
from __future__ import annotations

import ctypes
from pathlib import Path
from typing import Iterable, Optional

import torch

from .. import ops

_MIB = 1 << 20
_LIB: Optional[ctypes.CDLL] = None


def _lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        ops.load_extension(required=True)
        lib = ctypes.CDLL(str(Path(__file__).resolve().parent.parent / "_C.so"))
        lib.b200_l2_prefetch.argtypes = [ctypes.c_void_p, ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_void_p]
        lib.b200_l2_prefetch.restype = ctypes.c_int
        _LIB = lib
    return _LIB


def l2_prefetch(t: torch.Tensor, max_bytes: int = 0, stream: Optional[torch.cuda.Stream] = None) -> int:
    """Hint the first ``max_bytes`` (0 = all) of ``t``'s storage into L2.  Returns the
    bytes requested (0 on CPU tensors, where this is a no-op)."""
    if not t.is_cuda or t.numel() == 0:
        return 0
    nbytes = t.numel() * t.element_size()
    ptr = t.data_ptr()
    head = (-ptr) % 16                     # start at the next 16-byte boundary
    ptr, nbytes = ptr + head, nbytes - head
    if nbytes <= 0:
        return 0
    s = stream or torch.cuda.current_stream(t.device)
    rc = _lib().b200_l2_prefetch(ptr, nbytes, max_bytes, s.cuda_stream)
    if rc != 0:
        raise RuntimeError(f"l2_prefetch failed ({rc})")
    ops._count(1)
    return min(nbytes, max_bytes) if max_bytes else nbytes


class Prefetcher:
    """Per-model helper.  All methods are no-ops when disabled or on CPU."""

    def __init__(self, device: torch.device, enabled: bool = True, attn_mb: int = 32, dense_mlp_mb: int = 32,
                 expert_gate_up_mb: int = 24, expert_down_mb: int = 12, lm_head_mb: int = 48,
                 shared_gate_up_mb: int = 12, shared_down_mb: int = 6, kv_mb: int = 16) -> None:
        self.device = torch.device(device)
        self.enabled = bool(enabled) and self.device.type == "cuda"
        self.budget = dict(attn=attn_mb, dense_mlp=dense_mlp_mb, expert_gate_up=expert_gate_up_mb,
                           expert_down=expert_down_mb, lm_head=lm_head_mb, shared_gate_up=shared_gate_up_mb,
                           shared_down=shared_down_mb, kv=kv_mb)
        self.stream = torch.cuda.Stream(self.device) if self.enabled else None
        self.requested_bytes = 0

    @classmethod
    def from_plan(cls, device, plan) -> "Prefetcher":
        """``plan``: a ``KernelPlan`` (models/config_loader.py)."""
        return cls(device, plan.enable_prefetch, plan.attn_prefetch, plan.dense_mlp_prefetch,
                   plan.expert_gate_up_prefetch, plan.expert_down_prefetch, plan.lm_head_prefetch,
                   plan.shared_expert_gate_up_prefetch, plan.shared_expert_down_prefetch)

    # ------------------------------------------------------------------ core
    def _issue(self, tensors: Iterable[torch.Tensor], kind: str) -> int:
        budget = self.budget.get(kind, 0) * _MIB
        if not self.enabled or budget <= 0:
            return 0
        cur = torch.cuda.current_stream(self.device)
        self.stream.wait_stream(cur)                  # fork (a graph branch under capture)
        done = 0
        for t in tensors:
            if t is None or done >= budget:
                continue
            done += l2_prefetch(t, budget - done, self.stream)
        cur.wait_stream(self.stream)                  # join: the hint kernel itself is a few microseconds
        self.requested_bytes += done
        return done

    # --------------------------------------------------------------- by role
    def prefetch_weight(self, weight: torch.Tensor, kind: str = "dense_mlp") -> int:
        return self._issue([weight], kind)

    def prefetch_attention(self, layer) -> int:
        """The projections of an attention module (qkv / q_a / q_b / kv_a / o)."""
        names = ("qkv_proj", "q_a_proj", "q_b_proj", "q_proj", "kv_a_proj_with_mqa", "kv_b_proj", "o_proj")
        ws = [getattr(getattr(layer, n), "weight", None) for n in names if hasattr(layer, n)]
        return self._issue(ws, "attn")

    def prefetch_mlp(self, mlp) -> int:
        return self._issue([getattr(mlp.gate_up_proj, "weight", None), getattr(mlp.down_proj, "weight", None)],
                           "dense_mlp")

    def prefetch_moe(self, moe) -> int:
        """Expert weights (the slab of the first experts: routing is not known yet) and
        the shared experts."""
        n = self._issue([getattr(moe, "w13", None)], "expert_gate_up")
        n += self._issue([getattr(moe, "w2", None)], "expert_down")
        sh = getattr(moe, "shared_experts", None)
        if sh is not None:
            n += self._issue([getattr(sh.gate_up_proj, "weight", None)], "shared_gate_up")
            n += self._issue([getattr(sh.down_proj, "weight", None)], "shared_down")
        return n

    def prefetch_lm_head(self, lm_head) -> int:
        return self._issue([getattr(lm_head, "weight", None)], "lm_head")

    def prefetch_kvcache(self, kv_cache, block_ids: torch.Tensor, max_blocks: int = 64) -> int:
        """Blocks a request is about to attend over (e.g. just pulled from a prefill instance)."""
        if not self.enabled or self.budget["kv"] <= 0:
            return 0
        caches = kv_cache if isinstance(kv_cache, (tuple, list)) else (kv_cache,)
        ids = block_ids.tolist()[:max_blocks] if isinstance(block_ids, torch.Tensor) else list(block_ids)[:max_blocks]
        return self._issue([c[b] for c in caches for b in ids], "kv")
