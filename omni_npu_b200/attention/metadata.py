"""Per-step attention metadata and the forward context.

All length-dependent values (sequence lengths, block tables, slot mapping,
positions, query offsets) live in device tensors that the model runner owns
and rewrites in place each step, so a captured CUDA graph sees new lengths
without any host-side patching of kernel arguments.  (The reference instead
patches host-side sequence-length arguments of the captured attention ops
after every replay: omni_npu/compilation/acl_graph.py:243-265.)
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import torch


@dataclass
class AttentionMetadata:
    is_prefill: bool
    num_seqs: int                 # sequences in this step (padded size under a CUDA graph)
    num_tokens: int               # rows of the hidden-state tensor (padded size under a graph)
    max_q_len: int                # longest query in this step
    max_seq_len: int              # bound on kv length (for split planning)
    q_len: int                    # uniform query length in decode steps (1, or 1 + spec tokens)
    positions: torch.Tensor       # [num_tokens] int32 (or [3, num_tokens] for M-RoPE)
    slot_mapping: torch.Tensor    # [num_tokens] int32, -1 for padded tokens
    block_tables: torch.Tensor    # [num_seqs, max_blocks] int32
    seq_lens: torch.Tensor        # [num_seqs] int32, kv length including this step
    cu_q: torch.Tensor            # [num_seqs + 1] int32 query offsets
    num_actual_tokens: int = 0    # tokens that are not padding
    num_actual_seqs: int = 0
    extra: Dict[str, Any] = field(default_factory=dict)


class ForwardContext:
    def __init__(self, attn_metadata: Optional[AttentionMetadata], kv_caches, config=None,
                 in_graph_capture: bool = False) -> None:
        self.attn_metadata = attn_metadata
        self.kv_caches = kv_caches
        self.config = config
        self.in_graph_capture = in_graph_capture


_ctx: Optional[ForwardContext] = None


def get_forward_context() -> ForwardContext:
    if _ctx is None:
        raise RuntimeError("no forward context set")
    return _ctx


@contextlib.contextmanager
def set_forward_context(attn_metadata: Optional[AttentionMetadata], kv_caches, config=None,
                        in_graph_capture: bool = False):
    global _ctx
    prev = _ctx
    _ctx = ForwardContext(attn_metadata, kv_caches, config, in_graph_capture)
    try:
        yield _ctx
    finally:
        _ctx = prev
