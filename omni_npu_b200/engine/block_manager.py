"""Paged KV-cache block bookkeeping (host side).

A block holds ``block_size`` tokens of every layer's KV.  Blocks are handed
out from a LIFO free list; optional reserved blocks at the front of the pool
are never handed out (used for static attention-sink tokens, which the
reference implements by popping sink blocks from vLLM's free queue:
omni_npu/vllm_patches/patches/models/pangu_sink_swa_mla/patch_single_type_kv_cache_manager.py:26-62).
Blocks released by a finished PD-producer request can be parked for a delay
so a remote consumer can still pull them
(omni_npu/connector/llmdatadist_connector_v1.py:402-416).
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional, Sequence, Tuple


class BlockPool:
    def __init__(self, num_blocks: int, block_size: int, num_reserved: int = 0) -> None:
        if num_blocks <= num_reserved:
            raise ValueError("KV cache too small: %d blocks, %d reserved" % (num_blocks, num_reserved))
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.num_reserved = num_reserved
        self._free: List[int] = list(range(num_blocks - 1, num_reserved - 1, -1))
        self._delayed: Dict[str, Tuple[float, List[int]]] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def usage(self) -> float:
        total = self.num_blocks - self.num_reserved
        return 1.0 - len(self._free) / total if total else 0.0

    def blocks_needed(self, num_tokens: int, have: int = 0) -> int:
        return max(0, (num_tokens + self.block_size - 1) // self.block_size - have)

    def can_allocate(self, n: int) -> bool:
        return n <= len(self._free)

    def allocate(self, n: int) -> List[int]:
        if n > len(self._free):
            raise RuntimeError("out of KV blocks")
        out = self._free[-n:] if n else []
        if n:
            del self._free[-n:]
        out.reverse()
        return out

    def free(self, blocks: Sequence[int]) -> None:
        self._free.extend(reversed(list(blocks)))

    # ---- delayed release (PD producer side)
    def park(self, key: str, blocks: Sequence[int], delay_s: float, now: Optional[float] = None) -> None:
        now = time.monotonic() if now is None else now
        self._delayed[key] = (now + delay_s, list(blocks))

    def release_parked(self, key: str) -> bool:
        item = self._delayed.pop(key, None)
        if item is None:
            return False
        self.free(item[1])
        return True

    def expire_parked(self, now: Optional[float] = None) -> List[str]:
        now = time.monotonic() if now is None else now
        expired = [k for k, (t, _) in self._delayed.items() if t <= now]
        for k in expired:
            self.release_parked(k)
        return expired

    @property
    def num_parked(self) -> int:
        return len(self._delayed)
