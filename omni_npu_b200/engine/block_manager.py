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


def chain_block_hashes(token_ids: Sequence[int], block_size: int, prev: Optional[List[bytes]] = None,
                       upto_blocks: Optional[int] = None) -> List[bytes]:
    """Content hashes of the full blocks of ``token_ids``: block i hashes (hash of block i - 1, its
    tokens), so equal hashes mean equal prefixes.  ``prev`` are hashes already known (extended in
    place and returned); a block holding a negative token id (a placeholder) ends the chain."""
    import hashlib
    import struct
    out = prev if prev is not None else []
    n = len(token_ids) // block_size
    if upto_blocks is not None:
        n = min(n, upto_blocks)
    for i in range(len(out), n):
        blk = token_ids[i * block_size: (i + 1) * block_size]
        if min(blk) < 0:
            break
        h = hashlib.blake2b(out[i - 1] if i else b"", digest_size=16)
        h.update(struct.pack(f"<{block_size}q", *blk))
        out.append(h.digest())
    return out


class BlockPool:
    """Free list of KV blocks.  With ``prefix_caching`` a block may be shared by several requests
    (reference counts) and a full block whose content hash was registered stays findable after its
    last user frees it, until the block is needed again (least recently freed first)."""

    def __init__(self, num_blocks: int, block_size: int, num_reserved: int = 0, prefix_caching: bool = False) -> None:
        if num_blocks <= num_reserved:
            raise ValueError("KV cache too small: %d blocks, %d reserved" % (num_blocks, num_reserved))
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.num_reserved = num_reserved
        self._free: List[int] = list(range(num_blocks - 1, num_reserved - 1, -1))
        self._delayed: Dict[str, Tuple[float, List[int]]] = {}
        self.prefix_caching = prefix_caching
        self._ref: Dict[int, int] = {}                 # users of a block in use (prefix caching only)
        self._hash_of: Dict[int, bytes] = {}           # block -> registered content hash
        self._block_of: Dict[bytes, int] = {}          # content hash -> block
        self._cached_free: Dict[int, None] = {}        # unused blocks that still hold registered content, oldest first

    @property
    def num_free(self) -> int:
        return len(self._free) + len(self._cached_free)

    @property
    def usage(self) -> float:
        total = self.num_blocks - self.num_reserved
        return 1.0 - self.num_free / total if total else 0.0

    def blocks_needed(self, num_tokens: int, have: int = 0) -> int:
        return max(0, (num_tokens + self.block_size - 1) // self.block_size - have)

    def can_allocate(self, n: int) -> bool:
        return n <= self.num_free

    def allocate(self, n: int) -> List[int]:
        if n > self.num_free:
            raise RuntimeError("out of KV blocks")
        while len(self._free) < n:
            # give up the content that was freed longest ago
            blk = next(iter(self._cached_free))
            del self._cached_free[blk]
            self._block_of.pop(self._hash_of.pop(blk), None)
            self._free.insert(0, blk)
        out = self._free[-n:] if n else []
        if n:
            del self._free[-n:]
        out.reverse()
        if self.prefix_caching:
            for b in out:
                self._ref[b] = 1
        return out

    def free(self, blocks: Sequence[int]) -> None:
        if not self.prefix_caching:
            self._free.extend(reversed(list(blocks)))
            return
        for b in reversed(list(blocks)):
            left = self._ref.get(b, 1) - 1
            if left > 0:
                self._ref[b] = left
                continue
            self._ref.pop(b, None)
            if b in self._hash_of:
                self._cached_free[b] = None
            else:
                self._free.append(b)

    # ---- prefix caching
    def register(self, block: int, content_hash: bytes) -> None:
        """Record that ``block`` holds the full block with this content hash (first holder wins)."""
        if not self.prefix_caching or block in self._hash_of or content_hash in self._block_of:
            return
        self._hash_of[block] = content_hash
        self._block_of[content_hash] = block

    def match_prefix(self, hashes: Sequence[bytes]) -> List[int]:
        """Blocks holding the longest cached prefix of the hash chain (not yet acquired)."""
        out: List[int] = []
        for h in hashes:
            b = self._block_of.get(h)
            if b is None:
                break
            out.append(b)
        return out

    def acquire(self, blocks: Sequence[int]) -> None:
        """Take another reference on cached blocks (in use by others, or unused but still findable)."""
        for b in blocks:
            if b in self._cached_free:
                del self._cached_free[b]
                self._ref[b] = 1
            else:
                self._ref[b] = self._ref.get(b, 0) + 1

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
