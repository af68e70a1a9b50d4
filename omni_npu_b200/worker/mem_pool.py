"""Sleep mode: a tagged device-memory pool whose physical memory can be given back
and restored without invalidating the tensors that live in it.

``B200MemAllocator.get_instance().use_memory_pool(tag="weights")`` routes every
tensor allocated inside the ``with`` block through the virtual-memory allocator in
``csrc/alloc/vmm_allocator.cpp`` (a torch ``CUDAPluggableAllocator`` + ``MemPool``)
and tags it.  ``sleep(offload_tags=("weights",))`` copies the tagged allocations to
pinned host memory and releases the physical memory of every pool allocation
(untagged ones, e.g. the KV cache, are simply dropped); ``wake_up()`` maps fresh
memory at the same addresses and restores the saved bytes.

Counterpart of ``NpuMemAllocator`` (omni_npu/worker/npu_mem_pool.py:109-284); the
bookkeeping it does in Python callbacks is done natively here, so allocation and
free never take the interpreter lock.
"""
from __future__ import annotations

import ctypes
import gc
from contextlib import contextmanager
from pathlib import Path
from typing import Dict, Iterable, Optional, Sequence, Tuple, Union

import torch

from ..logger import logger

_RT_PATH = Path(__file__).resolve().parent.parent / "_runtime.so"
_RT: Optional[ctypes.CDLL] = None


def runtime_lib() -> ctypes.CDLL:
    """The host-side native runtime (``_runtime.so``), built in-tree on demand."""
    global _RT
    if _RT is None:
        if not _RT_PATH.exists():
            from .._build import build
            build()
        lib = ctypes.CDLL(str(_RT_PATH))
        ll, ci, vp, cp = ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_char_p
        lib.omni_vmm_set_driver.argtypes = [vp]
        lib.omni_vmm_set_tag.argtypes = [cp]
        lib.omni_vmm_malloc.argtypes = [ll, ci, vp]
        lib.omni_vmm_malloc.restype = vp
        lib.omni_vmm_free.argtypes = [vp, ll, ci, vp]
        lib.omni_vmm_sleep.argtypes = [ctypes.POINTER(cp), ci]
        lib.omni_vmm_sleep.restype = ll
        lib.omni_vmm_wake.argtypes = [ctypes.POINTER(cp), ci]
        lib.omni_vmm_wake.restype = ll
        lib.omni_vmm_stats.argtypes = [ctypes.POINTER(ll)]
        lib.omni_vmm_usage.argtypes = [cp]
        lib.omni_vmm_usage.restype = ll
        lib.omni_vmm_last_error.argtypes = [ctypes.c_char_p, ci]
        lib.omni_vmm_last_error.restype = ci
        _RT = lib
    return _RT


def _c_tags(tags: Sequence[str]):
    arr = (ctypes.c_char_p * max(len(tags), 1))()
    for i, t in enumerate(tags):
        arr[i] = t.encode()
    return arr, len(tags)


class B200MemAllocator:
    """Singleton: the native table is process-wide."""
    instance: Optional["B200MemAllocator"] = None
    default_tag = "default"

    @staticmethod
    def get_instance() -> "B200MemAllocator":
        if B200MemAllocator.instance is None:
            B200MemAllocator.instance = B200MemAllocator()
        return B200MemAllocator.instance

    def __init__(self) -> None:
        self.lib = runtime_lib()
        self.current_tag = self.default_tag
        self._pools: Dict[str, Tuple[object, object]] = {}
        self._sleeping = False

    # ------------------------------------------------------------------ pool
    def _allocator(self):
        alloc = torch.cuda.memory.CUDAPluggableAllocator(str(_RT_PATH), "omni_vmm_malloc", "omni_vmm_free")
        return alloc

    @contextmanager
    def use_memory_pool(self, tag: Optional[str] = None):
        """Allocate every CUDA tensor created inside the block from the sleepable pool."""
        tag = tag or self.default_tag
        assert isinstance(tag, str)
        old = self.current_tag
        self.current_tag = tag
        self.lib.omni_vmm_set_tag(tag.encode())
        if tag not in self._pools:
            alloc = self._allocator()
            pool = torch.cuda.MemPool(alloc.allocator())
            self._pools[tag] = (pool, alloc)
        pool, _ = self._pools[tag]
        try:
            with torch.cuda.use_mem_pool(pool):
                yield
        finally:
            self.current_tag = old
            self.lib.omni_vmm_set_tag(old.encode())

    # ----------------------------------------------------------- sleep / wake
    def sleep(self, offload_tags: Optional[Union[Tuple[str, ...], str]] = None) -> int:
        """Offload allocations tagged with ``offload_tags`` (default: the default tag) to
        pinned host memory, discard the rest, release all physical memory of the pool.
        Returns the bytes released."""
        if offload_tags is None:
            offload_tags = (self.default_tag,)
        elif isinstance(offload_tags, str):
            offload_tags = (offload_tags,)
        arr, n = _c_tags(tuple(offload_tags))
        released = int(self.lib.omni_vmm_sleep(arr, n))
        if released < 0:
            raise RuntimeError(f"sleep failed: {self.last_error()}")
        self._sleeping = True
        gc.collect()
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        logger.info("sleep: released %.2f GiB of device memory", released / 2**30)
        return released

    def wake_up(self, tags: Optional[Iterable[str]] = None) -> int:
        """Map memory again for allocations with one of ``tags`` (all if None) and restore
        what was offloaded.  Returns the bytes mapped."""
        arr, n = _c_tags(tuple(tags) if tags is not None else ())
        mapped = int(self.lib.omni_vmm_wake(arr, n))
        if mapped < 0:
            raise RuntimeError(f"wake_up failed: {self.last_error()}")
        self._sleeping = self.stats()["sleeping_bytes"] > 0
        return mapped

    # ------------------------------------------------------------------ info
    def get_current_usage(self, tag: Optional[str] = None) -> int:
        return int(self.lib.omni_vmm_usage(tag.encode() if tag else None))

    def stats(self) -> Dict[str, int]:
        out = (ctypes.c_longlong * 8)()
        self.lib.omni_vmm_stats(out)
        keys = ("allocations", "mapped_bytes", "sleeping_bytes", "host_backup_bytes", "mallocs", "frees",
                "sleeps", "wakes")
        return dict(zip(keys, (int(v) for v in out)))

    def last_error(self) -> str:
        buf = ctypes.create_string_buffer(128)
        code = self.lib.omni_vmm_last_error(buf, 128)
        return f"{buf.value.decode()} (driver error {code})"
