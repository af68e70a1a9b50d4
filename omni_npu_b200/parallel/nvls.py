"""All-reduce through the NVSwitch (NVLS): ``multimem.ld_reduce`` / ``multimem.st``.

The buffer comes from ``torch.distributed._symmetric_memory`` (CUDA VMM allocation, handle
exchange over the group's store, and a binding of every rank's allocation to one NVLink
multicast object); that is plumbing only.  The reduction kernels are this package's
(``csrc/comm/nvls_all_reduce.cu``): one-shot for small messages, two-shot for large ones, both
with an optional fused ``residual += sum; RMSNorm`` tail.

The switch adds the ranks' copies while the data crosses it, so each rank moves the message
over its link once (two-shot: 1/world in, 1/world out per rank and copy) whatever the world
size, where the peer-store kernels of ``symm_mem.py`` move ``world - 1`` copies.

A rank that dies while its memory is bound to a multicast object can fault the other ranks'
GPUs; failure-handling tests therefore run with ``OMNI_B200_NVLS=0``.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional

import torch

from .. import ops
from ..logger import logger

_LIB: Optional[ctypes.CDLL] = None


def _lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        ops.load_extension(required=True)
        lib = ctypes.CDLL(str(Path(__file__).resolve().parent.parent / "_C.so"))
        vp, ci, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
        lib.b200_nvls_flag_bytes.restype = sz
        lib.b200_nvls_all_reduce.argtypes = [vp, ctypes.POINTER(vp), ci, ci, sz, vp, vp, vp, vp, ctypes.c_float,
                                             ci, ci, ci, vp, vp, vp, vp]
        lib.b200_nvls_all_reduce.restype = ci
        _LIB = lib
    return _LIB


def nvls_enabled() -> bool:
    return os.environ.get("OMNI_B200_NVLS", "1") != "0"


class NvlsAllReduce:
    """bf16 all-reduce of ``[rows, h]`` tensors up to ``max_bytes`` through the switch."""

    ONE_SHOT_MAX_BYTES = int(os.environ.get("OMNI_B200_NVLS_ONE_SHOT_MAX", str(1 << 20)))

    def __init__(self, group, device: torch.device, max_bytes: int = 32 << 20) -> None:
        import torch.distributed._symmetric_memory as sm
        self.group, self.device = group, device
        self.world, self.rank = group.world_size, group.rank_in_group
        self.max_bytes = int(max_bytes)
        lib = _lib()
        self.flag_bytes = int(lib.b200_nvls_flag_bytes())
        self.half_bytes = 2 * self.max_bytes                    # input region + output region
        total = self.flag_bytes + 2 * self.half_bytes
        torch.cuda.set_device(device)
        self.buf = sm.empty(total, dtype=torch.uint8, device=device)
        self.handle = sm.rendezvous(self.buf, group.device_group)
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        if mc == 0:
            raise RuntimeError("the symmetric-memory allocation has no multicast mapping "
                               "(NVLS needs an NVSwitch system and multicast support in the driver)")
        self.mc_ptr = mc
        vp = ctypes.c_void_p
        self.peer_ptrs = (vp * 8)()
        for r, ptr in enumerate(self.handle.buffer_ptrs):
            self.peer_ptrs[r] = int(ptr)
        self.buf[: self.flag_bytes].zero_()
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.done = torch.zeros(1, dtype=torch.int32, device=device)
        self.status = ops.device_state(device).status
        torch.cuda.synchronize(device)
        group.barrier()
        logger.info("NVLS all-reduce ready: rank %d/%d, %d MiB symmetric buffer", self.rank, self.world, total >> 20)

    def fits(self, x: torch.Tensor) -> bool:
        return (x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.dim() >= 1
                and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384 and 0 < x.numel() * 2 <= self.max_bytes)

    def all_reduce(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
                   norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, mode: int = 0,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum of ``x`` over the group.  With ``residual``: ``residual += sum`` in place; with
        ``norm_weight`` the result is ``RMSNorm(residual or sum) * norm_weight``.  ``mode`` 0 picks
        one-shot up to ``ONE_SHOT_MAX_BYTES`` and two-shot above; 1 / 2 force a variant."""
        h = x.shape[-1]
        rows = x.numel() // h
        out = torch.empty_like(x) if out is None else out
        if mode == 0:
            mode = 1 if x.numel() * 2 <= self.ONE_SHOT_MAX_BYTES else 2
        rc = _lib().b200_nvls_all_reduce(
            self.mc_ptr, self.peer_ptrs, self.world, self.rank, self.half_bytes, x.data_ptr(), out.data_ptr(),
            residual.data_ptr() if residual is not None else None,
            norm_weight.data_ptr() if norm_weight is not None else None, eps, rows, h, mode,
            self.epoch.data_ptr(), self.done.data_ptr(), self.status.data_ptr(),
            torch.cuda.current_stream(self.device).cuda_stream)
        if rc != 0:
            raise RuntimeError(f"NVLS all_reduce failed ({rc})")
        ops._count(1)
        return out


def try_attach(group, device: torch.device, max_bytes: int = 32 << 20) -> Optional[NvlsAllReduce]:
    """An ``NvlsAllReduce`` for the group, or None when switched off or unsupported here."""
    if not nvls_enabled() or group.world_size < 2 or device.type != "cuda":
        return None
    try:
        return NvlsAllReduce(group, device, max_bytes)
    except Exception as e:
        logger.warning("NVLS all-reduce not available (%s): peer-store kernels and NCCL are used", e)
        return None
