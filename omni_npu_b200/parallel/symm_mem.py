"""Symmetric (peer-mapped) device memory for a process group and the collectives
built on it.

Every rank allocates one data buffer and one signal pad with ``cudaMalloc``,
exports CUDA IPC handles, exchanges them over the group's CPU (gloo) side and
maps every peer's buffers.  The kernels in ``csrc/comm/symm_collectives.cu``
then read and write peer memory directly over NVLink / NVSwitch:

* ``all_reduce``  one-shot for small messages, two-shot for large ones, with an
  optional fused ``residual += x; RMSNorm`` tail (the op that follows every
  row-parallel projection in a decoder layer);
* ``all_gather`` / ``reduce_scatter`` along dim 0 for the token-sharded
  (sequence-parallel) residual stream.

NCCL stays the fallback for anything these kernels do not cover (other dtypes,
messages larger than the buffer, point-to-point).
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
        vp, ci, sz, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_longlong
        lib.b200_symm_alloc.argtypes = [sz, ctypes.POINTER(vp), ctypes.c_char_p]
        lib.b200_symm_alloc.restype = ci
        lib.b200_symm_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
        lib.b200_symm_open.restype = ci
        lib.b200_symm_close.argtypes = [vp]
        lib.b200_symm_free.argtypes = [vp]
        lib.b200_symm_signal_words.restype = ci
        pp = ctypes.POINTER(vp)
        lib.b200_symm_all_reduce.argtypes = [pp, pp, ci, ci, sz, vp, vp, ll, vp, vp, ci, ctypes.c_float,
                                             ci, vp, vp, vp]
        lib.b200_symm_all_reduce.restype = ci
        lib.b200_symm_all_gather.argtypes = [pp, pp, ci, ci, sz, vp, vp, ll, vp, vp, vp]
        lib.b200_symm_all_gather.restype = ci
        lib.b200_symm_reduce_scatter.argtypes = [pp, pp, ci, ci, sz, vp, vp, ll, vp, vp, vp]
        lib.b200_symm_reduce_scatter.restype = ci
        lib.b200_symm_ll_arm.argtypes = [vp, ll, vp]
        lib.b200_symm_ll_arm.restype = ci
        lib.b200_symm_all_reduce_ll.argtypes = [pp, ci, ci, ll, vp, vp, vp, ll, vp, vp, ci, ctypes.c_float, vp, vp, vp]
        lib.b200_symm_all_reduce_ll.restype = ci
        lib.b200_gemm_all_reduce.argtypes = [vp, vp, vp, vp, vp, vp, ctypes.c_float, ci, ci, ci, ci, ci, ci, pp, ci, ci,
                                             ll, vp, vp, vp, ci, vp]
        lib.b200_gemm_all_reduce.restype = ci
        lib.b200_symm_wait_probe.argtypes = [vp, ctypes.c_uint, ctypes.c_uint, vp, vp, vp]
        lib.b200_symm_wait_probe.restype = ci
        lib.b200_symm_epoch_word.restype = ci
        lib.b200_symm_ag_flag_word.restype = ci
        lib.b200_symm_ag_stage.argtypes = [pp, pp, ci, ci, sz, vp, vp, ll, vp, vp, vp]
        lib.b200_symm_ag_stage.restype = ci
        lib.b200_gemm_all_gather.argtypes = [vp, pp, ll, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ci, ci, ci, vp,
                                             ci, vp]
        lib.b200_gemm_all_gather.restype = ci
        lib.b200_gemm_reduce_scatter_push.argtypes = [vp, vp, vp, ci, ci, ci, ci, ci, pp, vp, ll, ci, ci, ci, vp, ci, vp]
        lib.b200_gemm_reduce_scatter_push.restype = ci
        lib.b200_symm_rs_reduce.argtypes = [pp, pp, ci, ci, sz, vp, ll, ci, vp, vp, ctypes.c_float, vp, vp, vp]
        lib.b200_symm_rs_reduce.restype = ci
        _LIB = lib
    return _LIB


class SymmetricMemory:
    ONE_SHOT_FUSED_MAX_BYTES = 2 << 20      # above this the fused one-shot tail is not worth it

    LL_SLOT_BYTES = 2 << 20                 # largest message of the push ("LL") all-reduce

    def __init__(self, group, device: torch.device, half_bytes: int = 80 << 20) -> None:
        self.group = group
        self.device = device
        self.world = group.world_size
        self.rank = group.rank_in_group
        self.half_bytes = int(half_bytes)
        lib = _lib()
        torch.cuda.set_device(device)
        self._own = []
        self._opened = []

        def alloc(nbytes: int):
            ptr = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(64)
            # at least one 2 MiB page per allocation: the IPC handle then names exactly this buffer
            rc = lib.b200_symm_alloc(max(nbytes, 2 << 20), ctypes.byref(ptr), handle)
            if rc != 0:
                raise RuntimeError(f"symmetric memory allocation of {nbytes} bytes failed ({rc})")
            self._own.append(ptr)
            return ptr, handle.raw

        data_ptr, data_h = alloc(2 * self.half_bytes)
        sig_ptr, sig_h = alloc(lib.b200_symm_signal_words() * 4)
        # receive buffer of the push all-reduce: [3 slots][world sources][LL_SLOT_BYTES]
        self.ll_slot_vecs = self.LL_SLOT_BYTES // 16
        ll_total_vecs = 3 * self.world * self.ll_slot_vecs
        ll_ptr, ll_h = alloc(ll_total_vecs * 16)
        everyone = group.all_gather_object((data_h, sig_h, ll_h))
        vp = ctypes.c_void_p
        self.data_ptrs = (vp * 8)()
        self.signal_ptrs = (vp * 8)()
        self.ll_ptrs = (vp * 8)()
        for r, (dh, sh, lh) in enumerate(everyone):
            if r == self.rank:
                self.data_ptrs[r], self.signal_ptrs[r], self.ll_ptrs[r] = data_ptr.value, sig_ptr.value, ll_ptr.value
                continue
            for handle, table in ((dh, self.data_ptrs), (sh, self.signal_ptrs), (lh, self.ll_ptrs)):
                p = vp()
                rc = lib.b200_symm_open(handle, ctypes.byref(p))
                if rc != 0:
                    raise RuntimeError(f"cudaIpcOpenMemHandle failed for rank {r} ({rc}); "
                                       "peer access between the GPUs is required")
                table[r] = p.value
                self._opened.append(p)
        self.done = torch.zeros(4, dtype=torch.int32, device=device)
        self.ll_meta = torch.zeros(4, dtype=torch.int32, device=device)      # epoch + per-slot fill counts
        self.ll_done = torch.zeros(4, dtype=torch.int32, device=device)
        self.use_ll = os.environ.get("OMNI_B200_SYMM_LL", "1") != "0"
        self.fuse_gemm = os.environ.get("OMNI_B200_FUSE_GEMM_AR", "1") != "0"
        self.fuse_ag_gemm = os.environ.get("OMNI_B200_FUSE_AG_GEMM", "1") != "0"
        self.ag_ready = torch.zeros(8, dtype=torch.int32, device=device)    # per-source arrival counters
        self.status = ops.device_state(device).status
        if lib.b200_symm_ll_arm(ll_ptr, ll_total_vecs, self._stream()) != 0:
            raise RuntimeError("arming the push all-reduce buffer failed")
        torch.cuda.synchronize(device)
        group.barrier()
        logger.info("symmetric memory ready: rank %d/%d, %d MiB per rank", self.rank, self.world,
                    (2 * self.half_bytes) >> 20)

    # ------------------------------------------------------------------ helpers
    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _ok(self, x: torch.Tensor) -> bool:
        return (x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.numel() % 8 == 0
                and x.numel() > 0)

    # Largest message the peer-memory all-reduce kernels take; larger ones go to NCCL.  Chosen by
    # measurement, not by what fits the buffer: the push / one-shot kernels win for small messages
    # (1 MiB on 2 GPUs: 23.7 us against NCCL's 25.8 us), the two-shot kernel loses for large ones
    # (64 MiB on 2 GPUs: 424 us against 154 us; NCCL reduces inside the switch).
    # OMNI_B200_SYMM_AR_MAX_BYTES overrides it.
    ALL_REDUCE_MAX_BYTES = int(os.environ.get("OMNI_B200_SYMM_AR_MAX_BYTES", str(2 << 20)))

    def can_all_reduce(self, x: torch.Tensor) -> bool:
        nbytes = x.numel() * 2
        return (self._ok(x) and nbytes <= self.ALL_REDUCE_MAX_BYTES
                and nbytes * (1 + 1.0 / self.world) + 64 <= self.half_bytes)

    # --------------------------------------------------------------- collectives
    def _ll(self, x: torch.Tensor, out: torch.Tensor, residual, weight, h: int, eps: float) -> None:
        rc = _lib().b200_symm_all_reduce_ll(self.ll_ptrs, self.world, self.rank, self.ll_slot_vecs,
                                            self.ll_meta.data_ptr(), x.data_ptr(), out.data_ptr(), x.numel(),
                                            residual.data_ptr() if residual is not None else None,
                                            weight.data_ptr() if weight is not None else None, h, eps,
                                            self.ll_done.data_ptr(), self.status.data_ptr(), self._stream())
        if rc != 0:
            raise RuntimeError(f"symm push all_reduce failed ({rc})")
        ops._count(1)

    def all_reduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, mode: int = 0) -> torch.Tensor:
        """Sum over the group.  Returns a new tensor (``out`` if given).  ``mode``: 0 auto,
        1 one shot (pull), 2 two shot, 3 push (data-carried flags, no barrier)."""
        out = torch.empty_like(x) if out is None else out
        if mode == 3 or (mode == 0 and self.use_ll and x.numel() * 2 <= self.LL_SLOT_BYTES):
            self._ll(x, out, None, None, 0, 0.0)
            return out
        rc = _lib().b200_symm_all_reduce(self.data_ptrs, self.signal_ptrs, self.world, self.rank,
                                         self.half_bytes, x.data_ptr(), out.data_ptr(), x.numel(), None,
                                         None, 0, 0.0, mode, self.done.data_ptr(),
                                         self.status.data_ptr(), self._stream())
        if rc != 0:
            raise RuntimeError(f"symm all_reduce failed ({rc})")
        ops._count(1)
        return out

    def all_reduce_add_rms_norm(self, x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                                eps: float) -> torch.Tensor:
        """residual += all_reduce(x) (in place); returns RMSNorm(residual) * weight.
        Small messages run as ONE kernel; large ones as two-shot reduce + add/norm."""
        h = x.shape[-1]
        if (self.use_ll and x.numel() * 2 <= self.LL_SLOT_BYTES and h <= 16384 and residual.is_contiguous()
                and weight.is_contiguous()):
            out = torch.empty_like(x)
            self._ll(x, out, residual, weight, h, eps)
            return out
        if (x.numel() * 2 <= self.ONE_SHOT_FUSED_MAX_BYTES and h <= 16384 and residual.is_contiguous()
                and weight.is_contiguous()):
            out = torch.empty_like(x)
            rc = _lib().b200_symm_all_reduce(self.data_ptrs, self.signal_ptrs, self.world, self.rank,
                                             self.half_bytes, x.data_ptr(), out.data_ptr(), x.numel(),
                                             residual.data_ptr(), weight.data_ptr(), h, eps, 1,
                                             self.done.data_ptr(), self.status.data_ptr(), self._stream())
            if rc != 0:
                raise RuntimeError(f"symm fused all_reduce failed ({rc})")
            ops._count(1)
            return out
        y = self.all_reduce(x)
        return ops.fused_add_rms_norm(y, residual, weight, eps)

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """Concatenate every rank's ``x`` along dim 0."""
        out = torch.empty((self.world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        rc = _lib().b200_symm_all_gather(self.data_ptrs, self.signal_ptrs, self.world, self.rank,
                                         self.half_bytes, x.data_ptr(), out.data_ptr(), x.numel(),
                                         self.done.data_ptr(), self.status.data_ptr(), self._stream())
        if rc != 0:
            raise RuntimeError(f"symm all_gather failed ({rc})")
        ops._count(1)
        return out

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        """Sum over the group, rank r keeps rows [r*n, (r+1)*n) of dim 0."""
        assert x.shape[0] % self.world == 0
        n = x.shape[0] // self.world
        out = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        rc = _lib().b200_symm_reduce_scatter(self.data_ptrs, self.signal_ptrs, self.world, self.rank,
                                             self.half_bytes, x.data_ptr(), out.data_ptr(), out.numel(),
                                             self.done.data_ptr(), self.status.data_ptr(), self._stream())
        if rc != 0:
            raise RuntimeError(f"symm reduce_scatter failed ({rc})")
        ops._count(1)
        return out

    def can_fuse_gemm(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        """The one-kernel GEMM + all-reduce handles bf16 problems whose output fits one slot of the
        push buffer and whose K is short enough to need no split-K (decode-sized M)."""
        m, n = x.shape[0], w.shape[0]
        return (self.use_ll and self.fuse_gemm and x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and x.dim() == 2 and x.stride(1) == 1 and w.is_contiguous() and n % 8 == 0 and m <= 256
                and m * n * 2 <= self.LL_SLOT_BYTES and x.shape[1] <= 8192)

    def gemm_all_reduce(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                        residual: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
                        eps: float = 0.0, bn: int = 0) -> torch.Tensor:
        """Row-parallel projection of a tensor-parallel layer as ONE kernel: every rank computes
        its partial ``x @ w.T``, the GEMM epilogue pushes the tiles into all ranks' receive
        buffers, and the same kernel reduces the rows as they arrive.  With ``norm_weight``:
        ``residual += sum`` (in place) and the result is ``RMSNorm(residual) * norm_weight``;
        without: the result is ``sum (+ residual)``."""
        m, k = x.shape
        n = w.shape[0]
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
        # bn = 0: the kernel plans tile width / cluster split-K like the stand-alone decode GEMM
        rc = _lib().b200_gemm_all_reduce(
            x.data_ptr(), w.data_ptr(), out.data_ptr(), bias.data_ptr() if bias is not None else None,
            residual.data_ptr() if residual is not None else None,
            norm_weight.data_ptr() if norm_weight is not None else None, eps, m, n, k, x.stride(0), w.stride(0), bn,
            self.ll_ptrs, self.world, self.rank, self.ll_slot_vecs, self.ll_meta.data_ptr(), self.ll_done.data_ptr(),
            self.status.data_ptr(), 0, self._stream())
        if rc != 0:
            raise RuntimeError(f"fused gemm + all_reduce failed ({rc})")
        ops._count(1)
        return out

    # ------------------------------------------------- fused all-gather -> GEMM
    def can_all_gather_gemm(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        """bf16, whole 128-row tiles per rank, the block fits one staging half."""
        return (self.fuse_ag_gemm and x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and x.dim() == 2 and x.is_contiguous() and w.dim() == 2 and w.stride(1) == 1
                and x.shape[0] > 0 and x.shape[0] % 128 == 0 and x.shape[1] % 64 == 0
                and x.numel() * 2 <= self.half_bytes)

    def all_gather_gemm(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                        swiglu: bool = False, return_gathered: bool = False):
        """``all_gather(x, dim=0) @ w.T`` (+bias, optional fused SwiGLU) with the gather inside the
        GEMM kernel: every rank stages its rows in its symmetric buffer; while the tensor cores
        work on the own rows, the GEMM's epilogue warps pull the other ranks' rows over NVLink
        into a local buffer (each byte crosses the link once) and the tiles of a foreign block
        start as soon as it is complete."""
        lib = _lib()
        rows, k = x.shape
        n = w.shape[0]
        gathered = torch.empty((rows * self.world, k), dtype=torch.bfloat16, device=x.device)
        rc = lib.b200_symm_ag_stage(self.data_ptrs, self.signal_ptrs, self.world, self.rank, self.half_bytes,
                                    x.data_ptr(), gathered.data_ptr(), x.numel(), self.ag_ready.data_ptr(),
                                    self.done.data_ptr(), self._stream())
        if rc != 0:
            raise RuntimeError(f"all-gather staging failed ({rc})")
        out = torch.empty((rows * self.world, n // 2 if swiglu else n), dtype=torch.bfloat16, device=x.device)
        rc = lib.b200_gemm_all_gather(gathered.data_ptr(), self.data_ptrs, self.half_bytes,
                                      self.signal_ptrs[self.rank], self.ag_ready.data_ptr(), w.data_ptr(),
                                      out.data_ptr(), bias.data_ptr() if bias is not None else None, rows, n, k,
                                      w.stride(0), out.stride(0), 1 if swiglu else 0, self.world, self.rank,
                                      lib.b200_symm_epoch_word(), lib.b200_symm_ag_flag_word(),
                                      self.status.data_ptr(), 0, self._stream())
        if rc != 0:
            raise RuntimeError(f"fused all_gather + gemm failed ({rc})")
        ops._count(2)
        return (out, gathered) if return_gathered else out

    # ------------------------------------------------ fused GEMM -> reduce-scatter
    def can_gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        m, n = x.shape[0], w.shape[0]
        return (self.fuse_ag_gemm and x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and x.dim() == 2 and x.stride(1) == 1 and w.dim() == 2 and w.stride(1) == 1
                and m >= 128 * self.world and m % self.world == 0 and n % 16 == 0 and n <= 16384
                and m * n * 2 <= self.half_bytes)

    def gemm_reduce_scatter(self, x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                            residual: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
                            eps: float = 0.0) -> torch.Tensor:
        """``reduce_scatter(x @ w.T, dim=0)`` (+bias on one rank) with the transfer inside the GEMM:
        the epilogue stores every tile row into its owner's staging buffer over NVLink while
        later tiles are still being computed; a small second kernel signals, waits for all
        sources and sums this rank's rows (optionally ``+ residual`` and RMSNorm)."""
        lib = _lib()
        m, k = x.shape
        n = w.shape[0]
        rows = m // self.world
        rc = lib.b200_gemm_reduce_scatter_push(x.data_ptr(), w.data_ptr(),
                                               bias.data_ptr() if bias is not None else None, m, n, k, x.stride(0),
                                               w.stride(0), self.data_ptrs, self.signal_ptrs[self.rank],
                                               self.half_bytes, self.world, self.rank, lib.b200_symm_epoch_word(),
                                               self.status.data_ptr(), 0, self._stream())
        if rc != 0:
            raise RuntimeError(f"fused gemm + reduce_scatter (push) failed ({rc})")
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=x.device)
        rc = lib.b200_symm_rs_reduce(self.data_ptrs, self.signal_ptrs, self.world, self.rank, self.half_bytes,
                                     out.data_ptr(), rows, n, residual.data_ptr() if residual is not None else None,
                                     norm_weight.data_ptr() if norm_weight is not None else None, eps,
                                     self.done.data_ptr(), self.status.data_ptr(), self._stream())
        if rc != 0:
            raise RuntimeError(f"fused gemm + reduce_scatter (reduce) failed ({rc})")
        ops._count(2)
        return out

    def close(self) -> None:
        lib = _lib()
        try:
            torch.cuda.synchronize(self.device)
        except Exception:
            pass
        for p in self._opened:
            lib.b200_symm_close(p)
        for p in self._own:
            lib.b200_symm_free(p)
        self._opened, self._own = [], []


def wait_probe(flag: torch.Tensor, want: int, max_polls: int) -> int:
    """Run the collectives' bounded flag wait on ``flag`` (uint32/int32 [1] on the GPU) with a poll
    limit; returns the number of polls made.  When the flag never reaches ``want`` the kernel gives
    up, records status 5 (``ops.check_status`` raises) and returns: the failure path of the
    peer-memory kernels, reachable without a failing peer."""
    polls = torch.zeros(1, dtype=torch.int32, device=flag.device)
    st = ops.device_state(flag.device)
    rc = _lib().b200_symm_wait_probe(flag.data_ptr(), want, max_polls, st.status.data_ptr(), polls.data_ptr(),
                                     torch.cuda.current_stream(flag.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"wait probe launch failed ({rc})")
    return int(polls.item())


def attach_symmetric_memory(group, device: torch.device, half_bytes: Optional[int] = None):
    """Create the group's symmetric memory (idempotent) and hook it into its communicator."""
    if group.world_size <= 1 or group.comm.symm is not None:
        return group.comm.symm
    if group.world_size > 8:
        logger.warning("symmetric-memory collectives support up to 8 ranks; using NCCL")
        return None
    hb = half_bytes or int(os.environ.get("OMNI_B200_SYMM_HALF_MB", "80")) << 20
    # A rank that cannot set its buffers up (no peer access, handle exchange refused) must not leave
    # the others with peer-memory kernels that wait for it: the ranks agree on the outcome and fall
    # back to NCCL together.
    symm, err = None, None
    try:
        symm = SymmetricMemory(group, device, hb)
    except Exception as e:                                # noqa: BLE001 - any set-up failure means NCCL
        err = e
    ok = torch.tensor([0 if symm is None else 1], dtype=torch.int32)
    import torch.distributed as dist
    if group.cpu_group is not None:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group.cpu_group)
    if int(ok.item()) == 0:
        if symm is not None:
            symm.close()
        logger.warning("symmetric-memory collectives unavailable on %d ranks (%s); using NCCL",
                       group.world_size, err if err is not None else "another rank failed to set up")
        return None
    group.comm.symm = symm
    return group.comm.symm
