"""Expert-parallel dispatch / combine over peer-mapped buffers.

``EpBuffers`` owns, per expert-parallel group, the symmetric receive buffer
(token rows routed to this rank's experts), the symmetric expert-output buffer,
the replicated count matrix and the phase flags, and drives the kernels in
``csrc/moe/moe_ep.cu``.  A group of one rank uses the same kernels as the local
permute / un-permute, so single-GPU and expert-parallel runs share one path.

``ep_dispatch`` / ``ep_combine`` are what ``B200Communicator.dispatch`` /
``.combine`` call (the reference's communicator leaves them as no-ops and lets
vendor kernels talk to HCCL by name: omni_npu/distributed/communicator.py:263-278,
omni_npu/layers/fused_moe/npu_moe_prepare_finalize.py:66-119).  CPU tensors take
a plain PyTorch implementation with the same semantics (used by gloo tests).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

import torch

from .. import ops

_LIB = None


class _EpHostArgs(ctypes.Structure):
    _fields_ = [("recv_x", ctypes.c_void_p * 8), ("expert_y", ctypes.c_void_p * 8),
                ("counts", ctypes.c_void_p * 8), ("flags", ctypes.c_void_p * 8)]


def _lib():
    global _LIB
    if _LIB is None:
        ops.load_extension(required=True)
        lib = ctypes.CDLL(str(Path(__file__).resolve().parent.parent / "_C.so"))
        vp, ci, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.b200_ep_flag_words.restype = ci
        lib.b200_ep_dispatch.argtypes = [ctypes.POINTER(_EpHostArgs), ci, ci, ci, ci, vp, vp, ci, ci, ci, ll,
                                         vp, vp, vp, vp, vp, vp, vp]
        lib.b200_ep_dispatch.restype = ci
        lib.b200_ep_dispatch_fp8.argtypes = [ctypes.POINTER(_EpHostArgs), ci, ci, ci, ci, vp, vp, ci, ci, ci, ll,
                                             vp, vp, vp, vp, vp, vp, vp, vp, vp]
        lib.b200_ep_dispatch_fp8.restype = ci
        lib.b200_ep_combine.argtypes = [ctypes.POINTER(_EpHostArgs), ci, ci, ci, ci, vp, vp, vp, vp, vp, ci,
                                        ci, ci, ll, ll, vp, vp]
        lib.b200_ep_combine.restype = ci
        _LIB = lib
    return _LIB


@dataclass
class DispatchHandle:
    """What combine needs to find its way back."""
    topk_ids: torch.Tensor          # [T,k] int32 (global expert ids, -1 = inactive)
    topk_weights: torch.Tensor      # [T,k] fp32
    slots: Optional[torch.Tensor]   # [T*k] int32 row in the owner's buffers (CUDA path)
    num_tokens: int
    rows: int                       # rows of the local receive buffer in use (upper bound)
    expert_offsets: torch.Tensor    # [E_local+1] int32
    cpu_state: Optional[dict] = None


class EpBuffers:
    def __init__(self, group, device: torch.device, num_experts: int, hidden: int, max_tokens: int,
                 top_k: int, capacity_factor: float = 2.0, fp8_dispatch: bool = False) -> None:
        from ..parallel.symm_mem import _lib as symm_lib
        self.group, self.device = group, device
        self.world, self.rank = group.world_size, group.rank_in_group
        self.num_experts, self.hidden, self.top_k = num_experts, hidden, top_k
        assert num_experts % self.world == 0
        self.experts_per_rank = num_experts // self.world
        factor = 1.0 if self.world == 1 else capacity_factor
        self.cap_rows = int(max(256, factor * max_tokens * top_k))
        self.max_tokens = max_tokens
        lib = symm_lib()
        self._own, self._opened = [], []
        self._symm_lib = lib

        def alloc(nbytes):
            ptr = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(64)
            rc = lib.b200_symm_alloc(max(nbytes, 2 << 20), ctypes.byref(ptr), handle)
            if rc != 0:
                raise RuntimeError(f"EP buffer allocation of {nbytes} bytes failed ({rc})")
            self._own.append(ptr)
            return ptr, handle.raw

        row_bytes = hidden * 2
        mine = [alloc(self.cap_rows * row_bytes), alloc(self.cap_rows * row_bytes),
                alloc(self.world * num_experts * 4), alloc(_lib().b200_ep_flag_words() * 4)]
        # fp8 dispatch: rows arrive quantised (e4m3 + one fp32 scale per 128 columns) in two more
        # peer-mapped buffers; half the bytes of the bf16 rows cross the link
        self.fp8_dispatch = bool(fp8_dispatch) and hidden % 128 == 0
        if self.fp8_dispatch:
            mine += [alloc(self.cap_rows * hidden), alloc(self.cap_rows * (hidden // 128) * 4)]
        handles = [h for _, h in mine]
        everyone = group.all_gather_object(handles) if self.world > 1 else [handles]
        self.args = _EpHostArgs()
        q_table, s_table = (ctypes.c_void_p * 8)(), (ctypes.c_void_p * 8)()
        tables = (self.args.recv_x, self.args.expert_y, self.args.counts, self.args.flags) + \
            ((q_table, s_table) if self.fp8_dispatch else ())
        for r in range(self.world):
            for i, table in enumerate(tables):
                if r == self.rank:
                    table[r] = mine[i][0].value
                else:
                    p = ctypes.c_void_p()
                    if lib.b200_symm_open(everyone[r][i], ctypes.byref(p)) != 0:
                        raise RuntimeError(f"cannot map expert-parallel buffers of rank {r}")
                    table[r] = p.value
                    self._opened.append(p)
        # torch views of my own buffers (the grouped GEMMs read / write them in place)
        self.recv_x = _as_tensor(mine[0][0].value, (self.cap_rows, hidden), torch.bfloat16, device)
        self.expert_y = _as_tensor(mine[1][0].value, (self.cap_rows, hidden), torch.bfloat16, device)
        if self.fp8_dispatch:
            self.recv_q = _as_tensor(mine[4][0].value, (self.cap_rows, hidden), torch.uint8, device).view(torch.float8_e4m3fn)
            self.recv_s = _as_tensor(mine[5][0].value, (self.cap_rows, hidden // 128), torch.float32, device)
            # the kernel takes the two pointer tables from device memory
            self.q_ptrs = torch.tensor([int(q_table[r] or 0) for r in range(8)], dtype=torch.int64, device=device)
            self.s_ptrs = torch.tensor([int(s_table[r] or 0) for r in range(8)], dtype=torch.int64, device=device)
        i32 = dict(dtype=torch.int32, device=device)
        self.expert_offsets = torch.zeros(self.experts_per_rank + 1, **i32)
        self.send_base = torch.zeros(num_experts, **i32)
        self.cursors = torch.zeros(num_experts, **i32)
        self.slots = torch.zeros(max_tokens * top_k, **i32)
        self.total_recv = torch.zeros(1, **i32)
        self.status = ops.device_state(device).status
        torch.cuda.synchronize(device)
        if self.world > 1:
            group.barrier()

    def close(self) -> None:
        for p in self._opened:
            self._symm_lib.b200_symm_close(p)
        for p in self._own:
            self._symm_lib.b200_symm_free(p)
        self._opened, self._own = [], []


def _as_tensor(ptr: int, shape, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    """A torch tensor over memory this module allocated itself (kept alive by EpBuffers)."""
    n = 1
    for s in shape:
        n *= s

    class _Holder:
        pass

    h = _Holder()
    h.__cuda_array_interface__ = {"shape": (n * dtype.itemsize,), "typestr": "|u1", "data": (ptr, False),
                                  "version": 2}
    flat = torch.as_tensor(h, device=device)
    return flat.view(dtype).view(*shape)


# ----------------------------------------------------------------- public API
def ep_dispatch(comm, hidden: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor,
                num_experts: int, buffers: Optional[EpBuffers] = None, fp8: bool = False):
    """Send every token row to the ranks owning its experts.

    Returns ``(rows, expert_offsets, handle)``: ``rows`` [R,H] are the rows received
    for this rank's experts, grouped by local expert as ``expert_offsets`` says.  With ``fp8``
    (buffers built with ``fp8_dispatch``) the rows are quantised while they are scattered and
    ``rows`` is the pair ``(e4m3 rows [R,H], scales [R,H/128])``: one byte per element plus the
    scales cross the link (reference: ``quant_mode=2`` of the dispatch op,
    omni_npu/layers/fused_moe/npu_moe_prepare_finalize.py:66-81)."""
    t, k = topk_ids.shape
    if not hidden.is_cuda:
        rows, offsets, handle = _cpu_dispatch(comm, hidden, topk_ids, topk_weights, num_experts)
        if fp8:
            return ops.quant_fp8_1x128(rows), offsets, handle
        return rows, offsets, handle
    buf = buffers or comm.ep_buffers
    if buf is None:
        raise RuntimeError("expert-parallel buffers not initialised for this communicator")
    if t > buf.max_tokens:
        raise RuntimeError(f"{t} tokens exceed the dispatch capacity of {buf.max_tokens}")
    stream = torch.cuda.current_stream(hidden.device).cuda_stream
    common = (ctypes.byref(buf.args), buf.world, buf.rank, buf.num_experts,
              buf.cap_rows, hidden.data_ptr(), topk_ids.data_ptr(), t, k,
              hidden.shape[1], hidden.stride(0), buf.expert_offsets.data_ptr(),
              buf.send_base.data_ptr(), buf.cursors.data_ptr(), buf.slots.data_ptr(),
              buf.total_recv.data_ptr(), buf.status.data_ptr())
    if fp8:
        if not buf.fp8_dispatch:
            raise RuntimeError("these expert-parallel buffers were built without fp8 dispatch")
        rc = _lib().b200_ep_dispatch_fp8(*common, buf.q_ptrs.data_ptr(), buf.s_ptrs.data_ptr(), stream)
    else:
        rc = _lib().b200_ep_dispatch(*common, stream)
    if rc != 0:
        raise RuntimeError(f"ep_dispatch failed ({rc})")
    ops._count(3 if buf.world == 1 else 6)  # count, layout, scatter (+ flag kernels)
    # static upper bound on the rows in use (device-side counts decide the real extent)
    rows = buf.cap_rows if buf.world > 1 else max(t * k, 1)
    handle = DispatchHandle(topk_ids, topk_weights, buf.slots, t, rows, buf.expert_offsets)
    if fp8:
        return (buf.recv_q[:rows], buf.recv_s[:rows]), buf.expert_offsets, handle
    return buf.recv_x[:rows], buf.expert_offsets, handle


def ep_combine(comm, expert_out: torch.Tensor, handle: DispatchHandle,
               shared_out: Optional[torch.Tensor] = None, buffers: Optional[EpBuffers] = None,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Bring the expert outputs back and reduce them with the routing weights."""
    if handle.cpu_state is not None:
        return _cpu_combine(comm, expert_out, handle, shared_out)
    buf = buffers or comm.ep_buffers
    t, k = handle.topk_ids.shape
    h = buf.hidden
    if expert_out.data_ptr() != buf.expert_y.data_ptr():
        buf.expert_y[: expert_out.shape[0]].copy_(expert_out)
    out = torch.empty((t, h), dtype=torch.bfloat16, device=buf.device) if out is None else out
    stream = torch.cuda.current_stream(buf.device).cuda_stream
    rc = _lib().b200_ep_combine(ctypes.byref(buf.args), buf.world, buf.rank, buf.num_experts, buf.cap_rows,
                                out.data_ptr(), handle.topk_ids.data_ptr(), handle.topk_weights.data_ptr(),
                                handle.slots.data_ptr(), shared_out.data_ptr() if shared_out is not None else None,
                                t, k, h, out.stride(0), shared_out.stride(0) if shared_out is not None else 0,
                                buf.status.data_ptr(), stream)
    if rc != 0:
        raise RuntimeError(f"ep_combine failed ({rc})")
    ops._count(1 if buf.world == 1 else 5)
    return out


# ------------------------------------------------------------ CPU reference
def _cpu_dispatch(comm, hidden, topk_ids, topk_weights, num_experts):
    world, rank = comm.world_size, comm.rank_in_group
    epr = num_experts // world
    t, k = topk_ids.shape
    flat_ids = topk_ids.reshape(-1).long()
    active = flat_ids >= 0
    pair_idx = torch.arange(t * k)[active]
    ids = flat_ids[active]
    dest = ids // epr
    order = torch.argsort(dest * num_experts + ids, stable=True)
    pair_idx, ids, dest = pair_idx[order], ids[order], dest[order]
    send_rows = hidden[pair_idx // k]
    send_counts = [int((dest == d).sum()) for d in range(world)]
    if world > 1:
        recv_counts = comm.all_to_all_single(torch.tensor(send_counts)).tolist()
        rows = comm.all_to_all_single(send_rows, recv_counts, send_counts)
        rids = comm.all_to_all_single(ids, recv_counts, send_counts)
    else:
        recv_counts, rows, rids = send_counts, send_rows, ids
    local = rids - rank * epr
    lorder = torch.argsort(local, stable=True)
    rows = rows[lorder]
    counts = torch.bincount(local, minlength=epr)
    offsets = torch.zeros(epr + 1, dtype=torch.int32)
    offsets[1:] = counts.cumsum(0)
    handle = DispatchHandle(topk_ids, topk_weights, None, t, rows.shape[0], offsets,
                            cpu_state=dict(pair_idx=pair_idx, lorder=lorder, send_counts=send_counts,
                                           recv_counts=recv_counts, k=k))
    return rows, offsets, handle


def _cpu_combine(comm, expert_out, handle, shared_out):
    st = handle.cpu_state
    world = comm.world_size
    back = torch.empty_like(expert_out)
    back[st["lorder"]] = expert_out
    if world > 1:
        back = comm.all_to_all_single(back, st["send_counts"], st["recv_counts"])
    t, k = handle.topk_ids.shape
    out = torch.zeros(t, expert_out.shape[1], dtype=torch.float32)
    w = handle.topk_weights.reshape(-1)[st["pair_idx"]].float().unsqueeze(1)
    out.index_add_(0, st["pair_idx"] // k, back.float() * w)
    if shared_out is not None:
        out += shared_out.float()
    return out.to(expert_out.dtype)
