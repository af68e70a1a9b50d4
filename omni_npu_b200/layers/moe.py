"""Fused mixture-of-experts layer.

Pipeline (one code path for 1 GPU, tensor-parallel replicas and expert
parallelism):

    router GEMM (fp32 logits) -> top-k (softmax / sigmoid, bias correction,
    group-limited) -> dispatch (rows go straight into the owning rank's receive
    buffer, expert-sorted) -> grouped GEMM gate_up with SwiGLU epilogue ->
    grouped GEMM down -> combine (each token pulls its k outputs, weighted sum,
    + shared experts).

Shared experts run on a side stream while the routed experts run, as the
reference does (omni_npu/v1/layers/quantization/compressed_tensors/npu_compressed_tensors_moe.py:145-158).
Tokens are de-duplicated across attention-TP ranks before dispatch and
all-gathered afterwards when the residual stream is replicated
(omni_npu/v1/layers/fused_moe/layer.py:46-56,89-90).

Expert weights: ``w13`` [E_local, 2I, H] with gate / up rows interleaved in
groups of eight (SwiGLU epilogue layout), ``w2`` [E_local, H, I].
"""
from __future__ import annotations

from typing import Iterable, Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..ops import ref
from ..parallel import state as pstate
from .linear import ReplicatedLinear
from .mlp import FusedMLP
from .moe_dispatch import EpBuffers, ep_combine, ep_dispatch


def select_experts(router_logits: torch.Tensor, top_k: int, scoring_func: str = "softmax",
                   e_score_correction_bias: Optional[torch.Tensor] = None, n_group: int = 1,
                   topk_group: int = 1, renormalize: bool = False,
                   routed_scaling_factor: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """(weights fp32 [T,k], ids int32 [T,k]); counterpart of
    omni_npu/layers/fused_moe/layer.py:254-308."""
    ids, w = ops.moe_topk(router_logits.float(), e_score_correction_bias, top_k,
                          scoring_func == "sigmoid", n_group, topk_group, renormalize,
                          routed_scaling_factor)
    return w, ids


class FusedMoE(nn.Module):
    def __init__(self, num_experts: int, top_k: int, hidden_size: int, intermediate_size: int,
                 dtype=torch.bfloat16, device=None, scoring_func: str = "softmax",
                 renormalize: bool = False, routed_scaling_factor: float = 1.0, n_group: int = 1,
                 topk_group: int = 1, router_bias: bool = False, num_shared_experts: int = 0,
                 shared_intermediate_size: Optional[int] = None, enable_expert_parallel: bool = True,
                 prefix: str = "", max_tokens: int = 8192, quant: Optional[str] = None,
                 num_redundant_experts: int = 0, shared_quant_factory=None) -> None:
        super().__init__()
        self.num_experts, self.top_k = num_experts, top_k
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.scoring_func, self.renormalize = scoring_func, renormalize
        self.routed_scaling_factor = routed_scaling_factor
        self.n_group, self.topk_group = n_group, topk_group
        self.max_tokens = max_tokens
        self.dtype = dtype
        self.tp_group = pstate.get_tp_group()
        self.ep_group = pstate.get_ep_group() if enable_expert_parallel else None
        self.ep_size = self.ep_group.world_size if self.ep_group is not None else 1
        self.ep_rank = self.ep_group.rank_in_group if self.ep_group is not None else 0
        # physical expert slots = logical experts + redundant copies of the hot ones (parallel/eplb.py)
        self.num_physical = num_experts + num_redundant_experts
        assert self.num_physical % self.ep_size == 0
        self.local_experts = self.num_physical // self.ep_size
        self.expert_start = self.ep_rank * self.local_experts
        self.eplb = None
        if num_redundant_experts > 0:
            from ..parallel.eplb import EplbState
            self.eplb = EplbState(num_experts, num_redundant_experts, self.ep_size, device)
        self.gate = ReplicatedLinear(hidden_size, num_experts, dtype=dtype, device=device,
                                     prefix=f"{prefix}.gate")
        if router_bias:
            self.e_score_correction_bias = nn.Parameter(torch.zeros(num_experts, dtype=torch.float32,
                                                                    device=device), requires_grad=False)
        else:
            self.e_score_correction_bias = None
        wdt = torch.float8_e4m3fn if quant == "fp8" else dtype
        self.quant = quant
        self.w13 = nn.Parameter(torch.empty(self.local_experts, 2 * intermediate_size, hidden_size,
                                            dtype=wdt, device=device), requires_grad=False)
        self.w2 = nn.Parameter(torch.empty(self.local_experts, hidden_size, intermediate_size,
                                           dtype=wdt, device=device), requires_grad=False)
        if quant == "fp8":
            self.w13_scale = nn.Parameter(torch.ones(self.local_experts, (2 * intermediate_size + 127) // 128,
                                                     (hidden_size + 127) // 128, dtype=torch.float32,
                                                     device=device), requires_grad=False)
            self.w2_scale = nn.Parameter(torch.ones(self.local_experts, (hidden_size + 127) // 128,
                                                    (intermediate_size + 127) // 128, dtype=torch.float32,
                                                    device=device), requires_grad=False)
        self.shared_experts = None
        if num_shared_experts > 0:
            inter = (shared_intermediate_size or intermediate_size) * num_shared_experts
            # shared experts are replicated when tokens are de-duplicated across TP ranks
            # quantised checkpoints quantise the shared experts like every other linear
            self.shared_experts = FusedMLP(hidden_size, inter, dtype, device, prefix=f"{prefix}.shared_experts",
                                           quant_method_factory=shared_quant_factory,
                                           group=_solo_group() if self.ep_size > 1 else None,
                                           reduce_results=False, fuse_swiglu=shared_quant_factory is None)
        self.buffers: Optional[EpBuffers] = None
        self._side_stream: Optional[torch.cuda.Stream] = None
        self.expert_load: Optional[torch.Tensor] = None   # per-expert token counts (EPLB statistics)

    # ----------------------------------------------------------------- set-up
    def init_ep_buffers(self, comm=None) -> None:
        """Called once after loading (``prepare_communication_buffer_for_model``)."""
        dev = self.w13.device
        if dev.type != "cuda" or self.buffers is not None:
            return
        fp8 = self.quant == "fp8" and self.hidden_size % 128 == 0
        key = (id(self.ep_group), self.num_physical, self.hidden_size, self.top_k, fp8)
        shared = _SHARED_BUFFERS.get(key)
        if shared is None:
            group = self.ep_group if self.ep_group is not None else _solo_group()
            shared = EpBuffers(group, dev, self.num_physical if self.ep_size > 1 else self.local_experts,
                               self.hidden_size, self.max_tokens, self.top_k, fp8_dispatch=fp8)
            _SHARED_BUFFERS[key] = shared
        self.buffers = shared
        self._side_stream = torch.cuda.Stream(dev)

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, expert_id: Optional[int] = None,
                      shard: Optional[str] = None) -> bool:
        """Load one expert's gate / up / down tensor.  Returns False when the expert
        lives on another rank.  Without an expert id the tensor is a plain parameter of
        the layer (router bias) and is copied as is."""
        if expert_id is None:
            param.data.copy_(loaded.to(param.dtype))
            return True
        if self.eplb is not None:
            # every local slot that holds (a copy of) this expert receives the tensor
            mine = [j for j, e in enumerate(self.eplb.local_logical_ids(self.ep_rank)) if e == expert_id]
            for j in mine:
                self._load_slot(param, loaded, j, shard)
            return bool(mine)
        local = expert_id - self.expert_start
        if local < 0 or local >= self.local_experts:
            return False
        self._load_slot(param, loaded, local, shard)
        return True

    def _load_slot(self, param: nn.Parameter, loaded: torch.Tensor, local: int, shard: Optional[str]) -> None:
        i = self.intermediate_size
        if shard in ("gate", "up"):
            j = torch.arange(i, device=param.device)
            rows = (j // 8) * 16 + (0 if shard == "gate" else 8) + (j % 8)
            if param.dim() == 3 and param.shape[1] == 2 * i:
                param.data[local, rows] = loaded.to(param.device).to(param.dtype) \
                    if param.dtype != torch.float8_e4m3fn else loaded.to(param.device)
            else:   # block scales: gate blocks then up blocks are kept in checkpoint order
                nb = loaded.shape[0]
                off = 0 if shard == "gate" else nb
                param.data[local, off:off + nb].copy_(loaded)
        else:
            param.data[local].copy_(loaded if param.dtype == torch.float8_e4m3fn else loaded.to(param.dtype))

    def process_weights_after_loading(self) -> None:
        """Block-scaled e4m3 expert weights are expanded to the compute dtype once, after loading
        (the grouped kernel has no per-block scale path): ``w * scale`` per 128 x 128 block.  The
        gate / up rows of ``w13`` are interleaved in groups of 8, their scale blocks are not, so
        every stored row looks up the block of the checkpoint row it came from."""
        if self.quant != "fp8" or self.w13.dtype != torch.float8_e4m3fn:
            return
        i, h = self.intermediate_size, self.hidden_size
        if self.w13.is_cuda and h % 128 == 0 and i % 128 == 0:
            return        # stays e4m3: the grouped block-scaled kernel consumes weights and scales as loaded
        dev = self.w13.device
        r = torch.arange(2 * i, device=dev)
        is_up = (r // 8) % 2
        src = (r // 16) * 8 + r % 8                      # row inside the gate (or up) matrix
        nb = (i + 127) // 128
        blk = src // 128 + is_up * nb
        w13 = torch.empty(self.w13.shape, dtype=self.dtype, device=dev)
        w2 = torch.empty(self.w2.shape, dtype=self.dtype, device=dev)
        for e in range(self.local_experts):              # expert by expert: bounded temporary memory
            s13 = self.w13_scale[e][blk].repeat_interleave(128, dim=1)[:, :h]
            w13[e] = (self.w13[e].float() * s13).to(self.dtype)
            s2 = self.w2_scale[e].repeat_interleave(128, dim=0)[:h].repeat_interleave(128, dim=1)[:, :i]
            w2[e] = (self.w2[e].float() * s2).to(self.dtype)
        self.w13 = nn.Parameter(w13, requires_grad=False)
        self.w2 = nn.Parameter(w2, requires_grad=False)
        self.quant = "fp8-expanded"

    def rebalance(self, decay: float = 0.0) -> int:
        """Re-plan the expert placement from the load seen since the last call and move the
        expert weights accordingly (collective over the expert-parallel group; call between
        steps).  Returns the number of physical slots whose expert changed."""
        if self.eplb is None:
            return 0
        from ..parallel.eplb import rearrange_expert_weights
        group = self.ep_group if self.ep_size > 1 else None
        old, new = self.eplb.replan(group, decay)
        tensors = [self.w13.data, self.w2.data]
        if self.quant == "fp8":
            tensors += [self.w13_scale.data, self.w2_scale.data]
        moved = rearrange_expert_weights(tensors, old, new, group)
        self.eplb.set_placement(new)
        return moved

    # ----------------------------------------------------------------- forward
    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        """hidden [T,H] (replicated across TP ranks) -> [T,H]."""
        tp = self.tp_group.world_size
        t_full = hidden.shape[0]
        dedup = self.ep_size > 1 and tp > 1
        if dedup:
            # each TP rank handles a slice of the tokens; results are gathered afterwards
            per = (t_full + tp - 1) // tp
            lo = min(t_full, per * self.tp_group.rank_in_group)
            x = hidden[lo: min(t_full, lo + per)]
            if x.shape[0] < per:
                x = torch.cat([x, hidden.new_zeros(per - x.shape[0], hidden.shape[1])])
        else:
            x = hidden
        logits = self.gate(x, out_dtype=torch.float32)
        w, ids = select_experts(logits, self.top_k, self.scoring_func, self.e_score_correction_bias,
                                self.n_group, self.topk_group, self.renormalize,
                                self.routed_scaling_factor)
        if dedup and lo + per > t_full:
            pad_from = max(0, t_full - lo)
            ids = ids.clone()
            ids[pad_from:] = -1          # padded rows take part in nothing
        if self.eplb is not None:
            self.eplb.record(ids)
            ids = self.eplb.remap(ids)
        out = self._routed(x, w, ids)
        if dedup:
            out = self.tp_group.all_gather(out, dim=0)[:t_full]
        elif tp > 1 and self.ep_size == 1:
            pass  # experts replicated: nothing to reduce
        return out

    def _routed(self, x: torch.Tensor, w: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        comm = self.ep_group.comm if self.ep_size > 1 else _Solo.comm
        shared_out = None
        if x.is_cuda:
            if self.buffers is None:
                self.init_ep_buffers()
            ids_local = ids
            if self.shared_experts is not None:
                # shared experts overlap with dispatch + routed experts on a side stream
                cur = torch.cuda.current_stream(x.device)
                self._side_stream.wait_stream(cur)
                with torch.cuda.stream(self._side_stream):
                    shared_out = self.shared_experts(x)
            fp8_rows = self.quant == "fp8" and self.buffers.fp8_dispatch
            rows, offsets, handle = ep_dispatch(comm, x, ids_local, w, self.num_physical, self.buffers,
                                                fp8=fp8_rows)
            if self.quant == "fp8":
                # block-scaled e4m3 experts: the rows arrive quantised per token per 128 columns (the
                # scatter kernel quantises them on the way; without fp8 buffers they are quantised
                # here), SwiGLU fused into the first product's epilogue, requantise, second product
                rq, rs = rows if fp8_rows else ops.quant_fp8_1x128(rows)
                h1 = ops.grouped_gemm_fp8_block(rq, rs, self.w13, self.w13_scale, offsets, swiglu=True,
                                                up_scale_row0=(self.intermediate_size + 127) // 128)
                hq, hs = ops.quant_fp8_1x128(h1)
                y = ops.grouped_gemm_fp8_block(hq, hs, self.w2, self.w2_scale, offsets)
            else:
                h1 = ops.grouped_gemm(rows, self.w13, offsets, swiglu=True)
                y = ops.grouped_gemm(h1, self.w2, offsets)
            self.buffers.expert_y[: y.shape[0]].copy_(y)
            if shared_out is not None:
                torch.cuda.current_stream(x.device).wait_stream(self._side_stream)
            return ep_combine(comm, self.buffers.expert_y, handle, shared_out, self.buffers)
        # CPU / reference path
        if self.shared_experts is not None:
            shared_out = self.shared_experts(x)
        rows, offsets, handle = ep_dispatch(comm, x, ids, w, self.num_physical)
        h1 = ops.grouped_gemm(rows, self.w13, offsets, swiglu=True)
        y = ops.grouped_gemm(h1, self.w2, offsets)
        return ep_combine(comm, y, handle, shared_out)


_SHARED_BUFFERS: dict = {}


class _Solo:
    """A one-rank stand-in for a process group."""
    world_size = 1
    rank_in_group = 0

    class _Comm:
        world_size = 1
        rank_in_group = 0
        symm = None
        ep_buffers = None

    comm = _Comm()

    def all_gather_object(self, obj):
        return [obj]

    def all_reduce(self, x):
        return x

    def barrier(self):
        pass


def _solo_group():
    return _Solo()
