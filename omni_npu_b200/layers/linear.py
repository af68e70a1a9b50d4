"""Linear layers with tensor parallelism and input / output transforms.

Weights are stored ``[out, in]`` (K contiguous), which is the layout the
tcgen05 GEMM consumes for both operands, so no transpose or format cast is
needed at load time (the reference stores transposed weights in the NZ tile
format: omni_npu/v1/layers/linear.py:105-113).

Each layer may name an ``x_transform`` applied to its input and a
``y_transform`` applied to its output, chosen from NoOp / AllGather /
AllReduce / ReduceScatter / ALL2ALL over the layer's group
(omni_npu/v1/layers/linear.py:39-53).  AllGather-before and
AllReduce/ReduceScatter-after are the sequence-parallel ("FlashComm")
residual-stream pattern; on CUDA they run as fused GEMM+collective kernels
when the group has symmetric memory attached.

fp8 weights (e4m3 with 128x128 block scales, ``weight_scale_inv``) are
supported through ``Fp8BlockLinearMethod``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
from torch import nn

from .. import ops
from ..parallel import state as pstate
from ..parallel.state import GroupCoordinator

TRANSFORMS = ("NoOp", "AllGather", "AllReduce", "ReduceScatter", "ALL2ALL")


def apply_transform(x: torch.Tensor, kind: Optional[str], group: GroupCoordinator, dim: int = 0) -> torch.Tensor:
    if kind in (None, "NoOp") or group.world_size == 1:
        return x
    if kind == "AllGather":
        return group.all_gather(x, dim)
    if kind == "AllReduce":
        return group.all_reduce(x)
    if kind == "ReduceScatter":
        return group.reduce_scatter(x, dim)
    if kind == "ALL2ALL":
        return group.comm.all_to_all(x, scatter_dim=0, gather_dim=-1)
    raise ValueError(f"unknown transform {kind}")


class ReducedShard:
    """Result of a row-parallel projection that was already reduce-scattered inside its GEMM:
    ``tensor`` holds this rank's rows of the sum."""

    def __init__(self, tensor: torch.Tensor) -> None:
        self.tensor = tensor


def _sharded_input(layer: "LinearBase", x, swiglu: bool = False, out_dtype=None):
    """Input handed over as token shards (``layers.flashcomm.ShardedRows``): returns
    (y, None) when the gather was fused into the GEMM, else (None, gathered rows)."""
    y = gathered_gemm(layer, x.shard, swiglu, out_dtype)
    if y is not None:
        return y[: x.num_tokens], None
    return None, x.full()


def gathered_gemm(layer: "LinearBase", x: torch.Tensor, swiglu: bool = False,
                  out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """``all_gather(x) @ W^T`` as one kernel over peer memory when the layer is an unquantised bf16
    projection and the group has symmetric memory (the all-gather feeding a column-parallel
    projection of a sequence-sharded residual stream); None when the fused path does not apply."""
    symm = getattr(layer.group.comm, "symm", None)
    if (symm is None or not isinstance(layer.quant_method, UnquantizedLinearMethod) or x.dim() != 2
            or out_dtype not in (None, torch.bfloat16) or not symm.can_all_gather_gemm(x, layer.weight)):
        return None
    return symm.all_gather_gemm(x, layer.weight, layer.bias, swiglu)


# ------------------------------------------------------------------ methods
class UnquantizedLinearMethod:
    def create_weights(self, layer: "LinearBase", in_features: int, out_features: int,
                       dtype: torch.dtype, device) -> None:
        layer.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device),
                                    requires_grad=False)

    def process_weights_after_loading(self, layer: "LinearBase") -> None:
        pass

    def apply(self, layer: "LinearBase", x: torch.Tensor, bias: Optional[torch.Tensor],
              residual: Optional[torch.Tensor] = None, swiglu: bool = False,
              out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return ops.gemm(x, layer.weight, bias, residual, out_dtype, swiglu)


class Fp8BlockLinearMethod:
    """e4m3 weights with one fp32 scale per 128x128 block; activations are
    quantised per token per 128 columns on the fly."""

    def __init__(self, block: Tuple[int, int] = (128, 128)) -> None:
        self.block = block

    def create_weights(self, layer, in_features, out_features, dtype, device) -> None:
        bn, bk = self.block
        layer.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=torch.float8_e4m3fn,
                                                device=device), requires_grad=False)
        layer.weight_scale_inv = nn.Parameter(
            torch.ones((out_features + bn - 1) // bn, (in_features + bk - 1) // bk,
                       dtype=torch.float32, device=device), requires_grad=False)

    def process_weights_after_loading(self, layer) -> None:
        pass

    def apply(self, layer, x, bias, residual=None, swiglu=False, out_dtype=None):
        from .quant_fp8 import fp8_block_gemm
        return fp8_block_gemm(x, layer.weight, layer.weight_scale_inv, bias, residual, self.block,
                              swiglu=swiglu, out_dtype=out_dtype)


# -------------------------------------------------------------------- layers
class LinearBase(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool, dtype: torch.dtype,
                 device=None, quant_method=None, prefix: str = "",
                 group: Optional[GroupCoordinator] = None, x_transform: Optional[str] = None,
                 y_transform: Optional[str] = None) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.prefix = prefix
        self.group = group or pstate.get_layer_group(_layer_key(prefix)) or pstate.get_tp_group()
        self.tp_size = self.group.world_size
        self.tp_rank = self.group.rank_in_group
        planned_x, planned_y = pstate.get_layer_transforms(_layer_key(prefix))
        self.x_transform = x_transform if x_transform is not None else planned_x
        self.y_transform = y_transform if y_transform is not None else planned_y
        self.quant_method = quant_method or UnquantizedLinearMethod()
        self.dtype = dtype
        self._has_bias = bias

    def _create(self, in_local: int, out_local: int, device) -> None:
        self.quant_method.create_weights(self, in_local, out_local, self.dtype, device)
        if self._has_bias:
            self.bias = nn.Parameter(torch.zeros(out_local, dtype=self.dtype, device=device),
                                     requires_grad=False)
        else:
            self.bias = None

    def process_weights_after_loading(self) -> None:
        self.quant_method.process_weights_after_loading(self)


def _layer_key(prefix: str) -> str:
    """Last two dotted components of a module name, e.g. 'self_attn.o_proj'
    (the key per-layer groups are registered under)."""
    parts = prefix.split(".")
    return ".".join(parts[-2:]) if len(parts) >= 2 else prefix


class ReplicatedLinear(LinearBase):
    def __init__(self, in_features, out_features, bias=False, dtype=torch.bfloat16, device=None, **kw):
        super().__init__(in_features, out_features, bias, dtype, device, **kw)
        self._create(in_features, out_features, device)

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        x = apply_transform(x, self.x_transform, self.group)
        y = self.quant_method.apply(self, x, self.bias, out_dtype=out_dtype)
        return apply_transform(y, self.y_transform, self.group)

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        param.data.copy_(loaded.to(param.dtype))


class ColumnParallelLinear(LinearBase):
    """Output features sharded across the group."""

    def __init__(self, in_features, out_features, bias=False, dtype=torch.bfloat16, device=None,
                 gather_output: bool = False, **kw):
        super().__init__(in_features, out_features, bias, dtype, device, **kw)
        assert out_features % self.tp_size == 0
        self.out_local = out_features // self.tp_size
        self.gather_output = gather_output
        self._create(in_features, self.out_local, device)

    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        y = None
        if not isinstance(x, torch.Tensor):
            y, x = _sharded_input(self, x, out_dtype=out_dtype)
        elif self.x_transform == "AllGather" and self.tp_size > 1:
            y = gathered_gemm(self, x, out_dtype=out_dtype)
        if y is None:
            x = apply_transform(x, self.x_transform, self.group)
            y = self.quant_method.apply(self, x, self.bias, out_dtype=out_dtype)
        if self.gather_output and self.tp_size > 1:
            y = self.group.all_gather(y, dim=-1)
        return apply_transform(y, self.y_transform, self.group)

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        _copy_sharded(param, loaded, 0, self.tp_rank, self.tp_size)


class MergedColumnParallelLinear(LinearBase):
    """Several column-parallel projections sharing one input, stored as one
    weight so that one GEMM computes all of them (gate+up, q_a+kv_a, ...).
    With ``swiglu_interleave`` the two halves (gate, up) are stored interleaved
    in groups of 8 rows so the GEMM epilogue can apply silu(gate)*up."""

    def __init__(self, in_features, output_sizes: Sequence[int], bias=False, dtype=torch.bfloat16,
                 device=None, swiglu_interleave: bool = False, **kw):
        super().__init__(in_features, sum(output_sizes), bias, dtype, device, **kw)
        self.output_sizes = list(output_sizes)
        assert all(s % self.tp_size == 0 for s in output_sizes)
        self.local_sizes = [s // self.tp_size for s in output_sizes]
        self.swiglu_interleave = swiglu_interleave
        if swiglu_interleave:
            assert len(output_sizes) == 2 and output_sizes[0] == output_sizes[1]
            assert self.local_sizes[0] % 8 == 0
        self._create(in_features, sum(self.local_sizes), device)

    def forward(self, x: torch.Tensor, fuse_swiglu: bool = False) -> torch.Tensor:
        swiglu = fuse_swiglu and self.swiglu_interleave
        if not isinstance(x, torch.Tensor):
            y, x = _sharded_input(self, x, swiglu=swiglu)
            if y is not None:
                return y
        elif self.x_transform == "AllGather" and self.tp_size > 1:
            y = gathered_gemm(self, x, swiglu=swiglu)
            if y is not None:
                return y
        x = apply_transform(x, self.x_transform, self.group)
        return self.quant_method.apply(self, x, self.bias, swiglu=swiglu)

    def _rows_of(self, shard_id: int) -> torch.Tensor:
        """Row indices (in the local weight) that hold shard ``shard_id``."""
        n = self.local_sizes[shard_id]
        if not self.swiglu_interleave:
            off = sum(self.local_sizes[:shard_id])
            return torch.arange(off, off + n)
        j = torch.arange(n)
        return (j // 8) * 16 + shard_id * 8 + (j % 8)

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        if shard_id is None:
            # already-fused checkpoint tensor: split it into its parts
            blocks = param.dim() == 2 and param.shape[0] != sum(self.local_sizes) and param.dtype == torch.float32
            off = 0
            for i, s in enumerate(self.output_sizes):
                n = (s + 127) // 128 if blocks else s      # block-scale tensors count rows in blocks of 128
                self.weight_loader(param, loaded.narrow(0, off, n), i)
                off += n
            return
        n = self.local_sizes[shard_id]
        scale_like = param.dim() == 2 and param.shape[0] != sum(self.local_sizes) and param.dtype == torch.float32
        if scale_like:
            # block-scale tensor: rows are counted in blocks of 128 output features
            blk = 128
            nb = (n + blk - 1) // blk
            off = sum((s + blk - 1) // blk for s in self.local_sizes[:shard_id])
            src = loaded.narrow(0, self.tp_rank * nb, nb)
            param.data[off:off + nb].copy_(src)
            return
        src = loaded.narrow(0, self.tp_rank * n, n)
        rows = self._rows_of(shard_id).to(param.device)
        if param.dim() == 1:
            param.data[rows] = src.to(param.dtype).to(param.device)
        else:
            param.data[rows] = src.to(param.device).to(param.dtype) if param.dtype != torch.float8_e4m3fn \
                else src.to(param.device)


class QKVParallelLinear(LinearBase):
    """Fused q/k/v projection; heads sharded across the group (KV heads are
    replicated when there are fewer of them than ranks)."""

    def __init__(self, hidden_size, head_dim, num_heads, num_kv_heads, bias=False,
                 dtype=torch.bfloat16, device=None, head_dim_v: Optional[int] = None, **kw):
        self.head_dim = head_dim
        self.head_dim_v = head_dim_v or head_dim
        self.total_heads, self.total_kv_heads = num_heads, num_kv_heads
        super().__init__(hidden_size,
                         num_heads * head_dim + num_kv_heads * (head_dim + self.head_dim_v), bias,
                         dtype, device, **kw)
        tp = self.tp_size
        assert num_heads % tp == 0
        self.num_heads = num_heads // tp
        if num_kv_heads >= tp:
            assert num_kv_heads % tp == 0
            self.num_kv_heads, self.kv_replicas = num_kv_heads // tp, 1
        else:
            assert tp % num_kv_heads == 0
            self.num_kv_heads, self.kv_replicas = 1, tp // num_kv_heads
        self.q_size = self.num_heads * head_dim
        self.k_size = self.num_kv_heads * head_dim
        self.v_size = self.num_kv_heads * self.head_dim_v
        self._create(hidden_size, self.q_size + self.k_size + self.v_size, device)

    def forward(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        qkv = None
        if not isinstance(x, torch.Tensor):
            qkv, x = _sharded_input(self, x)
        elif self.x_transform == "AllGather" and self.tp_size > 1:
            qkv = gathered_gemm(self, x)
        if qkv is None:
            x = apply_transform(x, self.x_transform, self.group)
            qkv = self.quant_method.apply(self, x, self.bias)
        return (qkv[:, : self.q_size], qkv[:, self.q_size: self.q_size + self.k_size],
                qkv[:, self.q_size + self.k_size:])

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        assert shard_id in ("q", "k", "v")
        if shard_id == "q":
            off, n, r = 0, self.q_size, self.tp_rank
        elif shard_id == "k":
            off, n, r = self.q_size, self.k_size, self.tp_rank // self.kv_replicas
        else:
            off, n, r = self.q_size + self.k_size, self.v_size, self.tp_rank // self.kv_replicas
        src = loaded.narrow(0, r * n, n)
        dst = param.data.narrow(0, off, n)
        dst.copy_(src if dst.dtype == torch.float8_e4m3fn else src.to(dst.dtype))


class RowParallelLinear(LinearBase):
    """Input features sharded across the group; partial sums are reduced
    (all-reduce, or reduce-scatter when the residual stream is token-sharded)."""

    def __init__(self, in_features, out_features, bias=False, dtype=torch.bfloat16, device=None,
                 reduce_results: bool = True, **kw):
        super().__init__(in_features, out_features, bias, dtype, device, **kw)
        assert in_features % self.tp_size == 0
        self.in_local = in_features // self.tp_size
        self.reduce_results = reduce_results
        if self.y_transform is None and reduce_results:
            self.y_transform = "AllReduce"
        self._create(self.in_local, out_features, device)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
                reduce=True):
        """``reduce=False`` returns this rank's partial sums; the caller then reduces them
        itself, typically fused with the following residual add + RMSNorm.  ``reduce="scatter"``:
        see below."""
        x = apply_transform(x, self.x_transform, self.group)
        bias = self.bias if self.tp_rank == 0 else None
        if reduce == "scatter":
            # token-sharded residual stream: the caller wants this rank's rows of the reduced
            # product.  With peer memory the GEMM epilogue pushes its tiles to the row owners
            # and a small kernel sums them (ReducedShard); otherwise the partial goes back and
            # the caller reduce-scatters it.
            symm = getattr(self.group.comm, "symm", None) if self.tp_size > 1 else None
            if (symm is not None and isinstance(self.quant_method, UnquantizedLinearMethod) and residual is None
                    and symm.can_gemm_reduce_scatter(x, self.weight)):
                return ReducedShard(symm.gemm_reduce_scatter(x, self.weight, self.bias))
            return self.quant_method.apply(self, x, bias)
        if self.tp_size == 1 or not self.reduce_results or not reduce:
            return self.quant_method.apply(self, x, bias, residual=residual)
        y = self.quant_method.apply(self, x, bias)
        y = apply_transform(y, self.y_transform, self.group)
        if residual is not None:
            y = y + residual
        return y

    def weight_loader(self, param: nn.Parameter, loaded: torch.Tensor, shard_id=None) -> None:
        if param.dim() == 1:
            param.data.copy_(loaded.to(param.dtype))
            return
        _copy_sharded(param, loaded, 1, self.tp_rank, self.tp_size)


def row_parallel_add_rms_norm(linear: "RowParallelLinear", x: torch.Tensor, norm, residual: torch.Tensor):
    """``residual += all_reduce(linear(x))``; returns (RMSNorm(residual), residual).

    With the group's peer-mapped memory and a decode-sized problem this is ONE kernel (GEMM,
    push all-reduce, residual add and norm: ``SymmetricMemory.gemm_all_reduce``); otherwise the
    projection runs unreduced and the reduction is fused with the add + norm."""
    from .norm import reduce_add_rms_norm
    group = linear.group
    symm = getattr(group.comm, "symm", None) if group.world_size > 1 else None
    if (symm is not None and linear.x_transform is None and isinstance(linear.quant_method, UnquantizedLinearMethod)
            and residual is not None and residual.is_contiguous() and symm.can_fuse_gemm(x, linear.weight)):
        bias = linear.bias if (linear.bias is not None) else None
        out = symm.gemm_all_reduce(x, linear.weight, bias, residual, norm.weight, norm.eps)
        return out, residual
    return reduce_add_rms_norm(norm, linear(x, reduce=False), residual, group)


def _copy_sharded(param: nn.Parameter, loaded: torch.Tensor, dim: int, rank: int, world: int) -> None:
    if param.dim() == 2 and param.dtype == torch.float32 and loaded.dtype == torch.float32 \
            and loaded.shape != param.shape and world > 1 and loaded.shape[dim] % world != 0:
        # block-scale tensor whose block count does not divide evenly: take the covering slice
        per = param.shape[dim]
        start = min(rank * per, loaded.shape[dim] - per)
        param.data.copy_(loaded.narrow(dim, start, per))
        return
    n = loaded.shape[dim] // world if loaded.shape[dim] != param.shape[dim] else loaded.shape[dim]
    src = loaded.narrow(dim, rank * n, n) if n != loaded.shape[dim] else loaded
    param.data.copy_(src if param.dtype == torch.float8_e4m3fn else src.to(param.dtype))
