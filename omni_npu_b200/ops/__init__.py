"""Device ops of the framework.

Every function takes torch tensors.  CUDA tensors run the hand-written sm_100a
kernels from ``_C.so`` (``torch.ops.omni_b200.*``); a missing extension on a
CUDA tensor is an error, never a silent fallback.  CPU tensors run the fp32
PyTorch references in :mod:`omni_npu_b200.ops.ref`, which is what the gloo /
no-GPU plumbing tests exercise.

``launch_count()`` returns how many of this library's kernels have been
launched (graph replays add the number of kernels captured in the graph).
"""
from __future__ import annotations

import os
import threading
from pathlib import Path
from typing import Optional, Tuple

import torch

from . import ref

_PKG = Path(__file__).resolve().parent.parent
_LIB = _PKG / "_C.so"
_loaded = False
_load_error: Optional[str] = None
_lock = threading.Lock()


def load_extension(required: bool = False) -> bool:
    """Load ``_C.so`` (idempotent).  Returns whether the ops are available."""
    global _loaded, _load_error
    if _loaded:
        return True
    with _lock:
        if _loaded:
            return True
        if not _LIB.exists():
            _load_error = f"{_LIB} not built (run `python -m omni_npu_b200._build`)"
        else:
            try:
                torch.ops.load_library(str(_LIB))
                _loaded = True
            except Exception as e:  # pragma: no cover - depends on the box
                _load_error = f"loading {_LIB} failed: {e}"
    if required and not _loaded:
        raise RuntimeError("omni_npu_b200 CUDA extension unavailable: " + str(_load_error))
    return _loaded


def _C():
    load_extension(required=True)
    return torch.ops.omni_b200


# --------------------------------------------------------------- launch count
class _Counter:
    __slots__ = ("n", "capturing", "captured")

    def __init__(self) -> None:
        self.n = 0
        self.capturing = False
        self.captured = 0


_counter = _Counter()


def _count(k: int = 1) -> None:
    if _counter.capturing:
        _counter.captured += k
    else:
        _counter.n += k


def launch_count() -> int:
    return _counter.n


def add_launches(k: int) -> None:
    _counter.n += k


class count_capture:
    """Context manager used around CUDA-graph capture: kernels launched inside are
    tallied separately so each replay can add them to the global count."""

    def __enter__(self):
        self._saved = (_counter.capturing, _counter.captured)
        _counter.capturing, _counter.captured = True, 0
        return self

    def __exit__(self, *exc):
        self.kernels = _counter.captured
        _counter.capturing, _counter.captured = self._saved
        return False


# ------------------------------------------------------------------ workspaces
class _DeviceState:
    """Per-device persistent scratch for split-K GEMM and split-KV decode plus
    the kernel status word.  Allocated once, before any graph capture."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        # a plain (not inference-mode) tensor: the first kernel often runs under inference_mode, and an
        # inference tensor could not be cleared later by a caller outside that mode
        with torch.inference_mode(False):
            self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.gemm_ws_bytes = int(os.environ.get("OMNI_B200_GEMM_WS_MB", "64")) << 20
        self.gemm_ws = {}
        self.counters = {}
        self.attn_scratch = {}
        self.work_counters = {}
        self.plans = {}

    def gemm_workspace(self, stream_id: int, nbytes: int, ncounters: int):
        ws = self.gemm_ws.get(stream_id)
        if ws is None or ws.numel() < nbytes:
            ws = torch.empty(max(nbytes, self.gemm_ws_bytes), dtype=torch.uint8, device=self.device)
            self.gemm_ws[stream_id] = ws
        cnt = self.counters.get(stream_id)
        if cnt is None or cnt.numel() < ncounters:
            cnt = torch.zeros(max(ncounters, 65536), dtype=torch.int32, device=self.device)
            self.counters[stream_id] = cnt
        return ws, cnt

    def work_counter(self, stream_id: int):
        """Two zeroed ints per stream for kernels that hand out work items through a device
        counter; the kernel that uses them puts them back to zero before it ends."""
        wc = self.work_counters.get(stream_id)
        if wc is None:
            with torch.inference_mode(False):
                wc = torch.zeros(2, dtype=torch.int32, device=self.device)
            self.work_counters[stream_id] = wc
        return wc

    def decode_scratch(self, stream_id: int, nbytes: int):
        sc = self.attn_scratch.get(stream_id)
        if sc is None or sc.numel() < nbytes:
            sc = torch.empty(max(nbytes, 32 << 20), dtype=torch.uint8, device=self.device)
            self.attn_scratch[stream_id] = sc
        return sc


_states = {}


def device_state(device: torch.device) -> _DeviceState:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _states.get(idx)
    if st is None:
        st = _DeviceState(torch.device("cuda", idx))
        _states[idx] = st
    return st


def check_status(device: Optional[torch.device] = None) -> None:
    """Raise if any kernel recorded a bounded-wait timeout since the last check
    (synchronises the device)."""
    for st in _states.values():
        if device is not None and st.device != device:
            continue
        code = int(st.status.item())
        if code != 0:
            st.status.zero_()
            raise RuntimeError(f"omni_npu_b200 kernel reported status {code} (bounded wait expired)")


# ------------------------------------------------------------------------ GEMM
# smallest M routed to the CTA-pair GEMM (0 = never); prefill-sized problems only
PAIR_MIN_M = int(os.environ.get("OMNI_B200_GEMM_PAIR_MIN_M", "1024"))
# Plain bf16 products (no bias, residual, SwiGLU, scales or fused collective) of a decode-sized batch
# whose plan here is a cluster split-K: "library" hands them to cuBLAS, "own" keeps them on
# gemm_tcgen05_kernel.  Measured at M = 128 inside a CUDA graph (us, own / cuBLAS): 4096 x 4096
# 19.0 / 10.6, 6144 x 4096 20.2 / 12.6, 4096 x 14336 37.4 / 26.3: every CTA of the own kernel re-reads
# the 128-row activation slab of its K slice and the K slices meet in a 3-4 us exchange, which a
# library kernel that may share one activation load between the CTAs of a cluster does not pay.
# Row counts below 64 stay on the own kernel (not measured against the library there, and its result
# for a row does not depend on how many rows share the launch, which padded CUDA-graph steps rely on).
SMALL_M_GEMM = os.environ.get("OMNI_B200_SMALL_M_GEMM", "library")
SMALL_M_LIBRARY_ROWS = (64, 256)

def library_small_m(m: int, cluster_split_plan: bool, plain_bf16: bool) -> bool:
    """Whether ``gemm`` hands a product to cuBLAS: only a plain bf16 product (nothing fused, no forced
    tile or split), only when this package's plan for it is a cluster split-K, only for the row
    counts the comparison was measured on, and only while ``OMNI_B200_SMALL_M_GEMM`` says so."""
    return (SMALL_M_GEMM == "library" and plain_bf16 and cluster_split_plan
            and SMALL_M_LIBRARY_ROWS[0] <= m <= SMALL_M_LIBRARY_ROWS[1])


def gemm(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
         residual: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
         swiglu: bool = False, bn: int = 0, splits: int = 0, max_ctas: int = 0,
         pair: Optional[bool] = None) -> torch.Tensor:
    """``a[M,K] @ w[N,K].T`` (+bias, +residual).  bf16 or float8_e4m3fn inputs,
    fp32 accumulation, bf16 (default) or fp32 output.  ``swiglu`` fuses
    silu(gate)*up for weights laid out by :func:`ref.interleave_gate_up`.
    ``splits`` > 1 forces split-K (as a thread-block cluster when it fits), a
    negative value forces the workspace variant with |splits| slices.
    ``pair`` selects the CTA-pair kernel (256-row tiles over two SMs); by default
    it runs for M >= PAIR_MIN_M when no split-K was asked for."""
    if not a.is_cuda:
        return ref.gemm(a, w, bias, residual, out_dtype, swiglu)
    C = _C()
    st = device_state(a.device)
    m, k = a.shape
    n = w.shape[0]
    if pair is None:
        pair = PAIR_MIN_M > 0 and m >= PAIR_MIN_M and splits == 0 and bn == 0
    if pair:
        n_eff = n
        pbn = bn if bn > 0 else (256 if n_eff >= 256 else max(32, ((n_eff + 31) // 32) * 32))
        _count(1)
        return C.gemm_pair(a, w, bias, residual, out_dtype == torch.float32, swiglu, pbn, st.status, max_ctas)
    key = (m, n, k, a.dtype.itemsize, swiglu, bn, splits)
    plan = st.plans.get(key)
    if plan is None:
        plan = C.gemm_plan(m, n, k, a.dtype.itemsize, swiglu, bn, 1 if swiglu else splits)
        st.plans[key] = plan
    pbn, psplits, ws_bytes, ncnt, cluster = plan
    if library_small_m(m, bool(cluster), bias is None and residual is None and not swiglu and bn == 0
                       and splits == 0 and a.dtype == torch.bfloat16 and out_dtype in (None, torch.bfloat16)):
        return torch.nn.functional.linear(a, w)          # a library kernel: not counted as a launch of ours
    ws = cnt = None
    if psplits > 1 and not cluster:
        ws, cnt = st.gemm_workspace(torch.cuda.current_stream(a.device).cuda_stream, ws_bytes, ncnt)
    _count(1)
    return C.gemm(a, w, bias, residual, out_dtype == torch.float32, swiglu, pbn, psplits,
                  bool(cluster), ws, cnt, st.status, max_ctas)


def quant_int8_per_token(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dynamic symmetric int8 quantisation, one scale per row: (q int8 [T,H], scale fp32 [T])."""
    if not x.is_cuda:
        return ref.quant_int8_per_token(x)
    _count(1)
    return _C().quant_int8_per_token(x)


def gemm_fp8_block(a_q: torch.Tensor, a_scale: torch.Tensor, w_q: torch.Tensor, w_scale: torch.Tensor,
                   bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                   out_dtype: Optional[torch.dtype] = None, max_ctas: int = 0) -> torch.Tensor:
    """Block-scaled e4m3 product: ``a_q`` [M,K] with one scale per (row, 128 columns), ``w_q`` [N,K]
    with one scale per 128 x 128 block; each 128-wide K block is scaled before accumulation."""
    if not a_q.is_cuda:
        return ref.gemm_fp8_block(a_q, a_scale, w_q, w_scale, bias, residual, out_dtype)
    st = device_state(a_q.device)
    _count(1)
    return _C().gemm_fp8_block(a_q, a_scale.contiguous(), w_q, w_scale.contiguous(), bias, residual,
                               out_dtype == torch.float32, st.status, max_ctas)


def grouped_gemm_fp8_block(a_q: torch.Tensor, a_scale: torch.Tensor, w_q: torch.Tensor, w_scale: torch.Tensor,
                           expert_offsets: torch.Tensor, swiglu: bool = False, up_scale_row0: int = 0,
                           max_ctas: int = 0) -> torch.Tensor:
    """Per-expert block-scaled e4m3 GEMM: rows ``expert_offsets[e]:expert_offsets[e+1]`` of ``a_q`` times
    ``w_q[e].T`` with ``w_scale[e]`` (one scale per 128 x 128 block).  ``swiglu``: gate / up rows of
    ``w_q`` are interleaved in groups of 8 and the result is ``silu(gate) * up``; the scale rows are the
    gate blocks followed, from row ``up_scale_row0``, by the up blocks."""
    if not a_q.is_cuda:
        return ref.grouped_gemm_fp8_block(a_q, a_scale, w_q, w_scale, expert_offsets, swiglu, up_scale_row0)
    st = device_state(a_q.device)
    _count(1)
    return _C().grouped_gemm_fp8_block(a_q, a_scale.contiguous(), w_q, w_scale.contiguous(), expert_offsets, swiglu,
                                       up_scale_row0, st.status, max_ctas)


def dsa_indexer_topk(q: torch.Tensor, w: torch.Tensor, index_cache: torch.Tensor, block_tables: torch.Tensor,
                     positions: torch.Tensor, num_seqs: int, topk: int, cu_q: Optional[torch.Tensor] = None,
                     q_len: int = 1, max_ctx: int = 0, max_q: int = 0, return_scores: bool = False):
    """Sparse-attention indexer: ``score[t, j] = sum_h w[t, h] * relu(q[t, h] . k[j])`` over the cached
    keys ``j <= positions[t]`` of the token's sequence, then the ``topk`` best positions per token
    (int32 [T, topk], unordered, -1 padded).  ``cu_q`` [B + 1] gives the first query token of each
    sequence; without it every sequence has ``q_len`` tokens.  ``max_ctx`` / ``max_q`` bound the longest
    context / query run (both default to the largest possible value)."""
    t, h = q.shape[0], q.shape[1]
    bs = index_cache.shape[1]
    if max_ctx <= 0:
        max_ctx = block_tables.shape[1] * bs
    if max_q <= 0:
        max_q = q_len if cu_q is None else t
    if not q.is_cuda:
        return ref.dsa_indexer_topk(q, w, index_cache, block_tables, positions, num_seqs, topk, cu_q, q_len,
                                    return_scores)
    supported = (q.shape[2] == 128 and h % 16 == 0 and h <= 256 and bs % 8 == 0 and
                 (bs % 128 == 0 if bs >= 128 else 128 % bs == 0))
    if not supported:
        raise RuntimeError(f"dsa_indexer_topk: unsupported shape (heads {h}, dim {q.shape[2]}, page {bs})")
    st = device_state(q.device)
    _count(2)
    sel, scores = _C().dsa_indexer(q.contiguous(), w.float().contiguous(), index_cache, block_tables, cu_q,
                                   positions, num_seqs, q_len, max_ctx, max_q, topk, st.status)
    return (sel, scores) if return_scores else sel


def rms_norm_quant(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None,
                   kind: str = "int8", want_bf16: bool = False):
    """RMSNorm of ``x`` (or of ``x + residual``, which is written back to ``residual``) fused with
    per-token dynamic quantisation to int8 (scale = amax/127) or e4m3 (scale = amax/448).
    Returns (q [T,H], scale fp32 [T], normalised bf16 [T,H] or None)."""
    if not x.is_cuda:
        return ref.rms_norm_quant(x, weight, eps, residual, kind, want_bf16)
    _count(1)
    q, s, out = _C().rms_norm_quant(x, residual, weight, eps, 1 if kind == "fp8" else 2, want_bf16)
    return q, s, (out if want_bf16 else None)


def silu_and_mul_quant(x: torch.Tensor, kind: str = "int8") -> Tuple[torch.Tensor, torch.Tensor]:
    """``silu(x[:, :I]) * x[:, I:]`` fused with per-token dynamic quantisation: (q [T,I], scale [T])."""
    if not x.is_cuda:
        return ref.silu_and_mul_quant(x, kind)
    _count(1)
    return _C().silu_and_mul_quant(x, 1 if kind == "fp8" else 2)


def gemm_scaled(a_q: torch.Tensor, w_q: torch.Tensor, a_scale: torch.Tensor, w_scale: torch.Tensor,
                bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, bn: int = 0, max_ctas: int = 0) -> torch.Tensor:
    """``(a_q @ w_q.T) * a_scale[:, None] * w_scale[None, :]`` (+bias, +residual) for int8 or
    e4m3 operands; integer products accumulate exactly in 32 bits on the tensor cores."""
    if not a_q.is_cuda:
        return ref.gemm_scaled(a_q, w_q, a_scale, w_scale, bias, residual, out_dtype)
    st = device_state(a_q.device)
    if bn <= 0:
        n = w_q.shape[0]
        bn = 256 if n >= 2048 else (128 if n >= 128 else max(16, (n + 15) // 16 * 16))
    _count(1)
    return _C().gemm_scaled(a_q, w_q, a_scale.contiguous(), w_scale.reshape(-1).contiguous(), bias, residual,
                            out_dtype == torch.float32, bn, st.status, max_ctas)


def grouped_gemm(a: torch.Tensor, w: torch.Tensor, expert_offsets: torch.Tensor,
                 swiglu: bool = False, bn: int = 0, max_ctas: int = 0) -> torch.Tensor:
    """Per-expert GEMM: rows expert_offsets[e]:expert_offsets[e+1] of ``a`` times ``w[e].T``."""
    if not a.is_cuda:
        return ref.grouped_gemm(a, w, expert_offsets, swiglu)
    if bn <= 0:
        n = w.shape[1]
        bn = 256 if n % 256 == 0 else (128 if n % 128 == 0 else (64 if n % 64 == 0 else 32))
    st = device_state(a.device)
    _count(1)
    return _C().grouped_gemm(a, w, expert_offsets, swiglu, bn, st.status, max_ctas)


# ------------------------------------------------------------- norm/activation
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    if not x.is_cuda:
        return ref.rms_norm(x, w, eps)
    _count(1)
    return _C().rms_norm(x, w, eps)


def fused_add_rms_norm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor,
                       eps: float) -> torch.Tensor:
    """residual <- x + residual (in place); returns RMSNorm(residual) * w."""
    if not x.is_cuda:
        return ref.fused_add_rms_norm(x, residual, w, eps)
    _count(1)
    return _C().fused_add_rms_norm(x, residual, w, eps)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        return ref.silu_and_mul(x)
    _count(1)
    return _C().silu_and_mul(x)


def quant_fp8_1x128(x: torch.Tensor, ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    if not x.is_cuda:
        return ref.quant_fp8_1x128(x, ue8m0)
    _count(1)
    return _C().quant_fp8_1x128(x, ue8m0)


# ------------------------------------------------------------------ rope/cache
def rope_qk_(q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
             head_dim: int, rot_dim: int, neox: bool = True,
             mrope_section: Optional[Tuple[int, int, int]] = None,
             mrope_interleaved: bool = False) -> None:
    """In-place rotary embedding of q [T,Hq*D] and k [T,Hk*D].  With ``mrope_section`` the positions
    are [3, T] (temporal, row, column); plain [T] positions (text-only steps of a multimodal model)
    rotate every frequency with the one position, which is what three equal axes would give."""
    if mrope_section is not None and positions.dim() == 1:
        mrope_section = None
    if not q.is_cuda:
        kk = k if k.numel() else q[:, :head_dim]
        qo, ko = ref.rope_qk(q, kk, positions, cos_sin, head_dim, rot_dim, neox, mrope_section,
                             mrope_interleaved)
        q.copy_(qo)
        if k.numel():
            k.copy_(ko)
        return
    sec_t, sec_h = (-1, -1) if mrope_section is None else (mrope_section[0], mrope_section[1])
    _count(1)
    _C().rope_qk(q, k, positions, cos_sin, head_dim, rot_dim, neox, sec_t, sec_h, mrope_interleaved)


def rope_cache_gqa_(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor,
                    v_cache: torch.Tensor, positions: torch.Tensor, slot_mapping: torch.Tensor,
                    cos_sin: torch.Tensor, head_dim: int, rot_dim: int, neox: bool = True) -> None:
    """RoPE on q (in place) and k, then k / v stored into the paged cache."""
    if not q.is_cuda:
        qo, ko = ref.rope_qk(q, k, positions, cos_sin, head_dim, rot_dim, neox)
        q.copy_(qo)
        ref.gqa_cache_write(ko, v, k_cache, v_cache, slot_mapping)
        return
    _count(1)
    _C().rope_cache_gqa(q, k, v, k_cache, v_cache, positions, slot_mapping, cos_sin, head_dim,
                        rot_dim, neox)


def gqa_cache_write(k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    slot_mapping: torch.Tensor) -> None:
    if not k.is_cuda:
        return ref.gqa_cache_write(k, v, k_cache, v_cache, slot_mapping)
    _count(1)
    _C().gqa_cache_write(k, v, k_cache, v_cache, slot_mapping)


def paged_scatter_rows(dst: torch.Tensor, src: torch.Tensor, slot_mapping: torch.Tensor) -> None:
    if not src.is_cuda:
        return ref.paged_scatter_rows(dst, src, slot_mapping)
    _count(1)
    _C().paged_scatter_rows(dst, src, slot_mapping)


def mla_kv_rmsnorm_rope_cache(kv_c: torch.Tensor, k_pe: torch.Tensor, w: torch.Tensor,
                              cache: torch.Tensor, positions: torch.Tensor,
                              slot_mapping: torch.Tensor, cos_sin: torch.Tensor, eps: float,
                              neox: bool = False, want_outputs: bool = False):
    """RMSNorm(kv_c) and RoPE(k_pe) written into the paged latent cache row
    [norm(kv_c) | rope(k_pe)]; optionally also returned in token order."""
    t, l = kv_c.shape
    r = k_pe.shape[1]
    if not kv_c.is_cuda:
        kn = ref.rms_norm(kv_c, w, eps)
        half = r // 2
        cs = cos_sin[positions.long()]
        pe = ref._rope_one(k_pe.view(t, 1, r), cs[:, :half], cs[:, half:], r, neox).view(t, r)
        ref.paged_scatter_rows(cache, torch.cat([kn, pe], dim=-1), slot_mapping)
        return (kn, pe) if want_outputs else None
    kv_out = torch.empty_like(kv_c, memory_format=torch.contiguous_format) if want_outputs else None
    pe_out = torch.empty((t, r), dtype=k_pe.dtype, device=k_pe.device) if want_outputs else None
    _count(1)
    _C().mla_kv_rmsnorm_rope_cache(kv_c, k_pe, w, cache, kv_out, pe_out, positions, slot_mapping,
                                   cos_sin, eps, neox)
    return (kv_out, pe_out) if want_outputs else None


# ------------------------------------------------------------------- attention
def _pack_window(window: int, sink: int) -> int:
    """The kernels take the sliding window in the low 20 bits of one integer and the
    number of leading sink tokens above them."""
    if window >= (1 << 20) or sink >= (1 << 11) or window < 0 or sink < 0:
        raise ValueError(f"window {window} / sink {sink} out of range")
    return window | (sink << 20)


PREFILL_TCGEN05 = os.environ.get("OMNI_B200_PREFILL_TCGEN05", "1") != "0"


def gqa_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                block_tables: torch.Tensor, cu_q: torch.Tensor, seq_lens: torch.Tensor,
                num_seqs: int, max_q_len: int, num_q_heads: int, scale: float, causal: bool = True,
                window: int = 0, return_lse: bool = False, sink: int = 0, tcgen05: Optional[bool] = None):
    """Variable-length attention of this step's queries over the paged cache
    (which already holds this step's keys/values).  ``sink``: the first ``sink`` cached
    tokens of every sequence are attention sinks, visible through any sliding window.
    Head size 128 without window / sinks runs on tcgen05 with TMEM accumulators
    (``tcgen05=False`` or ``OMNI_B200_PREFILL_TCGEN05=0`` selects the ``mma.sync`` kernel)."""
    if not q.is_cuda:
        return ref.paged_attention(q, k_cache, v_cache, block_tables[:num_seqs], cu_q[: num_seqs + 1],
                                   seq_lens[:num_seqs], num_q_heads, scale, causal, window, return_lse, sink)
    _count(1)
    tc = PREFILL_TCGEN05 if tcgen05 is None else tcgen05
    out, lse = _C().gqa_prefill(q, k_cache, v_cache, block_tables, cu_q, seq_lens, num_seqs,
                                max_q_len, num_q_heads, scale, causal, _pack_window(window, sink), return_lse,
                                tc and window == 0 and sink == 0, device_state(q.device).status)
    return (out, lse) if return_lse else out


def merge_attn_states(outs: torch.Tensor, lses: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Combine N partial attention results over disjoint key sets.  ``outs`` [N, T, H, D],
    ``lses`` [N, T, H] (natural log-sum-exp of the scaled scores, -inf where a partial saw no
    key) -> (out [T, H, D], lse [T, H])."""
    if not outs.is_cuda:
        return ref.merge_attn_states(outs, lses)
    _count(1)
    return _C().lse_merge(outs.contiguous(), lses.float().contiguous())


def gather_cache(cache: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor) -> torch.Tensor:
    """Contiguous copy of the cached rows of each sequence, one sequence after another:
    cache [blocks, block_size, ...] -> [sum(seq_lens), ...]."""
    lens = seq_lens.tolist()
    total, longest = sum(lens), max(lens) if lens else 0
    if not cache.is_cuda:
        return ref.gather_cache(cache, block_tables, seq_lens)
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32, device=cache.device)
    cu[1:] = seq_lens.to(cache.device).cumsum(0)
    _count(1)
    return _C().gather_cache(cache, block_tables.contiguous(), cu, total, longest)


def decode_splits(num_seqs: int, num_kv_heads: int, max_seq_len: int, sms: int = 148) -> int:
    """Split-KV factor.  With at least one (sequence, kv head) item per SM the keys are not split:
    a split brings its own set-up and first-tile latency (4.4 us) and the merge kernel, and measured
    on 128 sequences x 1152 keys one split wins for 8, 4 and 2 kv heads (2 kv heads: 38.9 us against
    48.1 us with two).  With fewer items than SMs the keys are split until about 2.5 CTAs share an
    SM (one CTA alone streams at ~23 GB/s, an SM needs 45 GB/s), at least 256 keys per split."""
    base = max(1, num_seqs * num_kv_heads)
    if base >= sms:
        return 1
    want = (5 * sms // 2 + base - 1) // base
    cap = max(1, max_seq_len // 256)
    return max(1, min(want, cap, 16))


def decode_splits_persistent(num_seqs: int, num_kv_heads: int, max_seq_len: int, sms: int = 148) -> int:
    """Split-KV factor for the persistent decode kernel (two CTAs per SM walk the items
    sequence x kv head x split): the smallest factor whose item count fills the resident CTAs to
    within 7 % of a whole number of rounds, with at least 256 keys per split; when none gets that
    close, the one that comes closest."""
    slots = 2 * sms
    base = max(1, num_seqs * num_kv_heads)
    cap = max(1, min(16, max_seq_len // 256))
    best, best_eff = 1, 0.0
    for s in range(1, cap + 1):
        per = base * s / slots
        eff = per / max(1, -(-base * s // slots))
        if eff >= 0.93:
            return s
        if eff > best_eff + 1e-9:
            best, best_eff = s, eff
    return best


# Decode attention work distribution, OMNI_B200_DECODE_PERSISTENT = 0 | 1 | 2:
#   0  one CTA per (sequence, kv head, split) item;
#   1  persistent CTAs that take whole items from a device counter (measured 2-5 % slower than 0 on
#      128 sequences x 1152 keys x 8 kv heads: 130 us against 127 us);
#   2  persistent CTAs over a balanced cut of all key tiles: whole items leave the last round of the
#      resident CTAs partly empty (1024 items on 444 CTAs: three rounds for 2.3 rounds of work), the
#      balanced cut does not; pieces of items that cross a cut go through fp32 scratch and a merge
#      kernel.  Measured 127.5 us on the same shapes (4 / 2 kv heads: 80.9 / 52.2 us against 69.7 /
#      38.9 us for mode 0): the memory system is saturated with every resident CTA streaming, so the
#      rounds saved do not shorten the call.
DECODE_PERSISTENT = int(os.environ.get("OMNI_B200_DECODE_PERSISTENT", "0") or 0)


def decode_balanced_plan(seq_lens, num_kv_heads: int, ctas: int, tile: int = 64):
    """Host restatement of the balanced cut that ``gqa_decode_persist_kernel`` (mode 2) and its merge
    kernel derive on the device, for tests and capacity checks.  Returns one list per CTA of
    ``(sequence, kv head, first tile, tiles, scratch slot or -1)``."""
    nb = [max(1, -(-int(n) // tile)) for n in seq_lens]
    total = sum(nb) * num_kv_heads
    per = max(2, -(-total // ctas))
    starts, acc = [], 0
    for n in nb:
        starts.append(acc)
        acc += n * num_kv_heads
    plan = []
    for c in range(ctas):
        x, x_end = c * per, min(total, (c + 1) * per)
        segs = []
        while x < x_end:
            b = max(i for i in range(len(nb)) if starts[i] <= x)
            off = x - starts[b]
            kvh, t = divmod(off, nb[b])
            n = min(nb[b] - t, x_end - x)
            whole = t == 0 and n == nb[b]
            segs.append((b, kvh, t, n, -1 if whole else 2 * c + (0 if not segs else 1)))
            x += n
        plan.append(segs)
    return plan


def gqa_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
               block_tables: torch.Tensor, seq_lens: torch.Tensor, num_seqs: int, num_q_heads: int,
               scale: float, q_len: int = 1, window: int = 0, splits: int = 0,
               max_seq_len: int = 0, sink: int = 0, persistent=None) -> torch.Tensor:
    """Decode attention: q_len (usually 1) new tokens per sequence, sequences laid
    out back to back in q.  ``persistent`` (default: ``DECODE_PERSISTENT``): 0 / False = one CTA per
    item, 1 / True = persistent CTAs fed by a device counter, 2 = persistent CTAs over a balanced cut
    of the key tiles (``splits`` is ignored)."""
    if not q.is_cuda:
        cu = torch.arange(0, (num_seqs + 1) * q_len, q_len, dtype=torch.int32, device=q.device)
        return ref.paged_attention(q, k_cache, v_cache, block_tables[:num_seqs], cu,
                                   seq_lens[:num_seqs], num_q_heads, scale, True, window, False, sink)
    C = _C()
    hk, d = k_cache.shape[1], k_cache.shape[3]
    persistent = int(DECODE_PERSISTENT if persistent is None else persistent)
    st = device_state(q.device)
    stream_id = torch.cuda.current_stream(q.device).cuda_stream
    if persistent == 2:
        nbytes = C.gqa_decode_balanced_scratch_bytes(d, (num_q_heads // hk) * q_len)
        _count(2)
        return C.gqa_decode(q, k_cache, v_cache, block_tables, seq_lens, num_seqs, q_len, num_q_heads,
                            scale, _pack_window(window, sink), 1, st.decode_scratch(stream_id, nbytes),
                            st.status, 2, None)
    if splits <= 0:
        bound = max_seq_len if max_seq_len > 0 else block_tables.shape[1] * k_cache.shape[2]
        splits = (decode_splits_persistent if persistent else decode_splits)(num_seqs, hk, bound)
    scratch = None
    if splits > 1:
        nbytes = C.gqa_decode_scratch_bytes(num_seqs, hk, d, splits)
        scratch = st.decode_scratch(stream_id, nbytes)
    _count(2 if splits > 1 else 1)
    return C.gqa_decode(q, k_cache, v_cache, block_tables, seq_lens, num_seqs, q_len, num_q_heads,
                        scale, _pack_window(window, sink), splits, scratch, st.status, persistent,
                        st.work_counter(stream_id) if persistent else None)


# -------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor) -> torch.Tensor:
    if not logits.is_cuda:
        return ref.argmax(logits)
    _count(1)
    return _C().argmax(logits)


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           top_k: Optional[torch.Tensor] = None, top_p: Optional[torch.Tensor] = None,
           seeds: Optional[torch.Tensor] = None, step_offset: Optional[torch.Tensor] = None,
           generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Temperature / top-k / top-p sampling; rows with temperature < 1e-5 are greedy."""
    if not logits.is_cuda:
        return ref.sample(logits, temperature, top_k, top_p, generator, seeds, step_offset)
    _count(1)
    return _C().sample(logits, temperature, top_k, top_p, seeds, step_offset)


def spec_verify(draft: torch.Tensor, target: torch.Tensor, bonus: torch.Tensor, cu: torch.Tensor,
                max_spec: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Accept draft tokens while they equal the target's tokens (see ref.spec_verify)."""
    if not draft.is_cuda:
        return ref.spec_verify(draft, target, bonus, cu, max_spec)
    _count(1)
    return _C().spec_verify(draft.int().contiguous(), target.int().contiguous(), bonus.int().contiguous(),
                            cu.int().contiguous(), max_spec)


# ------------------------------------------------------------------------- MoE
def moe_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], k: int, sigmoid: bool = False,
             n_group: int = 1, topk_group: int = 1, renorm: bool = False,
             scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Router top-k (softmax or sigmoid scores, optional bias correction and
    group-limited selection)."""
    if not logits.is_cuda:
        return ref.moe_topk(logits, bias, k, sigmoid, n_group, topk_group, renorm, scale)
    _count(1)
    return _C().moe_topk(logits.contiguous(), bias, k, sigmoid, n_group, topk_group, renorm, scale)


def mla_decode(q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, seq_lens: torch.Tensor,
               num_seqs: int, num_heads: int, scale: float, q_len: int = 1,
               topk_indices: Optional[torch.Tensor] = None, splits: int = 0,
               max_seq_len: int = 0, return_lse: bool = False):
    """Absorbed multi-head latent attention (MQA over the 576-wide latent cache);
    optionally restricted to ``topk_indices`` (sparse attention).  ``return_lse`` also returns
    the natural log-sum-exp of the scaled scores [T, N] (for merging partial results)."""
    if not q.is_cuda:
        return ref.mla_decode(q, cache, block_tables[:num_seqs], seq_lens[:num_seqs], num_seqs, q_len,
                              num_heads, scale, topk_indices, return_lse)
    C = _C()
    st = device_state(q.device)
    t = num_seqs * q_len
    tiles = (num_heads + 15) // 16
    if splits <= 0:
        bound = topk_indices.shape[1] if topk_indices is not None else (
            max_seq_len if max_seq_len > 0 else block_tables.shape[1] * cache.shape[1])
        splits = max(1, min((2 * 148 + t * tiles - 1) // max(1, t * tiles), max(1, bound // 256), 16))
    scratch = None
    if splits > 1:
        nbytes = C.mla_decode_scratch_bytes(t, num_heads, splits)
        scratch = st.decode_scratch(torch.cuda.current_stream(q.device).cuda_stream, nbytes)
    _count(2 if splits > 1 else 1)
    out, lse = C.mla_decode(q, cache, block_tables, seq_lens, topk_indices, num_seqs, q_len, num_heads, scale,
                            splits, scratch, st.status, return_lse)
    return (out, lse) if return_lse else out


# ------------------------------------------------------------------ KV transfer
def kv_p2p_copy(desc: torch.Tensor, src_blocks: torch.Tensor, dst_blocks: torch.Tensor,
                max_block_bytes: int) -> None:
    """One launch copies blocks ``src_blocks[i] -> dst_blocks[i]`` for every cache
    tensor described by ``desc`` (int64 [n,3]: source base, destination base, block
    bytes).  Sources may be another GPU's memory mapped through CUDA IPC."""
    _count(1)
    _C().kv_p2p_copy(desc, src_blocks, dst_blocks, int(max_block_bytes))
