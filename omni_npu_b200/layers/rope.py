"""Rotary position embedding family.

Every variant only differs in the inverse frequencies / magnitude scale it
bakes into a ``[max_pos, rot_dim]`` fp32 table (cos | sin); applying the
rotation is one kernel shared by all of them.  ``get_rope`` is the factory
keyed on the HF ``rope_scaling`` dictionary, covering default, linear,
dynamic NTK (by factor or fixed alpha), llama3, mllama4, YaRN, DeepSeek-YaRN, longrope,
xdrope (text positions) and (interleaved) M-RoPE
(reference: omni_npu/v1/layers/rotary_embedding/__init__.py:26-292 and
omni_npu/layers/rotary_embedding/*.py).
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch
from torch import nn

from .. import ops
from ..ops import ref


def _base_inv_freq(rot_dim: int, base: float) -> torch.Tensor:
    return 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))


def yarn_find_correction_dim(num_rot: float, dim: int, base: float, max_pos: int) -> float:
    return (dim * math.log(max_pos / (num_rot * 2 * math.pi))) / (2 * math.log(base))


def yarn_find_correction_range(low_rot: float, high_rot: float, dim: int, base: float,
                               max_pos: int) -> Tuple[int, int]:
    low = math.floor(yarn_find_correction_dim(low_rot, dim, base, max_pos))
    high = math.ceil(yarn_find_correction_dim(high_rot, dim, base, max_pos))
    return max(low, 0), min(high, dim - 1)


def yarn_linear_ramp_mask(low: float, high: float, dim: int) -> torch.Tensor:
    if low == high:
        high += 0.001
    return ((torch.arange(dim, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)


def yarn_get_mscale(scale: float = 1.0, mscale: float = 1.0) -> float:
    if scale <= 1:
        return 1.0
    return 0.1 * mscale * math.log(scale) + 1.0


class RotaryEmbedding(nn.Module):
    """Holds the cos/sin table and applies the rotation to q and k in place."""

    def __init__(self, head_dim: int, rot_dim: int, max_position: int, base: float,
                 is_neox: bool = True, inv_freq: Optional[torch.Tensor] = None, mscale: float = 1.0,
                 mrope_section: Optional[Tuple[int, int, int]] = None,
                 mrope_interleaved: bool = False, device=None) -> None:
        super().__init__()
        self.head_dim, self.rot_dim = head_dim, rot_dim
        self.max_position, self.base = max_position, base
        self.is_neox = is_neox
        self.mscale = mscale
        self.mrope_section = mrope_section
        self.mrope_interleaved = mrope_interleaved
        inv = inv_freq if inv_freq is not None else _base_inv_freq(rot_dim, base)
        cache = ref.build_cos_sin_cache(rot_dim, max_position, base, inv, mscale)
        self.register_buffer("cos_sin_cache", cache.to(device) if device is not None else cache,
                             persistent=False)

    def get_cos_sin(self, positions: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        cs = self.cos_sin_cache[positions.long()]
        half = self.rot_dim // 2
        return cs[..., :half], cs[..., half:]

    def forward(self, positions: torch.Tensor, q: torch.Tensor, k: torch.Tensor):
        """q [T, Hq*D], k [T, Hk*D]; rotated in place and returned."""
        ops.rope_qk_(q, k, positions, self.cos_sin_cache, self.head_dim, self.rot_dim, self.is_neox,
                     self.mrope_section, self.mrope_interleaved)
        return q, k


class XDRotaryEmbedding(RotaryEmbedding):
    """Rotary embedding whose frequency bands take their position from one of several axes
    (``xdrope_section``: how many frequency indices each axis owns, e.g. four axes for
    sequence / time / height / width).  ``positions`` is [axes, T]; a 1-D tensor means that all
    axes carry the same index, which is the plain rotation.  The table is the fixed-alpha NTK one
    the factory builds (reference: XDRotaryEmbedding selected by
    omni_npu/v1/layers/rotary_embedding/__init__.py:168-187)."""

    def __init__(self, *args, xdrope_section: Tuple[int, ...], **kw) -> None:
        super().__init__(*args, **kw)
        half = self.rot_dim // 2
        if sum(xdrope_section) != half:
            raise ValueError(f"xdrope_section {xdrope_section} must sum to rot_dim / 2 = {half}")
        self.xdrope_section = tuple(int(x) for x in xdrope_section)
        axis = torch.cat([torch.full((n,), a, dtype=torch.long) for a, n in enumerate(self.xdrope_section)])
        self.register_buffer("axis_of_freq", axis, persistent=False)

    def forward(self, positions: torch.Tensor, q: torch.Tensor, k: torch.Tensor):
        if positions.dim() == 1:
            return super().forward(positions, q, k)
        if positions.shape[0] != len(self.xdrope_section):
            raise ValueError(f"positions carry {positions.shape[0]} axes, the sections name {len(self.xdrope_section)}")
        half = self.rot_dim // 2
        # per token and frequency index: the position of the axis that owns the index
        pos = positions.long()[self.axis_of_freq.to(positions.device)].t()           # [T, half]
        idx = torch.arange(half, device=pos.device)
        cos = self.cos_sin_cache[pos, idx].float()                                   # [T, half]
        sin = self.cos_sin_cache[pos, half + idx].float()
        for x in (q, k):
            v = x.view(x.shape[0], -1, self.head_dim)
            rot = v[..., : self.rot_dim].float()
            c, s_ = cos[:, None, :], sin[:, None, :]
            if self.is_neox:
                x0, x1 = rot[..., :half], rot[..., half:]
                out = torch.cat((x0 * c - x1 * s_, x1 * c + x0 * s_), dim=-1)
            else:
                x0, x1 = rot[..., 0::2], rot[..., 1::2]
                out = torch.stack((x0 * c - x1 * s_, x1 * c + x0 * s_), dim=-1).flatten(-2)
            v[..., : self.rot_dim] = out.to(x.dtype)
        return q, k


class DualChunkRotaryEmbedding(nn.Module):
    """Rotations for dual-chunk attention (long contexts cut into chunks of ``chunk_size`` with a
    local window of ``local_size``): keys are rotated by their position inside a chunk, and the
    query is produced five times, for attention inside its chunk, to the chunk before it, to
    earlier chunks, and the two "critical" variants used when chunks are selected.  All five are
    the plain rotation at a remapped position, so one table serves them (reference: the
    dual_chunk_attention_config branch of omni_npu/v1/layers/rotary_embedding/__init__.py:69-86).

    ``forward`` returns ``(queries, key)`` with ``queries`` = the five variants concatenated along
    the last dimension in the order (intra, successor, inter, successor-critical, inter-critical)."""

    def __init__(self, head_dim: int, rot_dim: int, max_position: int, base: float, is_neox: bool,
                 chunk_size: int, local_size: int, device=None) -> None:
        super().__init__()
        self.chunk_size, self.local_size = int(chunk_size), int(local_size)
        self.chunk_len = self.chunk_size - self.local_size
        if self.chunk_len <= 0:
            raise ValueError("chunk_size must exceed local_size")
        self.max_position = max_position
        # largest remapped position: chunk_len - 1 + chunk_size (inter-critical)
        self.rope = RotaryEmbedding(head_dim, rot_dim, self.chunk_size + self.chunk_len + 1, base, is_neox,
                                    device=device)

    def remap(self, positions: torch.Tensor):
        """The six position tensors: key, then the five query variants."""
        r = positions % self.chunk_len
        succ = torch.clamp(r + self.chunk_len, max=self.chunk_size)
        inter = torch.full_like(r, min(2 * self.chunk_len - 1, self.chunk_size))
        return r, r, succ, inter, r + self.chunk_len, r + self.chunk_size

    def forward(self, positions: torch.Tensor, q: torch.Tensor, k: torch.Tensor,
                offsets: Optional[torch.Tensor] = None):
        if offsets is not None:
            positions = positions + offsets
        maps = self.remap(positions.to(torch.int32))
        outs = []
        none = q.new_zeros((q.shape[0], 0))
        for i, pos in enumerate(maps[1:]):
            qi = q.clone()
            # the key is rotated together with the first query variant (same remapped position)
            self.rope(pos.contiguous(), qi, k if i == 0 else none)
            outs.append(qi)
        return torch.cat(outs, dim=-1), k


def _linear_inv_freq(rot_dim: int, base: float, factor: float) -> torch.Tensor:
    return _base_inv_freq(rot_dim, base) / factor


def _ntk_inv_freq(rot_dim: int, base: float, factor: float, max_pos: int, orig_max: int) -> torch.Tensor:
    new_base = base * ((factor * max_pos / orig_max) - (factor - 1)) ** (rot_dim / (rot_dim - 2))
    return _base_inv_freq(rot_dim, new_base)


def _llama3_inv_freq(rot_dim: int, base: float, factor: float, low: float, high: float,
                     orig_max: int) -> torch.Tensor:
    inv = _base_inv_freq(rot_dim, base)
    low_wl, high_wl = orig_max / low, orig_max / high
    wl = 2 * math.pi / inv
    smooth = (orig_max / wl - low) / (high - low) if high != low else torch.zeros_like(inv)
    new = torch.where(wl < high_wl, inv,
                      torch.where(wl > low_wl, inv / factor, (1 - smooth) * inv / factor + smooth * inv))
    return new


def _yarn_inv_freq(rot_dim: int, base: float, factor: float, orig_max: int, beta_fast: float,
                   beta_slow: float, extrapolation_factor: float = 1.0) -> torch.Tensor:
    pos_freqs = base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim)
    extra, inter = 1.0 / pos_freqs, 1.0 / (factor * pos_freqs)
    low, high = yarn_find_correction_range(beta_fast, beta_slow, rot_dim, base, orig_max)
    mask = (1 - yarn_linear_ramp_mask(low, high, rot_dim // 2)) * extrapolation_factor
    return inter * (1 - mask) + extra * mask


_ROPE_CACHE: Dict[Any, RotaryEmbedding] = {}


def get_rope(head_dim: int, rot_dim: int, max_position: int, base: float, is_neox: bool = True,
             rope_scaling: Optional[Dict[str, Any]] = None, device=None,
             dual_chunk_attention_config: Optional[Dict[str, Any]] = None) -> nn.Module:
    dca = {k: v for k, v in (dual_chunk_attention_config or {}).items() if k in ("chunk_size", "local_size")}
    key = (head_dim, rot_dim, max_position, base, is_neox,
           tuple(sorted((k, str(v)) for k, v in (rope_scaling or {}).items())), str(device),
           tuple(sorted(dca.items())))
    hit = _ROPE_CACHE.get(key)
    if hit is not None:
        return hit
    if dual_chunk_attention_config is not None:
        rope = DualChunkRotaryEmbedding(head_dim, rot_dim, max_position, base, is_neox,
                                        dca.get("chunk_size", 8192), dca.get("local_size", 1024), device)
        _ROPE_CACHE[key] = rope
        return rope
    rs = dict(rope_scaling or {})
    kind = rs.get("rope_type", rs.get("type", "default"))
    mrope = rs.get("mrope_section")
    inv, mscale, max_pos = None, 1.0, max_position
    if kind in ("default", "mrope", "mllama4") or kind is None:
        # mllama4 rotates interleaved pairs with the plain frequencies: the caller passes is_neox=False
        pass
    elif kind == "linear":
        inv = _linear_inv_freq(rot_dim, base, rs["factor"])
        max_pos = int(max_position * rs["factor"])
    elif kind in ("dynamic", "xdrope") and "alpha" in rs:
        # fixed-alpha NTK: base * alpha^(d / (d - 2)); xdrope adds per-axis sections, which coincide
        # for text-only positions (all axes carry the same index), so one table serves it
        inv = _base_inv_freq(rot_dim, base * float(rs["alpha"]) ** (rot_dim / (rot_dim - 2)))
    elif kind in ("dynamic", "ntk"):
        if "factor" not in rs:
            raise ValueError("dynamic rope scaling needs either 'alpha' or 'factor'")
        orig = rs.get("original_max_position_embeddings", max_position)
        max_pos = int(orig * rs["factor"]) if kind == "dynamic" else max_position
        inv = _ntk_inv_freq(rot_dim, base, rs["factor"], max_pos, orig)
    elif kind == "llama3":
        inv = _llama3_inv_freq(rot_dim, base, rs["factor"], rs.get("low_freq_factor", 1.0),
                               rs.get("high_freq_factor", 4.0),
                               rs.get("original_max_position_embeddings", 8192))
    elif kind == "yarn":
        orig = rs.get("original_max_position_embeddings", max_position)
        inv = _yarn_inv_freq(rot_dim, base, rs["factor"], orig, rs.get("beta_fast", 32),
                             rs.get("beta_slow", 1))
        mscale = yarn_get_mscale(rs["factor"]) * rs.get("attn_factor", 1.0)
        max_pos = int(orig * rs["factor"])
    elif kind in ("deepseek_yarn", "deepseek_llama_scaling"):
        orig = rs.get("original_max_position_embeddings", max_position)
        inv = _yarn_inv_freq(rot_dim, base, rs["factor"], orig, rs.get("beta_fast", 32),
                             rs.get("beta_slow", 1))
        mscale = (yarn_get_mscale(rs["factor"], rs.get("mscale", 1.0))
                  / yarn_get_mscale(rs["factor"], rs.get("mscale_all_dim", 0.0))
                  * rs.get("attn_factor", 1.0))
        max_pos = int(orig * rs["factor"])
    elif kind in ("longrope", "su"):
        orig = rs.get("original_max_position_embeddings", max_position)
        factors = torch.tensor(rs["long_factor"] if max_position > orig else rs["short_factor"],
                               dtype=torch.float32)
        inv = _base_inv_freq(rot_dim, base) / factors
        scale = max_position / orig
        mscale = 1.0 if scale <= 1.0 else math.sqrt(1 + math.log(scale) / math.log(orig))
    else:
        raise ValueError(f"unknown rope scaling type {kind!r}")
    max_pos = min(max_pos, 1 << 20)
    xd = rs.get("xdrope_section")
    if xd:
        rope = XDRotaryEmbedding(head_dim, rot_dim, max_pos, base, is_neox, inv, mscale, None, False, device,
                                 xdrope_section=tuple(xd))
    else:
        rope = RotaryEmbedding(head_dim, rot_dim, max_pos, base, is_neox, inv, mscale,
                               tuple(mrope) if mrope else None,
                               bool(rs.get("mrope_interleaved", False)), device)
    _ROPE_CACHE[key] = rope
    return rope
