"""Qwen3-VL: vision transformer + Qwen3 decoder with M-RoPE and DeepStack.

Vision side.  Images / video frames arrive as flattened patches ``[L, C*T*P*P]`` with a
grid ``(t, h, w)`` per item, ordered in 2x2 *merge blocks* (the HF processor's order).
``patch_embed`` (a strided Conv3d, evaluated as one GEMM) lifts them to the ViT width;
learned position embeddings are bilinearly interpolated from a square table to the
item's grid; every block is pre-LayerNorm attention (2-D rotary over (row, col), full
attention inside one frame) + GELU MLP.  ``merger`` concatenates each 2x2 block and
projects it to the text width.  At the layers listed in ``deepstack_visual_indexes`` a
second kind of merger taps the hidden states; those *DeepStack* features are added to
the text hidden states of the visual tokens after the first decoder layers.

Text side.  Qwen3 (per-head q/k RMSNorm) with 3-axis rotary positions (temporal, height,
width; interleaved sections).  Text-only requests use ordinary positions, for which the
three axes coincide, and run through the engine like any Qwen3 model.

Counterpart of omni_npu/v1/models/qwen/qwen3_vl.py:129-1688 (vision tower :129-608, LLM with
DeepStack :1084-1183, wrapper and M-RoPE positions :1185-1688) and of the embedding merge in
omni_npu/v1/models/qwen/utils.py:48-97.  Image decoding / resizing is the HF processor's job.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..attention.metadata import get_forward_context
from ..config import EngineConfig, ModelConfig
from ..layers.embedding import ParallelLMHead
from ..layers.norm import reduce_add_rms_norm
from ..parallel import state as pstate
from .llama import LlamaAttention, LlamaDecoderLayer, LlamaModel
from .utils import load_stacked_weights


@dataclass
class VisionConfig:
    depth: int = 27
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 4096
    num_position_embeddings: int = 2304
    deepstack_visual_indexes: List[int] = field(default_factory=lambda: [8, 16, 24])
    hidden_act: str = "gelu_pytorch_tanh"

    @classmethod
    def from_dict(cls, d: Dict) -> "VisionConfig":
        names = cls.__dataclass_fields__
        return cls(**{k: v for k, v in d.items() if k in names})


def _linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16:
        return ops.gemm(x, w, b)
    return F.linear(x, w, b)


class VisionBlock(nn.Module):
    def __init__(self, c: VisionConfig, dtype, device) -> None:
        super().__init__()
        h = c.hidden_size
        kw = dict(dtype=dtype, device=device)
        self.norm1 = nn.LayerNorm(h, eps=1e-6, **kw)
        self.norm2 = nn.LayerNorm(h, eps=1e-6, **kw)
        self.attn_qkv = nn.Linear(h, 3 * h, bias=True, **kw)
        self.attn_proj = nn.Linear(h, h, bias=True, **kw)
        self.linear_fc1 = nn.Linear(h, c.intermediate_size, bias=True, **kw)
        self.linear_fc2 = nn.Linear(c.intermediate_size, h, bias=True, **kw)
        self.num_heads = c.num_heads
        self.tanh_gelu = c.hidden_act == "gelu_pytorch_tanh"

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, frames: Sequence[int]) -> torch.Tensor:
        l, h = x.shape
        d = h // self.num_heads
        qkv = _linear(self.norm1(x), self.attn_qkv.weight, self.attn_qkv.bias).view(l, 3, self.num_heads, d)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
        q, k = _rotate(q, cos, sin), _rotate(k, cos, sin)
        out = torch.empty_like(q)
        s = 0
        for n in frames:                         # full attention inside one frame
            qs, ks, vs = (t[s:s + n].transpose(0, 1).unsqueeze(0) for t in (q, k, v))
            out[s:s + n] = F.scaled_dot_product_attention(qs, ks, vs).squeeze(0).transpose(0, 1)
            s += n
        x = x + _linear(out.reshape(l, h), self.attn_proj.weight, self.attn_proj.bias)
        y = _linear(self.norm2(x), self.linear_fc1.weight, self.linear_fc1.bias)
        y = F.gelu(y, approximate="tanh" if self.tanh_gelu else "none")
        return x + _linear(y, self.linear_fc2.weight, self.linear_fc2.bias)


def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [L, H, D]; cos/sin [L, D] (neox halves)."""
    xf = x.float()
    d = x.shape[-1] // 2
    rot = torch.cat([-xf[..., d:], xf[..., :d]], dim=-1)
    return (xf * cos.unsqueeze(1) + rot * sin.unsqueeze(1)).to(x.dtype)


class PatchMerger(nn.Module):
    def __init__(self, c: VisionConfig, dtype, device, postshuffle_norm: bool) -> None:
        super().__init__()
        self.merged = c.hidden_size * c.spatial_merge_size ** 2
        self.postshuffle = postshuffle_norm
        kw = dict(dtype=dtype, device=device)
        self.norm = nn.LayerNorm(self.merged if postshuffle_norm else c.hidden_size, eps=1e-6, **kw)
        self.linear_fc1 = nn.Linear(self.merged, self.merged, bias=True, **kw)
        self.linear_fc2 = nn.Linear(self.merged, c.out_hidden_size, bias=True, **kw)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.norm(x.view(-1, self.merged)) if self.postshuffle else self.norm(x).view(-1, self.merged)
        y = F.gelu(_linear(x, self.linear_fc1.weight, self.linear_fc1.bias))
        return _linear(y, self.linear_fc2.weight, self.linear_fc2.bias)


class VisionTransformer(nn.Module):
    def __init__(self, c: VisionConfig, dtype, device) -> None:
        super().__init__()
        self.cfg = c
        kw = dict(dtype=dtype, device=device)
        patch_elems = c.in_channels * c.temporal_patch_size * c.patch_size ** 2
        self.patch_embed = nn.Linear(patch_elems, c.hidden_size, bias=True, **kw)      # the Conv3d as a GEMM
        self.pos_embed = nn.Embedding(c.num_position_embeddings, c.hidden_size, **kw)
        self.grid_side = int(round(math.sqrt(c.num_position_embeddings)))
        self.blocks = nn.ModuleList([VisionBlock(c, dtype, device) for _ in range(c.depth)])
        self.merger = PatchMerger(c, dtype, device, postshuffle_norm=False)
        self.deepstack_merger_list = nn.ModuleList([PatchMerger(c, dtype, device, True)
                                                    for _ in c.deepstack_visual_indexes])
        head_dim = c.hidden_size // c.num_heads
        self.rot_dim = head_dim // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, self.rot_dim, 2, dtype=torch.float32) / self.rot_dim))
        self.register_buffer("inv_freq", inv.to(device) if device is not None else inv, persistent=False)

    # ---------------------------------------------------------------- geometry
    def _merge_order(self, h: int, w: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        """Row / column of every patch of an h x w grid in merge-block order."""
        m = self.cfg.spatial_merge_size
        rows = torch.arange(h, device=device).view(h // m, m, 1, 1).expand(h // m, m, w // m, m)
        cols = torch.arange(w, device=device).view(1, 1, w // m, m).expand(h // m, m, w // m, m)
        rows = rows.permute(0, 2, 1, 3).reshape(-1)
        cols = cols.permute(0, 2, 1, 3).reshape(-1)
        return rows, cols

    def rotary_cos_sin(self, grid_thw: Sequence[Sequence[int]], device) -> Tuple[torch.Tensor, torch.Tensor]:
        parts = []
        for t, h, w in grid_thw:
            rows, cols = self._merge_order(h, w, device)
            fr = torch.outer(rows.float(), self.inv_freq.to(device))
            fc = torch.outer(cols.float(), self.inv_freq.to(device))
            parts.append(torch.cat([fr, fc], dim=-1).repeat(t, 1))          # [t*h*w, rot_dim]
        freqs = torch.cat(parts, dim=0)
        emb = torch.cat([freqs, freqs], dim=-1)
        return emb.cos(), emb.sin()

    def interpolated_pos_embed(self, grid_thw: Sequence[Sequence[int]], device) -> torch.Tensor:
        """Bilinear interpolation of the square table of learned embeddings to each item's
        grid, emitted in merge-block order."""
        side = self.grid_side
        table = self.pos_embed.weight
        outs = []
        for t, h, w in grid_thw:
            ys = torch.linspace(0, side - 1, h, device=device)
            xs = torch.linspace(0, side - 1, w, device=device)
            y0, x0 = ys.floor().long(), xs.floor().long()
            y1, x1 = (y0 + 1).clamp(max=side - 1), (x0 + 1).clamp(max=side - 1)
            fy, fx = (ys - y0.float()).unsqueeze(1), (xs - x0.float()).unsqueeze(0)

            def at(yy, xx):
                return table[(yy.unsqueeze(1) * side + xx.unsqueeze(0)).reshape(-1)].float().view(h, w, -1)

            emb = (at(y0, x0) * ((1 - fy) * (1 - fx)).unsqueeze(-1) + at(y0, x1) * ((1 - fy) * fx).unsqueeze(-1)
                   + at(y1, x0) * (fy * (1 - fx)).unsqueeze(-1) + at(y1, x1) * (fy * fx).unsqueeze(-1))
            rows, cols = self._merge_order(h, w, device)
            outs.append(emb[rows, cols].repeat(t, 1))
        return torch.cat(outs, dim=0).to(table.dtype)

    # ----------------------------------------------------------------- forward
    def forward(self, pixel_values: torch.Tensor, grid_thw: Sequence[Sequence[int]]):
        """pixel_values [L, C*T*P*P].  Returns (embeds [L/4, out], [deepstack embeds ...])."""
        device = pixel_values.device
        x = _linear(pixel_values.to(self.patch_embed.weight.dtype), self.patch_embed.weight, self.patch_embed.bias)
        x = x + self.interpolated_pos_embed(grid_thw, device)
        cos, sin = self.rotary_cos_sin(grid_thw, device)
        frames = [h * w for t, h, w in grid_thw for _ in range(t)]
        deep = []
        for i, blk in enumerate(self.blocks):
            x = blk(x, cos, sin, frames)
            if i in self.cfg.deepstack_visual_indexes:
                deep.append(self.deepstack_merger_list[self.cfg.deepstack_visual_indexes.index(i)](x))
        return self.merger(x), deep


# --------------------------------------------------------------------- text
class Qwen3VLAttention(LlamaAttention):
    """Rotary positions may have three axes ([3, T]); the fused rope + cache-write kernel
    handles the ordinary 1-axis case, the 3-axis case goes through the M-RoPE op."""

    def forward(self, hidden: torch.Tensor, reduce: bool = True) -> torch.Tensor:
        md = get_forward_context().attn_metadata
        if md.positions.dim() == 1:
            return super().forward(hidden, reduce)
        q, k, v = self.qkv_proj(hidden)
        t = q.shape[0]
        if self.qk_norm:
            q = self.q_norm(q.reshape(-1, self.head_dim)).view(t, -1)
            k = self.k_norm(k.reshape(-1, self.head_dim)).view(t, -1)
        q, k = self.rotary(md.positions, q.contiguous(), k.contiguous())
        o = self.attn(q, k, v, None, apply_rope=False)
        return self.o_proj(o, reduce=reduce)


class Qwen3VLDecoderLayer(LlamaDecoderLayer):
    def __init__(self, cfg: ModelConfig, layer_idx: int, device, prefix: str) -> None:
        super().__init__(cfg, layer_idx, device, prefix)
        self.self_attn = Qwen3VLAttention(cfg, layer_idx, device, f"{prefix}.self_attn")


class Qwen3VLTextModel(LlamaModel):
    def __init__(self, cfg: ModelConfig, device, prefix: str = "model") -> None:
        super().__init__(cfg, device, prefix)
        self.layers = nn.ModuleList([Qwen3VLDecoderLayer(cfg, i, device, f"{prefix}.layers.{i}")
                                     for i in range(cfg.num_layers)])

    def forward(self, input_ids, positions, inputs_embeds=None, deepstack: Optional[List[torch.Tensor]] = None,
                visual_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        hidden = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
        tp = pstate.get_tp_group()
        residual = None
        for i, layer in enumerate(self.layers):
            hidden, residual = layer(hidden, residual)
            if deepstack is not None and i < len(deepstack):
                # DeepStack: the layer's output (hidden + residual, once reduced) of the visual
                # tokens receives the tapped vision features; adding them to the residual is
                # equivalent and keeps the un-reduced `hidden` untouched
                residual = residual.clone()
                residual[visual_mask] += deepstack[i].to(residual.dtype)
        hidden, _ = reduce_add_rms_norm(self.norm, hidden, residual, tp)
        return hidden


def merge_multimodal_embeddings(inputs_embeds: torch.Tensor, mm_embeds: torch.Tensor,
                                is_multimodal: torch.Tensor) -> torch.Tensor:
    """Overwrite the rows of ``inputs_embeds`` at placeholder positions with ``mm_embeds`` (in
    place).  The counts must agree."""
    n = int(is_multimodal.sum())
    if n != mm_embeds.shape[0]:
        raise ValueError(f"attempted to assign {mm_embeds.shape[0]} multimodal tokens to {n} placeholders")
    inputs_embeds[is_multimodal] = mm_embeds.to(inputs_embeds.dtype)
    return inputs_embeds


class Qwen3VLForConditionalGeneration(nn.Module):
    stacked_params_mapping = [
        (".qkv_proj", ".q_proj", "q"), (".qkv_proj", ".k_proj", "k"), (".qkv_proj", ".v_proj", "v"),
        (".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1),
    ]

    def __init__(self, engine_config: EngineConfig, device=None) -> None:
        super().__init__()
        cfg = engine_config.model
        self.config = cfg
        hf = cfg.hf_config or {}
        self.vision_config = VisionConfig.from_dict(hf.get("vision_config") or {})
        if "vision_config" not in hf:
            self.vision_config.out_hidden_size = cfg.hidden_size
        self.image_token_id = hf.get("image_token_id", 151655)
        self.video_token_id = hf.get("video_token_id", 151656)
        self.vision_start_token_id = hf.get("vision_start_token_id", 151652)
        self.visual = VisionTransformer(self.vision_config, cfg.dtype, device)
        self.model = Qwen3VLTextModel(cfg, device)
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype, device) \
            if not cfg.tie_word_embeddings else self.model.embed_tokens
        if cfg.tie_word_embeddings:
            self.lm_head.__class__ = ParallelLMHead
        self._pending_deepstack: Optional[List[torch.Tensor]] = None
        self._pending_mask: Optional[torch.Tensor] = None

    # ------------------------------------------------------------- multimodal
    def embed_multimodal(self, pixel_values: torch.Tensor, grid_thw: Sequence[Sequence[int]]):
        """(image embeds [N, H], DeepStack embeds) for the items described by ``grid_thw``."""
        return self.visual(pixel_values, grid_thw)

    def embed_input_ids(self, input_ids: torch.Tensor, mm_embeds: Optional[torch.Tensor] = None,
                        deepstack: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        embeds = self.model.embed_tokens(input_ids)
        if mm_embeds is None:
            self._pending_deepstack = self._pending_mask = None
            return embeds
        mask = (input_ids == self.image_token_id) | (input_ids == self.video_token_id)
        embeds = merge_multimodal_embeddings(embeds, mm_embeds, mask)
        self._pending_deepstack, self._pending_mask = deepstack, mask
        return embeds

    def get_mrope_input_positions(self, input_tokens: Sequence[int], image_grid_thw: Sequence[Sequence[int]],
                                  second_per_grid: float = 1.0) -> Tuple[torch.Tensor, int]:
        """3-axis positions for a prompt with image placeholders.  Text tokens advance all
        axes together; the tokens of an image share the temporal index and enumerate
        (row, col) of the merged grid; text after an image continues from the largest index
        used so far + 1.  Returns ([3, T] int64, delta) where delta = next position - T."""
        m = self.vision_config.spatial_merge_size
        toks = list(input_tokens)
        pos: List[torch.Tensor] = []
        i, nxt, img = 0, 0, 0
        while i < len(toks):
            if toks[i] in (self.image_token_id, self.video_token_id) and img < len(image_grid_thw):
                t, h, w = image_grid_thw[img]
                gh, gw = h // m, w // m
                n = t * gh * gw
                tt = torch.arange(t).view(t, 1, 1).expand(t, gh, gw).reshape(-1)
                hh = torch.arange(gh).view(1, gh, 1).expand(t, gh, gw).reshape(-1)
                ww = torch.arange(gw).view(1, 1, gw).expand(t, gh, gw).reshape(-1)
                pos.append(torch.stack([tt, hh, ww]) + nxt)
                nxt += max(t, gh, gw)
                i += n
                img += 1
            else:
                j = i
                while j < len(toks) and not (toks[j] in (self.image_token_id, self.video_token_id)
                                              and img < len(image_grid_thw)):
                    j += 1
                pos.append((torch.arange(j - i) + nxt).unsqueeze(0).expand(3, -1))
                nxt += j - i
                i = j
        out = torch.cat(pos, dim=1) if pos else torch.zeros(3, 0, dtype=torch.long)
        return out, nxt - len(toks)

    # ----------------------------------------------------------------- forward
    def forward(self, input_ids, positions, inputs_embeds=None):
        deep, mask = self._pending_deepstack, self._pending_mask
        self._pending_deepstack = self._pending_mask = None
        return self.model(input_ids, positions, inputs_embeds, deep, mask)

    def compute_logits(self, hidden):
        return self.lm_head.compute_logits(hidden)

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        def rename(name: str) -> Optional[str]:
            name = name.replace("model.language_model.", "model.").replace("model.visual.", "visual.")
            if name.startswith("visual."):
                name = name.replace(".attn.qkv.", ".attn_qkv.").replace(".attn.proj.", ".attn_proj.")
                name = name.replace(".mlp.linear_fc", ".linear_fc")
                if name.startswith("visual.patch_embed.proj."):
                    name = name.replace("visual.patch_embed.proj.", "visual.patch_embed.")
            return name

        def reshape(items):
            for name, t in items:
                if name.endswith("patch_embed.proj.weight") and t.dim() == 5:
                    t = t.reshape(t.shape[0], -1)          # Conv3d kernel -> GEMM weight
                yield name, t

        skip = ("rotary_emb.inv_freq",) + (("lm_head.weight",) if self.config.tie_word_embeddings else ())
        return load_stacked_weights(self, reshape(weights), self.stacked_params_mapping, skip_substrings=skip,
                                    rename=rename)
