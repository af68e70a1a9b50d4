"""OpenPangu-VL: a windowed vision transformer in front of a Pangu language model.

Vision tower (Qwen2.5-VL style, with Pangu's changes):

* patches ``[in_channels * temporal_patch * patch^2]`` -> linear patch embedding (the Conv3d as a GEMM);
* 2-D rotary position embedding over (row, col) of the patch grid, patches ordered so that the
  ``spatial_merge_size^2`` patches of one merged token are adjacent;
* blocks = RMSNorm, attention, RMSNorm, MLP (SiLU-gated, or GELU).  Most blocks attend inside
  ``window_size`` pixel windows (the merged tokens are permuted so a window is contiguous), the
  blocks listed in ``fullatt_block_indexes`` attend over the whole frame;
* the outputs of several late blocks (``mm_unit_vision_select_layer``, default last and third
  from last) each go through the final RMSNorm and their own patch merger; the merged features
  are summed and the window permutation is undone.

The language model is the sink-attention Pangu decoder of ``models/pangu.py`` (separate K / V
head sizes, learned sink tokens, sliding windows, optional MoE), addressed with 3-axis M-RoPE
positions when the prompt contains images.

Counterpart of the reference's OpenPangu-VL model patch
(omni_npu/vllm_patches/patches/models/pangu72b-vl/patch_openpangu_vl.py:357-1005: vision
attention / MLP / block / rotary / patch merger / transformer with ``get_window_index`` and the
multi-layer mergers, and the model class that joins it to the Pangu decoder).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ..config import EngineConfig
from .pangu import PanguProMoEV2ForCausalLM
from .qwen3_vl import _linear, _rotate, merge_multimodal_embeddings


@dataclass
class OpenPanguVisionConfig:
    depth: int = 32
    hidden_size: int = 1280
    intermediate_size: int = 3420
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 4096
    window_size: int = 112
    fullatt_block_indexes: List[int] = field(default_factory=lambda: [7, 15, 23, 31])
    hidden_act: str = "silu"
    mm_unit_vision_select_layer: List[int] = field(default_factory=lambda: [-1, -3])
    rms_norm_eps: float = 1e-6

    @classmethod
    def from_dict(cls, d: Dict) -> "OpenPanguVisionConfig":
        names = cls.__dataclass_fields__
        return cls(**{k: v for k, v in d.items() if k in names})


class _RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, dtype, device) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device), requires_grad=False)
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(x.dtype)


class OpenPanguVisionBlock(nn.Module):
    def __init__(self, c: OpenPanguVisionConfig, dtype, device) -> None:
        super().__init__()
        h = c.hidden_size
        kw = dict(dtype=dtype, device=device)
        self.norm1 = _RMSNorm(h, c.rms_norm_eps, dtype, device)
        self.norm2 = _RMSNorm(h, c.rms_norm_eps, dtype, device)
        self.attn_qkv = nn.Linear(h, 3 * h, bias=True, **kw)
        self.attn_proj = nn.Linear(h, h, bias=True, **kw)
        self.gated = c.hidden_act == "silu"
        if self.gated:
            self.gate_up_proj = nn.Linear(h, 2 * c.intermediate_size, bias=True, **kw)
            self.down_proj = nn.Linear(c.intermediate_size, h, bias=True, **kw)
        else:
            self.fc1 = nn.Linear(h, c.intermediate_size, bias=True, **kw)
            self.fc2 = nn.Linear(c.intermediate_size, h, bias=True, **kw)
        self.num_heads = c.num_heads

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, segments: Sequence[int]) -> torch.Tensor:
        """``segments``: lengths of the runs of tokens that attend to one another (windows, or frames)."""
        l, h = x.shape
        d = h // self.num_heads
        qkv = _linear(self.norm1(x), self.attn_qkv.weight, self.attn_qkv.bias).view(l, 3, self.num_heads, d)
        q, k, v = _rotate(qkv[:, 0], cos, sin), _rotate(qkv[:, 1], cos, sin), qkv[:, 2]
        out = torch.empty_like(q)
        s = 0
        for n in segments:
            qs, ks, vs = (t[s:s + n].transpose(0, 1).unsqueeze(0) for t in (q, k, v))
            out[s:s + n] = F.scaled_dot_product_attention(qs, ks, vs).squeeze(0).transpose(0, 1)
            s += n
        x = x + _linear(out.reshape(l, h), self.attn_proj.weight, self.attn_proj.bias)
        y = self.norm2(x)
        if self.gated:
            gu = _linear(y, self.gate_up_proj.weight, self.gate_up_proj.bias)
            i = gu.shape[-1] // 2
            y = _linear(F.silu(gu[:, :i]) * gu[:, i:], self.down_proj.weight, self.down_proj.bias)
        else:
            y = _linear(F.gelu(_linear(y, self.fc1.weight, self.fc1.bias)), self.fc2.weight, self.fc2.bias)
        return x + y


class OpenPanguPatchMerger(nn.Module):
    """RMSNorm per patch, then the ``merge^2`` adjacent patches of a token through a 2-layer MLP."""

    def __init__(self, c: OpenPanguVisionConfig, dtype, device) -> None:
        super().__init__()
        self.merged = c.hidden_size * c.spatial_merge_size ** 2
        kw = dict(dtype=dtype, device=device)
        self.ln_q = _RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, device)
        self.fc1 = nn.Linear(self.merged, self.merged, bias=True, **kw)
        self.fc2 = nn.Linear(self.merged, c.out_hidden_size, bias=True, **kw)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.ln_q(x).view(-1, self.merged)
        return _linear(F.gelu(_linear(y, self.fc1.weight, self.fc1.bias)), self.fc2.weight, self.fc2.bias)


def window_index(grid_thw: Sequence[Sequence[int]], window_size: int, patch_size: int, merge: int
                 ) -> Tuple[torch.Tensor, List[int]]:
    """Permutation of the merged tokens that makes every attention window contiguous, and the
    window lengths in merged tokens (empty windows dropped).  A window covers ``window_size``
    pixels, i.e. ``window_size / patch_size / merge`` merged tokens, per side; windows at the
    right / bottom edge are smaller."""
    side = window_size // merge // patch_size
    order: List[torch.Tensor] = []
    lengths: List[int] = []
    base = 0
    for t, h, w in grid_thw:
        gh, gw = h // merge, w // merge
        idx = torch.arange(t * gh * gw).view(t, gh, gw)
        for ti in range(t):
            for y0 in range(0, gh, side):
                for x0 in range(0, gw, side):
                    win = idx[ti, y0:y0 + side, x0:x0 + side].reshape(-1)
                    order.append(win + base)
                    lengths.append(win.numel())
        base += t * gh * gw
    return torch.cat(order) if order else torch.zeros(0, dtype=torch.long), lengths


class OpenPanguVisionTransformer(nn.Module):
    def __init__(self, c: OpenPanguVisionConfig, dtype, device) -> None:
        super().__init__()
        self.cfg = c
        kw = dict(dtype=dtype, device=device)
        patch_elems = c.in_channels * c.temporal_patch_size * c.patch_size ** 2
        self.patch_embed = nn.Linear(patch_elems, c.hidden_size, bias=False, **kw)
        self.blocks = nn.ModuleList([OpenPanguVisionBlock(c, dtype, device) for _ in range(c.depth)])
        self.final_layernorm = _RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, device)
        # selected layers, deepest first (the order the mergers are stored in)
        self.take = sorted({c.depth + i for i in c.mm_unit_vision_select_layer}, reverse=True)
        self.merger = nn.ModuleList([OpenPanguPatchMerger(c, dtype, device) for _ in self.take])

    def rotary_cos_sin(self, grid_thw: Sequence[Sequence[int]], device) -> Tuple[torch.Tensor, torch.Tensor]:
        """cos / sin [L, head_dim] in merge order: the first half of the rotary pairs turns with
        the row, the second half with the column."""
        c = self.cfg
        m = c.spatial_merge_size
        d = c.hidden_size // c.num_heads
        inv = 1.0 / (10000.0 ** (torch.arange(0, d // 2, 2, dtype=torch.float32, device=device) / (d // 2)))
        rows, cols = [], []
        for t, h, w in grid_thw:
            order = torch.arange(h * w, device=device).view(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            rows.append((order // w).repeat(t))
            cols.append((order % w).repeat(t))
        r, cl = torch.cat(rows).float(), torch.cat(cols).float()
        freqs = torch.cat([torch.outer(r, inv), torch.outer(cl, inv)], dim=-1)
        emb = torch.cat([freqs, freqs], dim=-1)
        return emb.cos(), emb.sin()

    def forward(self, pixel_values: torch.Tensor, grid_thw: Sequence[Sequence[int]]) -> torch.Tensor:
        """pixel_values [L, in_channels * temporal_patch * patch^2] with the patches of a merged token
        adjacent; returns [L / merge^2, out_hidden_size] in the same (un-windowed) order."""
        c = self.cfg
        unit = c.spatial_merge_size ** 2
        x = _linear(pixel_values.to(self.patch_embed.weight.dtype), self.patch_embed.weight, None)
        cos, sin = self.rotary_cos_sin(grid_thw, x.device)
        perm, win_lengths = window_index(grid_thw, c.window_size, c.patch_size, c.spatial_merge_size)
        perm = perm.to(x.device)
        l = x.shape[0]

        def windowed(t: torch.Tensor) -> torch.Tensor:
            return t.view(l // unit, unit, -1)[perm].reshape(l, -1)

        x, cos, sin = windowed(x), windowed(cos), windowed(sin)
        windows = [n * unit for n in win_lengths]
        frames = [h * w for t, h, w in grid_thw for _ in range(t)]     # a frame's windows are consecutive
        taken: Dict[int, torch.Tensor] = {}
        for i, blk in enumerate(self.blocks):
            x = blk(x, cos, sin, frames if i in c.fullatt_block_indexes else windows)
            if i in self.take:
                taken[i] = self.final_layernorm(x)
        out = sum(self.merger[j](taken[layer]) for j, layer in enumerate(self.take))
        inverse = torch.empty_like(perm)
        inverse[perm] = torch.arange(perm.numel(), device=perm.device)
        return out[inverse]


class OpenPanguVLForConditionalGeneration(nn.Module):
    """Vision tower + Pangu decoder.  Image / video placeholder tokens of the prompt are replaced
    by the tower's merged features before the first decoder layer."""

    def __init__(self, engine_config: EngineConfig, device=None) -> None:
        super().__init__()
        cfg = engine_config.model
        self.config = cfg
        hf = cfg.hf_config or {}
        self.vision_config = OpenPanguVisionConfig.from_dict(hf.get("vision_config") or {})
        if "vision_config" not in hf:
            self.vision_config.out_hidden_size = cfg.hidden_size
        self.image_token_id = hf.get("image_token_id", 151655)
        self.video_token_id = hf.get("video_token_id", 151656)
        self.visual = OpenPanguVisionTransformer(self.vision_config, cfg.dtype, device)
        self.language_model = PanguProMoEV2ForCausalLM(engine_config, device)

    # the KV-cache layout and the sink blocks are the language model's
    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            if name in ("get_kv_cache_spec", "allocate_kv_cache", "num_reserved_kv_blocks", "num_kv_layers"):
                return getattr(super().__getattr__("language_model"), name)
            raise

    def embed_multimodal(self, pixel_values: torch.Tensor, grid_thw: Sequence[Sequence[int]]) -> torch.Tensor:
        return self.visual(pixel_values, grid_thw)

    def embed_input_ids(self, input_ids: torch.Tensor, mm_embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
        embeds = self.language_model.model.embed_tokens(input_ids)
        if mm_embeds is None:
            return embeds
        mask = (input_ids == self.image_token_id) | (input_ids == self.video_token_id)
        return merge_multimodal_embeddings(embeds, mm_embeds, mask)

    def get_mrope_input_positions(self, input_tokens: Sequence[int], image_grid_thw: Sequence[Sequence[int]]
                                  ) -> Tuple[torch.Tensor, int]:
        """3-axis positions: text advances all axes together, the tokens of an image share the
        temporal index and enumerate (row, col) of the merged grid; text after an image goes on
        from the largest index used + 1.  Returns ([3, T] int64, next position - T)."""
        m = self.vision_config.spatial_merge_size
        toks = list(input_tokens)
        special = (self.image_token_id, self.video_token_id)
        pos: List[torch.Tensor] = []
        i = nxt = img = 0
        while i < len(toks):
            if toks[i] in special and img < len(image_grid_thw):
                t, h, w = image_grid_thw[img]
                gh, gw = h // m, w // m
                tt = torch.arange(t).view(t, 1, 1).expand(t, gh, gw).reshape(-1)
                hh = torch.arange(gh).view(1, gh, 1).expand(t, gh, gw).reshape(-1)
                ww = torch.arange(gw).view(1, 1, gw).expand(t, gh, gw).reshape(-1)
                pos.append(torch.stack([tt, hh, ww]) + nxt)
                nxt += max(t, gh, gw)
                i += t * gh * gw
                img += 1
            else:
                j = i
                while j < len(toks) and not (toks[j] in special and img < len(image_grid_thw)):
                    j += 1
                pos.append((torch.arange(j - i) + nxt).unsqueeze(0).expand(3, -1))
                nxt += j - i
                i = j
        out = torch.cat(pos, dim=1) if pos else torch.zeros(3, 0, dtype=torch.long)
        return out, nxt - len(toks)

    def forward(self, input_ids, positions, inputs_embeds=None):
        return self.language_model(input_ids, positions, inputs_embeds)

    def compute_logits(self, hidden):
        return self.language_model.compute_logits(hidden)

    # ---------------------------------------------------------------- weights
    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        """``visual.*`` tensors go to the tower (q / k / v and gate / up are stored fused; the patch
        Conv3d kernel is flattened), everything else to the language model."""
        vis: Dict[str, Dict[str, torch.Tensor]] = {}
        loaded = set()
        lang: List[Tuple[str, torch.Tensor]] = []
        params = dict(self.visual.named_parameters())
        for name, t in weights:
            if not name.startswith(("visual.", "model.visual.")):
                lang.append((name[len("language_model."):] if name.startswith("language_model.") else name, t))
                continue
            n = name.split("visual.", 1)[1]
            n = n.replace(".attn.qkv.", ".attn_qkv.").replace(".attn.proj.", ".attn_proj.")
            if n.startswith("merger."):
                n = n.replace(".mlp.0.", ".fc1.").replace(".mlp.2.", ".fc2.")
            n = n.replace(".mlp.", ".").replace("patch_embed.proj.", "patch_embed.")
            parts = None
            for fused, names in ((".attn_qkv.", (".attn.q.", ".attn.k.", ".attn.v.")),
                                 (".gate_up_proj.", (".gate_proj.", ".up_proj."))):
                for k, piece in enumerate(names):
                    if piece in n:
                        parts = (n.replace(piece, fused), k, len(names))
            if parts is not None:
                tgt, k, cnt = parts
                slot = vis.setdefault(tgt, {})
                slot[k] = t
                if len(slot) == cnt:
                    params[tgt].data.copy_(torch.cat([slot[j] for j in range(cnt)], dim=0).to(params[tgt].dtype))
                    loaded.add("visual." + tgt)
                continue
            if n == "patch_embed.weight" and t.dim() > 2:
                t = t.reshape(t.shape[0], -1)
            if n in params:
                params[n].data.copy_(t.to(params[n].dtype))
                loaded.add("visual." + n)
        loaded |= {"language_model." + k for k in self.language_model.load_weights(lang)}
        return loaded
