"""Multi-token-prediction (MTP) head: the draft model of self-speculative decoding.

An MTP layer predicts the token after next.  For the token at position p it takes the
embedding of token p+1 and the target model's final hidden state at p,

    h = eh_proj( concat( enorm(embed(x[p+1])), hnorm(hidden[p]) ) )
    h = decoder_block(h)                    # one ordinary decoder layer with its own KV cache
    logits = head( norm(h) )                # -> a draft for x[p+2]

so one extra layer pass per step yields one draft token per request.  The block reuses
the target model's decoder-layer class (MLA + MoE for DeepSeek, GQA + MLP for
Llama-style models), the embedding and, unless the checkpoint brings its own, the LM head.

Counterpart of ``DeepSeekMultiTokenPredictorLayer`` / ``DeepSeekMTP``
(omni_npu/v1/models/deepseek/deepseek_mtp.py:63-104,106-200) including the checkpoint
name mapping of its ``_rewrite_spec_layer_name`` (:400-430): weights of
``model.layers.<num_hidden_layers + i>.*`` belong to MTP layer i; ``embed_tokens`` and
``shared_head.head`` may be omitted (shared with the target model).
"""
from __future__ import annotations

import re
from typing import Callable, Iterable, List, Optional, Tuple

import torch
from torch import nn

from ..config import EngineConfig
from ..layers.linear import ReplicatedLinear
from ..layers.norm import RMSNorm
from ..parallel import state as pstate

_LAYER_RE = re.compile(r"^model\.layers\.(\d+)\.(.*)$")
# sub-modules of an MTP layer that are not part of its decoder block
_MTP_OWN = ("enorm", "hnorm", "eh_proj", "shared_head", "embed_tokens")


class MultiTokenPredictorLayer(nn.Module):
    def __init__(self, engine: EngineConfig, layer_idx: int, device, block_factory: Callable[[int, str], nn.Module],
                 prefix: str) -> None:
        super().__init__()
        cfg = engine.model
        self.layer_idx = layer_idx
        self.enorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)
        self.hnorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)
        self.eh_proj = ReplicatedLinear(2 * cfg.hidden_size, cfg.hidden_size, dtype=cfg.dtype, device=device,
                                        prefix=f"{prefix}.eh_proj")
        self.mtp_block = block_factory(layer_idx, prefix)
        self.shared_head_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.dtype, device)
        self.tp_group = pstate.get_tp_group()

    def forward(self, inputs_embeds: torch.Tensor, previous_hidden: torch.Tensor) -> torch.Tensor:
        h = self.eh_proj(torch.cat([self.enorm(inputs_embeds), self.hnorm(previous_hidden)], dim=-1))
        out = self.mtp_block(h, None) if not getattr(self.mtp_block, "takes_pending", False) else \
            self.mtp_block(h, None, False)
        hidden, residual = out[0], out[1]
        pending = out[2] if len(out) > 2 else True
        # the block leaves its MLP output un-reduced (and un-added): finish it here
        if pending and self.tp_group.world_size > 1:
            hidden = self.tp_group.all_reduce(hidden)
        return self.shared_head_norm(hidden + residual)


class MultiTokenPredictor(nn.Module):
    """``num_nextn_predict_layers`` MTP layers on top of a target model."""

    def __init__(self, engine: EngineConfig, device, block_factory: Callable[[int, str], nn.Module],
                 num_layers: Optional[int] = None) -> None:
        super().__init__()
        cfg = engine.model
        self.first_layer = cfg.num_layers
        n = num_layers if num_layers is not None else max(1, cfg.num_nextn_predict_layers)
        self.layers = nn.ModuleList([
            MultiTokenPredictorLayer(engine, cfg.num_layers + i, device, block_factory,
                                     f"model.layers.{cfg.num_layers + i}") for i in range(n)])
        self.own_head: Optional[nn.Module] = None        # set when the checkpoint brings shared_head.head

    @property
    def num_mtp_layers(self) -> int:
        return len(self.layers)

    def forward(self, inputs_embeds: torch.Tensor, previous_hidden: torch.Tensor, spec_step: int = 0) -> torch.Tensor:
        return self.layers[spec_step % len(self.layers)](inputs_embeds, previous_hidden)

    # ------------------------------------------------------------- weights
    def rewrite_name(self, name: str) -> Optional[str]:
        """Checkpoint name -> parameter path inside this module, or None if the tensor
        belongs to the target model."""
        m = _LAYER_RE.match(name)
        if m is None:
            return None
        idx, rest = int(m.group(1)), m.group(2)
        if idx < self.first_layer or idx >= self.first_layer + len(self.layers):
            return None
        i = idx - self.first_layer
        if rest.startswith("embed_tokens."):
            return "__shared_embedding__"
        if rest.startswith("shared_head.head."):
            return "__shared_head__"
        if rest.startswith("shared_head.norm."):
            return f"layers.{i}.shared_head_norm." + rest[len("shared_head.norm."):]
        if rest.split(".")[0] in _MTP_OWN:
            return f"layers.{i}.{rest}"
        return f"layers.{i}.mtp_block.{rest}"

    def split_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]):
        """Partition a checkpoint stream into (target-model tensors, MTP tensors renamed to
        ``model.layers.<idx>...`` paths relative to the block, shared tensors)."""
        mine: List[Tuple[str, torch.Tensor]] = []
        theirs: List[Tuple[str, torch.Tensor]] = []
        for name, t in weights:
            new = self.rewrite_name(name)
            if new is None:
                theirs.append((name, t))
            elif not new.startswith("__"):
                mine.append((new, t))
        return theirs, mine


def select_rows(hidden: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    return hidden.index_select(0, rows.long())


class _StandaloneMTP(nn.Module):
    """A draft model made of the MTP layers of a checkpoint alone, for deployments that load
    the draft as its own model (architectures ``DeepSeekMTPModel`` / ``OpenPanguMTPModel``).
    It owns an embedding and an LM head (the checkpoint usually repeats both under the MTP
    layer's prefix).  ``forward`` needs the target model's hidden states."""
    layer_cls_path = ("omni_npu_b200.models.deepseek", "DeepseekDecoderLayer")

    def __init__(self, engine_config: EngineConfig, device=None) -> None:
        super().__init__()
        import importlib

        from ..layers.embedding import ParallelLMHead, VocabParallelEmbedding
        cfg = engine_config.model
        self.config = cfg
        mod, name = self.layer_cls_path
        layer_cls = getattr(importlib.import_module(mod), name)
        self.embed_tokens = VocabParallelEmbedding(cfg.vocab_size, cfg.hidden_size, cfg.dtype, device)
        self.mtp = MultiTokenPredictor(engine_config, device,
                                       lambda idx, prefix: layer_cls(engine_config, idx, device, prefix))
        self.lm_head = ParallelLMHead(cfg.vocab_size, cfg.hidden_size, cfg.dtype, device)
        self.num_kv_layers = cfg.num_layers + self.mtp.num_mtp_layers      # cache indices follow the target's

    def forward(self, input_ids, positions, previous_hidden, spec_step: int = 0):
        return self.mtp(self.embed_tokens(input_ids), previous_hidden, spec_step)

    def compute_logits(self, hidden):
        return self.lm_head.compute_logits(hidden)

    def load_weights(self, weights: Iterable[Tuple[str, torch.Tensor]]) -> set:
        from .utils import load_stacked_weights
        renamed: List[Tuple[str, torch.Tensor]] = []
        for name, t in weights:
            new = self.mtp.rewrite_name(name)
            if new is None:
                if name in ("model.embed_tokens.weight", "lm_head.weight"):
                    renamed.append((name.replace("model.", ""), t))
                continue
            if new == "__shared_embedding__":
                renamed.append(("embed_tokens.weight", t))
            elif new == "__shared_head__":
                renamed.append(("lm_head.weight", t))
            else:
                renamed.append(("mtp." + new, t))
        stacked = [(".gate_up_proj", ".gate_proj", 0), (".gate_up_proj", ".up_proj", 1)]
        return load_stacked_weights(self, renamed, stacked, skip_substrings=("rotary_emb.inv_freq",))


class DeepSeekMTP(_StandaloneMTP):
    layer_cls_path = ("omni_npu_b200.models.deepseek", "DeepseekDecoderLayer")


class OpenPanguMTP(_StandaloneMTP):
    layer_cls_path = ("omni_npu_b200.models.pangu", "PanguUltraDecoderLayer")
