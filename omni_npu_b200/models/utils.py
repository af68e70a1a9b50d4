"""Weight-loading helpers shared by the model classes."""
from __future__ import annotations

import glob
import json
import os
from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Set, Tuple

import torch
from torch import nn


def default_weight_loader(param: nn.Parameter, loaded: torch.Tensor) -> None:
    if param.shape != loaded.shape:
        raise ValueError(f"shape mismatch: parameter {tuple(param.shape)} vs checkpoint {tuple(loaded.shape)}")
    param.data.copy_(loaded if param.dtype == torch.float8_e4m3fn else loaded.to(param.dtype))


def _owner_loader(model: nn.Module, name: str):
    """The ``weight_loader`` of the module that owns parameter ``name``, if any."""
    mod_name = name.rsplit(".", 1)[0] if "." in name else ""
    try:
        mod = model.get_submodule(mod_name)
    except AttributeError:
        return None
    return getattr(mod, "weight_loader", None)


def load_stacked_weights(model: nn.Module, weights: Iterable[Tuple[str, torch.Tensor]],
                         stacked: Sequence[Tuple[str, str, object]],
                         skip_substrings: Sequence[str] = (),
                         rename=None) -> Set[str]:
    """Generic loader: checkpoint tensors whose name contains a ``stacked`` source
    pattern go into the fused parameter with the given shard id; everything else
    is loaded by name through the owning module's ``weight_loader``."""
    params: Dict[str, nn.Parameter] = dict(model.named_parameters())
    loaded: Set[str] = set()
    for name, tensor in weights:
        if any(s in name for s in skip_substrings):
            continue
        if rename is not None:
            name = rename(name)
            if name is None:
                continue
        done = False
        for fused, src, shard in stacked:
            if src not in name:
                continue
            target = name.replace(src, fused)
            if target not in params:
                continue
            loader = _owner_loader(model, target)
            loader(params[target], tensor, shard)
            loaded.add(target)
            done = True
            break
        if done:
            continue
        if name not in params:
            continue
        loader = _owner_loader(model, name)
        if loader is not None:
            loader(params[name], tensor)
        else:
            default_weight_loader(params[name], tensor)
        loaded.add(name)
    return loaded


def iter_safetensors(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yield (name, tensor) from every ``*.safetensors`` shard of an HF directory
    (index file order when present)."""
    from safetensors import safe_open
    index = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        files = [os.path.join(path, x) for x in files]
    else:
        files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no safetensors files under {path}")
    for fn in files:
        with safe_open(fn, framework="pt", device="cpu") as f:
            for k in f.keys():
                yield k, f.get_tensor(k)


@torch.no_grad()
def random_init_(model: nn.Module, seed: int = 0, std: float = 0.02, by_name: Optional[bool] = None) -> None:
    """Deterministic random initialisation (normal, std 0.02; norm weights 1).
    Each parameter has its own stream, seeded from ``seed`` and the parameter's
    index in name order, or (``by_name``; default: ``OMNI_B200_INIT_BY_NAME=1``;
    always used for pipeline stages) from a checksum of its NAME, so that a stage
    holding a subset of the layers draws the same values for them as a process
    holding the whole model.  Tensor-parallel shards are drawn per shard (a shard
    is not a slice of the unsharded draw)."""
    import zlib
    if by_name is None:
        by_name = os.environ.get("OMNI_B200_INIT_BY_NAME", "0") == "1"
    g = torch.Generator(device="cpu")
    for i, (name, p) in enumerate(sorted(model.named_parameters(), key=lambda kv: kv[0])):
        if by_name:
            i = zlib.crc32(name.encode()) % 1000003
        g.manual_seed(seed * 1000003 + i)
        if "norm" in name and p.dim() == 1 and "bias" not in name:
            p.data.fill_(1.0)
        elif name.endswith("weight_scale_inv"):
            p.data.fill_(1.0)
        elif name.endswith(".bias") or "e_score_correction_bias" in name:
            p.data.zero_()
        elif p.device.type == "cuda" and p.numel() >= (1 << 22):
            gg = torch.Generator(device=p.device)
            gg.manual_seed(seed * 1000003 + i)
            tmp = torch.empty(p.shape, dtype=torch.bfloat16, device=p.device).normal_(0.0, std, generator=gg)
            p.data.copy_(tmp if p.dtype != torch.float8_e4m3fn else (tmp.float() * (448 * 0.25 / (3 * std))).to(p.dtype))
            del tmp
        else:
            tmp = torch.empty(p.shape, dtype=torch.float32).normal_(0.0, std, generator=g)
            p.data.copy_(tmp.to(p.dtype) if p.dtype != torch.float8_e4m3fn
                         else (tmp * (448 * 0.25 / (3 * std))).to(p.dtype))


# ------------------------------------------------------------------ pipeline parallelism
class PPMissingLayer(nn.Module):
    """Placeholder for a module that lives on another pipeline stage: no
    parameters, returns its first input unchanged.  Keeping the placeholder in
    the ``ModuleList`` leaves the checkpoint's layer numbering intact, so weight
    names need no translation per stage.
    (reference: ``PPMissingLayer`` use in omni_npu/v1/models/deepseek/deepseek_v3.py:370-393)"""

    def forward(self, *args, **kwargs):
        return args[0] if args else next(iter(kwargs.values()))


class IntermediateTensors:
    """Named activations handed from one pipeline stage to the next
    (``hidden_states`` and, for pre-norm decoders that carry it, ``residual``).
    (reference: ``IntermediateTensors`` in omni_npu/v1/models/deepseek/deepseek_v3.py:436-456 and
    the runner's buffer allocation in omni_npu/worker/npu_model_runner.py:494-508)"""

    def __init__(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.tensors = tensors

    def __getitem__(self, key: str) -> torch.Tensor:
        return self.tensors[key]

    def __contains__(self, key: str) -> bool:
        return key in self.tensors

    def items(self):
        return self.tensors.items()


def pp_layer_range(num_layers: int, pp_rank: int, pp_size: int) -> Tuple[int, int]:
    """[start, end) of the decoder layers owned by stage ``pp_rank``.  Layers are
    split evenly; a remainder goes to the middle stages first and the last stage
    last, because the first stage also holds the embedding and the last the LM
    head and sampler.  ``OMNI_B200_PP_LAYER_PARTITION`` (comma-separated counts)
    overrides the split."""
    override = os.environ.get("OMNI_B200_PP_LAYER_PARTITION")
    if override:
        counts = [int(x) for x in override.split(",")]
        if len(counts) != pp_size or sum(counts) != num_layers or min(counts) < 0:
            raise ValueError(f"OMNI_B200_PP_LAYER_PARTITION={override!r} does not split {num_layers} "
                             f"layers over {pp_size} stages")
    else:
        base, rem = divmod(num_layers, pp_size)
        counts = [base] * pp_size
        order = list(range(1, pp_size - 1)) + [0, pp_size - 1]
        for i in range(rem):
            counts[order[i % pp_size]] += 1
    start = sum(counts[:pp_rank])
    return start, start + counts[pp_rank]


def build_pipeline_layers(num_layers: int, make_layer, pp_group) -> Tuple[nn.ModuleList, int, int]:
    """``ModuleList`` of ``num_layers`` entries in which only this stage's layers are real
    (``make_layer(global_index)``), the rest ``PPMissingLayer``.  Layers are built with their
    GLOBAL index (dense-vs-MoE pattern, window pattern, weight names); afterwards every
    ``layer_idx`` attribute inside them, which indexes the per-stage list of KV caches, is
    shifted to the position within the stage.  ``pp_group`` None = no pipeline."""
    if pp_group is None or pp_group.world_size == 1:
        return nn.ModuleList([make_layer(i) for i in range(num_layers)]), 0, num_layers
    start, end = pp_layer_range(num_layers, pp_group.rank_in_group, pp_group.world_size)
    layers = nn.ModuleList([make_layer(i) if start <= i < end else PPMissingLayer() for i in range(num_layers)])
    for layer in layers[start:end]:
        for m in layer.modules():
            if isinstance(getattr(m, "layer_idx", None), int):
                m.layer_idx -= start
    return layers, start, end
