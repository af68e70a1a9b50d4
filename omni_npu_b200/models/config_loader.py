"""Deployment plans ("best-practice" configurations) chosen from the model's
fingerprint, its quantisation, the role of this instance and the performance mode.

A plan is a small JSON document with two sections:

``parallel``  per-layer process groups and transforms (``layer_parallel_config``),
              dense-MLP / o_proj / eh_proj group sizes, sequence-parallel width,
              redundant shared experts, input splitting;
``kernels``   which fused paths and tuning knobs the model code should use on
              B200: fused KV-RMSNorm+RoPE+cache write, MoE dispatch mode for prefill
              and decode, peer-memory all-reduce fused with the next norm,
              CTA-pair GEMM for prefill, L2 prefetch budgets (MiB), DSA, MLA
              all-to-all for long prefill, micro-batching.

Lookup: ``configs/fingerprints.json`` maps a model name to the HF-config fields
that identify it; ``configs/<mode>/index.json`` maps (model, hardware, precision)
to plan files per PD scheme (``"1P1D"``, ``"hybrid"``, ``"pd_elastic_scaling"``),
with a prefill file and a decode file for disaggregated serving.  Unknown keys in
a plan are ignored, missing ones keep their defaults, and an unknown task falls
back to the defaults with a warning.

Same job as omni_npu/v1/models/config_loader/loader.py:22-360 and the older
omni_npu/v0/models/config_loader/loader.py:48-170 (its extra knobs live in
``KernelPlan`` too); the plans themselves are written for 8 x B200 boxes.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field, fields
from pathlib import Path
from typing import Any, Dict, Mapping, Optional, Tuple

from ..logger import logger

CONFIG_ROOT = Path(__file__).resolve().parent / "configs"
HARDWARE = "B200"


@dataclass
class TaskProfile:
    model_name: str = "llama"
    hardware_platform: str = HARDWARE
    is_pd_disaggregation: bool = False
    is_prefill_node: bool = True            # decode instance when False
    quant_type: str = "bf16"
    prefill_node_num: int = 1
    decode_node_num: int = 1
    enable_eplb: bool = False
    enable_pd_elastic_scaling: bool = False
    enable_chunked_prefill: bool = False
    graph_mode: str = "cuda_graph"          # "eager_mode" | "cuda_graph"
    enable_low_latency: bool = False
    enable_host_kv_pool: bool = False


@dataclass
class ParallelPlan:
    dense_mlp_tp_size: int = 1
    o_proj_tp_size: int = 1
    eh_proj_tp_size: int = 1
    attn_sp_size: int = 1
    redundancy_shared_expert_num: int = 0
    enable_share_expert_tp: bool = False
    input_split: bool = False
    layer_parallel_config: Dict[str, Any] = field(default_factory=dict)


@dataclass
class KernelPlan:
    # attention front end
    enable_kv_rmsnorm_rope_cache: bool = True
    enable_mla_prolog: bool = False
    enable_dsa: bool = True
    merge_qkv: bool = True
    fa_quant: bool = False
    # MoE
    prefill_moe_all_to_all: bool = True
    decode_moe_dispatch_combine: bool = True
    moe_multi_stream_tune: bool = False
    best_ep: bool = False
    shared_experts_to_grouped_gemm: bool = False
    fuse_swiglu_quant: bool = False
    experts_pruning: bool = False
    # communication
    decode_flash_comm_1: bool = True          # token-sharded residual stream between layers
    fused_allreduce_norm: bool = True         # peer-memory all-reduce + residual + RMSNorm in one kernel
    two_stage_comm: bool = False              # hierarchical collectives: pointless on one NVSwitch domain
    enable_pipeline_comm: bool = False
    enable_round_pipeline_comm: bool = False
    prefill_enable_long_seq: bool = False
    prefill_enable_mla_alltoall: bool = False
    prefill_enable_mla_alltoall_local: bool = False
    # GEMM / scheduling
    cta_pair_gemm_min_m: int = 1024
    enable_prefill_micro_batch: bool = False
    enable_mlp_seq_split: bool = False
    control_accept_rate: float = -1.0         # outside [0, 1] = off; forces the MTP acceptance rate (testing only)
    mtp_remove_redundant_kv: bool = False
    # L2 prefetch budgets, MiB (0 = off)
    enable_prefetch: bool = True
    expert_gate_up_prefetch: int = 24
    expert_down_prefetch: int = 12
    dense_mlp_prefetch: int = 32
    lm_head_prefetch: int = 48
    attn_prefetch: int = 32
    shared_expert_gate_up_prefetch: int = 12
    shared_expert_down_prefetch: int = 6
    use_host_kv_pool: bool = False

    def __post_init__(self) -> None:
        if not self.enable_prefetch:
            self.zero_prefetch()
        if os.getenv("ENABLE_OMNI_CACHE", "0") == "1":
            self.use_host_kv_pool = True
        if self.enable_pipeline_comm and self.enable_round_pipeline_comm:
            raise ValueError("enable_pipeline_comm and enable_round_pipeline_comm are mutually exclusive")
        # the 126 MB L2 cannot hold more than this many MiB of hints at once
        total = (self.expert_gate_up_prefetch + self.expert_down_prefetch + self.attn_prefetch)
        if total > 96:
            raise ValueError(f"prefetch budgets for one layer add up to {total} MiB, more than L2 can keep")

    def zero_prefetch(self) -> None:
        for f in fields(self):
            if f.name.endswith("_prefetch") and f.name != "enable_prefetch":
                setattr(self, f.name, 0)


@dataclass
class ModelExtraConfig:
    parallel: ParallelPlan = field(default_factory=ParallelPlan)
    kernels: KernelPlan = field(default_factory=KernelPlan)
    task: TaskProfile = field(default_factory=TaskProfile)
    source: Optional[str] = None            # plan file the values came from

    # names the reference's model code uses for the same three sections
    @property
    def parall_config(self) -> ParallelPlan:
        return self.parallel

    @property
    def operator_opt_config(self) -> KernelPlan:
        return self.kernels

    @property
    def task_config(self) -> TaskProfile:
        return self.task

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=2, default=str)


model_extra_config = ModelExtraConfig()


# ------------------------------------------------------------------ helpers
def _keep_known(cls, data: Mapping[str, Any]) -> Dict[str, Any]:
    names = {f.name for f in fields(cls)}
    unknown = sorted(set(data) - names)
    if unknown:
        logger.debug("%s: ignoring unknown keys %s", cls.__name__, unknown)
    return {k: v for k, v in data.items() if k in names}


def _read_json(path: Path):
    try:
        with open(path, "r") as f:
            return json.load(f)
    except json.JSONDecodeError as e:
        raise RuntimeError(f"invalid JSON in {path}: {e}") from e


def _as_dict(hf_config) -> Dict[str, Any]:
    if isinstance(hf_config, Mapping):
        return dict(hf_config)
    if hasattr(hf_config, "to_dict"):
        try:
            return dict(hf_config.to_dict())
        except Exception:
            pass
    return dict(vars(hf_config))


def _bits(v) -> int:
    return int(min(v.values())) if isinstance(v, Mapping) else int(v)


def quant_type_of(hf: Mapping[str, Any]) -> str:
    """'bf16', 'fp8' (block-scaled fp8 checkpoints), or 'w<W>a<A>c<C>' for
    int-quantised compressed-tensors checkpoints ('..._fa_c8' for the quantised
    attention scheme)."""
    q = hf.get("quantization_config")
    if not q:
        return "bf16"
    if str(q.get("quant_method", "")).lower() == "fp8" or str(q.get("fmt", "")).lower() == "e4m3":
        return "fp8"
    if str(q.get("format", "")).strip() != "int-quantized":
        return "bf16"
    g0 = q["config_groups"]["group_0"]
    name = f"w{_bits(g0['weights']['num_bits'])}a{_bits(g0['input_activations']['num_bits'])}"
    kv = q.get("kv_cache_scheme")
    if kv == "Opti-C8":
        return name + "_fa_c8"
    if isinstance(kv, Mapping):
        return f"{name}c{kv['num_bits']}"
    return name + "c16"


def parse_hf_config(hf_config, config_root: Path = CONFIG_ROOT) -> Tuple[str, str]:
    """(model name, quant type).  The name is the unique entry of
    ``fingerprints.json`` whose fields all equal the HF config's; no match falls
    back to ``model_type``; several matches are settled by ``model_type`` when it
    is itself one of the candidates."""
    hf = _as_dict(hf_config)
    prints = _read_json(config_root / "fingerprints.json")
    matches = [name for name, want in prints.items()
               if all(k in hf and hf[k] == v for k, v in want.items())]
    model_type = hf.get("model_type", "unknown")
    if not matches:
        name = model_type
    elif len(matches) == 1:
        name = matches[0]
    elif model_type in matches:
        name = model_type
    else:
        raise RuntimeError(f"HF config matches several known models {matches}; cannot pick a deployment plan")
    return name, quant_type_of(hf)


def pd_scheme_of(task: TaskProfile) -> str:
    if task.is_pd_disaggregation:
        return "pd_elastic_scaling" if task.enable_pd_elastic_scaling else \
            f"{task.prefill_node_num}P{task.decode_node_num}D"
    return "hybrid"


def find_plan_file(task: TaskProfile, config_root: Path = CONFIG_ROOT) -> Optional[Path]:
    mode = "latency" if task.enable_low_latency else "throughput"
    index_path = config_root / mode / "index.json"
    if not index_path.exists():
        return None
    entry = next((e for e in _read_json(index_path)
                  if e["model"] == task.model_name and e["hardware"] == task.hardware_platform
                  and e["precision"] == task.quant_type), None)
    label = f"{task.model_name}_{task.quant_type}_{task.hardware_platform}_{pd_scheme_of(task)}"
    if entry is None:
        logger.warning("no deployment plan for %s in mode '%s'; using defaults", label, mode)
        return None
    files = entry["configs"].get(pd_scheme_of(task))
    if not files:
        logger.warning("no deployment plan for %s in mode '%s'; using defaults", label, mode)
        return None
    if task.is_pd_disaggregation:
        rel = files.get("prefill_config_file" if task.is_prefill_node else "decode_config_file")
    else:
        rel = files.get("config_file")
    if rel is None:
        return None
    path = config_root / mode / rel
    if not path.exists():
        raise RuntimeError(f"task {label} needs plan file {path}, which does not exist")
    return path


def apply_eager_mode(cfg: ModelExtraConfig) -> None:
    """Without CUDA graphs there is no side-stream scheduling to tune and prefetch
    hints only add launches: switch them off (omni_npu/v1/models/config_loader/features.py:14-34)."""
    if cfg.task.graph_mode != "eager_mode":
        return
    k = cfg.kernels
    k.moe_multi_stream_tune = False
    k.enable_prefetch = False
    k.zero_prefetch()
    logger.warning("eager mode: multi-stream MoE tuning and weight prefetch are disabled")


def build_model_extra_config(task: TaskProfile, config_root: Path = CONFIG_ROOT) -> ModelExtraConfig:
    path = find_plan_file(task, config_root)
    cfg = ModelExtraConfig(task=task)
    if path is not None:
        data = _read_json(path)
        cfg.parallel = ParallelPlan(**_keep_known(ParallelPlan, data.get("parallel", data.get("model_parallel_config", {}))))
        cfg.kernels = KernelPlan(**_keep_known(KernelPlan, data.get("kernels", data.get("operator_optimization_config", {}))))
        cfg.source = str(path)
        logger.info("deployment plan for %s_%s_%s_%s: %s", task.model_name, task.quant_type,
                    task.hardware_platform, pd_scheme_of(task), path)
    apply_eager_mode(cfg)
    if task.enable_host_kv_pool:
        cfg.kernels.use_host_kv_pool = True
    return cfg


def update_task_config(**kw) -> ModelExtraConfig:
    """Change fields of the current task and reload the plan (module-level singleton)."""
    task = model_extra_config.task
    for k, v in kw.items():
        if hasattr(task, k):
            setattr(task, k, v)
    new = build_model_extra_config(task)
    model_extra_config.parallel, model_extra_config.kernels = new.parallel, new.kernels
    model_extra_config.task, model_extra_config.source = new.task, new.source
    return model_extra_config


def load_model_extra_config(hf_config, *, enforce_eager: bool = False, enable_chunked_prefill: bool = False,
                            enable_eplb: bool = False, additional_config: Optional[Mapping[str, Any]] = None,
                            env: Optional[Mapping[str, str]] = None) -> ModelExtraConfig:
    """Fill the module-level ``model_extra_config`` for this process.  The instance
    role comes from ``ROLE`` (``prefill`` / ``decode``; unset = hybrid), the pod counts
    from ``PREFILL_POD_NUM`` / ``DECODE_POD_NUM``."""
    env = os.environ if env is None else env
    extra = dict(additional_config or {})
    name, quant = parse_hf_config(hf_config)
    role = env.get("ROLE")
    return update_task_config(
        model_name=name, quant_type=quant, hardware_platform=HARDWARE,
        is_pd_disaggregation=role is not None, is_prefill_node=(role == "prefill") if role else True,
        prefill_node_num=int(env.get("PREFILL_POD_NUM", 1)), decode_node_num=int(env.get("DECODE_POD_NUM", 1)),
        enable_eplb=enable_eplb, enable_chunked_prefill=enable_chunked_prefill,
        enable_low_latency=bool(extra.get("enable_low_latency", False)),
        enable_pd_elastic_scaling=bool(extra.get("enable_pd_elastic_scaling", False)),
        enable_host_kv_pool=bool(extra.get("enable_omni_cache", extra.get("enable_host_kv_pool", False))),
        graph_mode="eager_mode" if enforce_eager else "cuda_graph")


def is_mlp_weight_prefetch_on() -> bool:
    k = model_extra_config.kernels
    return bool(k.enable_prefetch and k.expert_gate_up_prefetch and k.expert_down_prefetch)


def apply_to_runtime(cfg: Optional[ModelExtraConfig] = None) -> None:
    """Push the plan into the running process: per-layer groups + transforms, and the
    GEMM routing threshold.  Collective: every rank calls it with the same plan."""
    from .. import ops
    from ..parallel import state as pstate
    cfg = cfg or model_extra_config
    if cfg.parallel.layer_parallel_config and pstate.model_parallel_is_initialized():
        pstate.apply_layer_parallel_config(cfg.parallel.layer_parallel_config)
    if "OMNI_B200_GEMM_PAIR_MIN_M" not in os.environ and cfg.source is not None:
        ops.PAIR_MIN_M = int(cfg.kernels.cta_pair_gemm_min_m)
