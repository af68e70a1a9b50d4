"""vLLM ``Platform`` for B200.

Device identity, distributed backend, worker / communicator / attention
backend / graph-wrapper class paths and configuration defaults, i.e. the same
responsibilities as ``NPUPlatform`` (omni_npu/platform.py:45-187).  The class
derives from vLLM's ``Platform`` when vLLM is importable; without vLLM a plain
base class keeps the module importable so the standalone engine and the tests
can still use its helpers.
"""
from __future__ import annotations

import contextlib
import os
from typing import Any, Optional, Tuple

import torch

from . import compat
from .logger import logger, update_vllm_logging_config

if compat.vllm_available():
    _Base = compat.platform_base()
    _Enum = compat.platform_enum()
else:  # pragma: no cover - exercised only without vLLM
    class _Base:  # type: ignore[no-redef]
        pass

    class _Enum:  # type: ignore[no-redef]
        OOT = "oot"

update_vllm_logging_config()

WORKER_CLS = "omni_npu_b200.worker.vllm_worker.B200Worker"
COMMUNICATOR_CLS = "omni_npu_b200.parallel.vllm_communicator.B200VllmCommunicator"
GRAPH_WRAPPER_CLS = "omni_npu_b200.compilation.cuda_graph.CUDAGraphWrapper"
COMPILE_BACKEND_CLS = "omni_npu_b200.compilation.eager_backend.EagerGraphBackend"
ATTN_BACKENDS = {
    "gqa": "omni_npu_b200.attention.vllm_backends.B200AttentionBackend",
    "mla": "omni_npu_b200.attention.vllm_backends.B200MLABackend",
    "dsa": "omni_npu_b200.attention.vllm_backends.B200DSABackend",
}
DEFAULT_BLOCK_SIZE = 16


class B200Platform(_Base):
    _enum = getattr(_Enum, "OOT", None)
    device_name: str = "cuda"
    device_type: str = "cuda"
    dispatch_key: str = "CUDA"
    ray_device_key: str = "GPU"
    dist_backend: str = "nccl"
    device_control_env_var: str = "CUDA_VISIBLE_DEVICES"
    simple_compile_backend: str = "eager"
    supported_quantization = ["fp8", "compressed-tensors", "b200-compressed-tensors"]

    # ------------------------------------------------------------ device
    @classmethod
    def set_device(cls, device: torch.device) -> None:
        torch.cuda.set_device(device)

    @classmethod
    def get_device_name(cls, device_id: int = 0) -> str:
        return torch.cuda.get_device_name(device_id)

    @classmethod
    def get_device_capability(cls, device_id: int = 0):
        major, minor = torch.cuda.get_device_capability(device_id)
        try:
            from vllm.platforms.interface import DeviceCapability
            return DeviceCapability(major=major, minor=minor)
        except Exception:
            return (major, minor)

    @classmethod
    def get_device_total_memory(cls, device_id: int = 0) -> int:
        return torch.cuda.get_device_properties(device_id).total_memory

    @classmethod
    def device_count(cls) -> int:
        return torch.cuda.device_count()

    @classmethod
    def mem_get_info(cls, device: Optional[torch.device] = None) -> Tuple[int, int]:
        return torch.cuda.mem_get_info(device)

    @classmethod
    def get_current_memory_usage(cls, device: Optional[torch.device] = None) -> float:
        torch.cuda.reset_peak_memory_stats(device)
        return torch.cuda.max_memory_allocated(device)

    @classmethod
    def inference_mode(cls):
        return torch.inference_mode(mode=True)

    @classmethod
    def is_pin_memory_available(cls) -> bool:
        return True

    @classmethod
    def manual_seed_all(cls, seed: int) -> None:
        torch.cuda.manual_seed_all(seed)

    def is_cuda_alike(self) -> bool:
        return True

    def is_sleep_mode_available(self) -> bool:
        return True

    # ------------------------------------------------------------ hooks
    @classmethod
    def import_kernels(cls) -> None:
        """Load the native extension, patch the compile decorators so that prefill
        steps run eagerly, and register the KV connectors."""
        from . import ops
        ops.load_extension(required=True)
        # optional hooks: a failure is logged and does not keep the platform from loading
        try:
            from .compilation.decorators import patch_compile_decorators
            patch_compile_decorators()
        except Exception as e:
            logger.warning("compile-decorator patch not installed: %s", e)
        try:
            from .kv_transfer.register import register_connectors
            register_connectors()
        except Exception as e:
            logger.warning("KV connectors not registered: %s", e)

    @classmethod
    def pre_register_and_update(cls, parser=None) -> None:
        """Runs before the engine config exists: registers the out-of-tree layer
        overrides and quantisation configs and extends the CLI."""
        try:
            from .layers import vllm_custom_ops  # noqa: F401  (@register_oot side effects)
        except Exception as e:
            logger.warning("out-of-tree custom ops not registered: %s", e)
        if parser is not None:
            try:
                from .patches.common.engine_args import add_cli_args
                add_cli_args(parser)
            except Exception as e:
                logger.warning("CLI arguments not added: %s", e)

    @classmethod
    def check_and_update_config(cls, vllm_config: Any) -> None:
        pc = getattr(vllm_config, "parallel_config", None)
        if pc is not None and getattr(pc, "worker_cls", "auto") == "auto":
            pc.worker_cls = WORKER_CLS
        cc = getattr(vllm_config, "cache_config", None)
        if cc is not None and not getattr(cc, "block_size", None):
            cc.block_size = DEFAULT_BLOCK_SIZE
        sc = getattr(vllm_config, "scheduler_config", None)
        if sc is not None and getattr(sc, "async_scheduling", False) \
                and os.environ.get("OMNI_B200_VLLM_ASYNC", "1") == "0":
            # OMNI_B200_VLLM_ASYNC=0: strictly alternating schedule / execute (debugging aid)
            with contextlib.suppress(Exception):
                sc.async_scheduling = False
        comp = getattr(vllm_config, "compilation_config", None)
        if comp is not None:
            # fusion passes of the tracing compiler do not apply: the kernels are already fused
            pass_cfg = getattr(comp, "pass_config", None)
            for name in ("enable_fusion", "enable_attn_fusion", "enable_noop", "fuse_norm_quant",
                         "fuse_act_quant", "fuse_attn_quant"):
                if pass_cfg is not None and hasattr(pass_cfg, name):
                    with contextlib.suppress(Exception):
                        setattr(pass_cfg, name, False)
        ac = getattr(vllm_config, "additional_config", None) or {}
        vllm_config.b200_options = dict(ac)
        logger.info("B200 platform configured: worker=%s block_size=%s", WORKER_CLS,
                    getattr(cc, "block_size", None))

    @classmethod
    def update_block_size_for_backend(cls, vllm_config: Any) -> None:
        """The worker sizes its own paged cache from ``cache_config.block_size`` when it is built;
        the block size must not change afterwards."""

    @classmethod
    def get_attn_backend_cls(cls, selected_backend=None, attn_selector_config=None, num_heads=None,
                             *args, **kwargs) -> str:
        use_mla = bool(getattr(attn_selector_config, "use_mla", kwargs.get("use_mla", False)))
        use_sparse = bool(getattr(attn_selector_config, "use_sparse", kwargs.get("use_sparse", False)))
        if use_mla and use_sparse:
            return ATTN_BACKENDS["dsa"]
        if use_mla:
            return ATTN_BACKENDS["mla"]
        return ATTN_BACKENDS["gqa"]

    @classmethod
    def get_device_communicator_cls(cls) -> str:
        return COMMUNICATOR_CLS

    @classmethod
    def get_punica_wrapper(cls) -> str:
        return "vllm.lora.punica_wrapper.punica_gpu.PunicaWrapperGPU"

    @classmethod
    def support_static_graph_mode(cls) -> bool:
        return True

    @classmethod
    def get_static_graph_wrapper_cls(cls) -> str:
        return GRAPH_WRAPPER_CLS

    @classmethod
    def get_compile_backend(cls) -> str:
        return COMPILE_BACKEND_CLS

    @classmethod
    def support_hybrid_kv_cache(cls) -> bool:
        return False

    @classmethod
    def use_custom_allreduce(cls) -> bool:
        return True

    @classmethod
    def supports_fp8(cls) -> bool:
        return True

    @classmethod
    def opaque_attention_op(cls) -> bool:
        return True

    @classmethod
    def verify_quantization(cls, quant: str) -> None:
        if quant and quant not in cls.supported_quantization:
            raise ValueError(f"{quant} quantization is not supported on the B200 platform")


class B200CpuPlatform(B200Platform):
    """The same plugin surface on a machine without a GPU: device ``cpu``, gloo process groups,
    the fp32 reference ops instead of the CUDA kernels.  Selected with ``OMNI_B200_PLUGIN=cpu``;
    meant for plumbing tests of the platform / worker / model runner under a vLLM engine."""
    device_name: str = "cpu"
    device_type: str = "cpu"
    dispatch_key: str = "CPU"
    dist_backend: str = "gloo"
    device_control_env_var: str = "OMNI_B200_CPU_VISIBLE_DEVICES"

    @classmethod
    def set_device(cls, device: torch.device) -> None:
        pass

    @classmethod
    def get_device_name(cls, device_id: int = 0) -> str:
        return "cpu"

    @classmethod
    def get_device_capability(cls, device_id: int = 0):
        return None

    @classmethod
    def get_device_total_memory(cls, device_id: int = 0) -> int:
        import psutil
        return psutil.virtual_memory().total

    @classmethod
    def device_count(cls) -> int:
        return 1

    @classmethod
    def mem_get_info(cls, device: Optional[torch.device] = None) -> Tuple[int, int]:
        import psutil
        vm = psutil.virtual_memory()
        return vm.available, vm.total

    @classmethod
    def get_current_memory_usage(cls, device: Optional[torch.device] = None) -> float:
        return 0.0

    @classmethod
    def is_pin_memory_available(cls) -> bool:
        return False

    @classmethod
    def manual_seed_all(cls, seed: int) -> None:
        torch.manual_seed(seed)

    def is_cuda_alike(self) -> bool:
        return False

    def is_sleep_mode_available(self) -> bool:
        return False

    @classmethod
    def import_kernels(cls) -> None:
        try:
            from .kv_transfer.register import register_connectors
            register_connectors()
        except Exception as e:
            logger.warning("KV connectors not registered: %s", e)

    @classmethod
    def use_custom_allreduce(cls) -> bool:
        return False

    @classmethod
    def get_punica_wrapper(cls) -> str:
        return "vllm.lora.punica_wrapper.punica_cpu.PunicaWrapperCPU"
