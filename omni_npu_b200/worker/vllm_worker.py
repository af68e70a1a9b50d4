"""vLLM worker for B200.

A B200 is a CUDA device, so vLLM's own GPU worker and model runner already drive it; this
class derives from them and adds what the platform plugin promises on top
(omni_npu/worker/npu_worker.py:77-299 is the reference's counterpart, which has to replace
far more because its device is not CUDA):

* the device communicator, attention backends, custom ops, KV connector and patches are
  installed by the platform / plugin entry points before the worker is built;
* sleep mode routes model weights and KV cache through the VMM pool of
  ``worker/mem_pool.py`` (physical memory released on ``sleep``, restored on ``wake_up``);
* the best-practice deployment plan for the model is loaded after ``init_device`` and its
  per-layer groups are created;
* the profiler can be started by a token-count trigger (``VLLM_TORCH_PROFILER_DIR`` +
  ``PROFILER_TOKEN_THRESHOLD`` / ``PROFILER_STOP_STEP``);
* token recovery wraps ``execute_model`` when ``USE_HA=1``.
"""
from __future__ import annotations

import os
from typing import Any, Optional

from .. import compat
from ..ha.monitor import token_recover_wrapper
from ..logger import logger

if compat.vllm_available():
    try:
        from vllm.v1.worker.gpu_worker import Worker as _GPUWorker
    except Exception:                                     # CPU-only environment without the CUDA worker
        _GPUWorker = object
else:
    _GPUWorker = object


class B200Worker(_GPUWorker):  # type: ignore[misc, valid-type]
    def __init__(self, *args: Any, **kwargs: Any) -> None:
        super().__init__(*args, **kwargs)
        self.ha_agent = None
        self._profile_threshold = int(os.environ.get("PROFILER_TOKEN_THRESHOLD", "0"))
        self._profile_stop_step = int(os.environ.get("PROFILER_STOP_STEP", "5"))
        self._profile_steps_left = 0

    # ---------------------------------------------------------------- set-up
    def init_device(self) -> None:
        super().init_device()
        try:
            from ..models import config_loader
            mc = self.vllm_config.model_config
            config_loader.load_model_extra_config(
                mc.hf_config, enforce_eager=bool(getattr(mc, "enforce_eager", False)),
                enable_chunked_prefill=bool(getattr(self.vllm_config.scheduler_config, "enable_chunked_prefill", False)),
                enable_eplb=bool(getattr(self.vllm_config.parallel_config, "enable_eplb", False)),
                additional_config=getattr(self.vllm_config, "additional_config", None))
            config_loader.apply_to_runtime()
        except Exception as e:                             # a missing plan is not fatal: defaults apply
            logger.warning("deployment plan not applied: %s", e)
        from ..ha.common import HAEnv
        env = HAEnv.from_environ()
        if env.use_ha:
            from ..ha.monitor import HAWorkerAgent
            self.ha_agent = HAWorkerAgent(env, getattr(self, "rank", 0), getattr(self, "local_rank", 0)).start()

    # -------------------------------------------------------------- sleep mode
    def sleep(self, level: int = 1) -> None:
        from .mem_pool import B200MemAllocator
        alloc = B200MemAllocator.get_instance()
        released = alloc.sleep(offload_tags=("weights",) if level == 1 else ())
        logger.info("sleep level %d: %.2f GiB released", level, released / 2**30)

    def wake_up(self, tags: Optional[list] = None) -> None:
        from .mem_pool import B200MemAllocator
        B200MemAllocator.get_instance().wake_up(tags)

    def _maybe_pool(self, tag: str):
        import contextlib
        if getattr(self.vllm_config.model_config, "enable_sleep_mode", False):
            from .mem_pool import B200MemAllocator
            return B200MemAllocator.get_instance().use_memory_pool(tag=tag)
        return contextlib.nullcontext()

    def load_model(self, *args: Any, **kwargs: Any) -> None:
        with self._maybe_pool("weights"):
            super().load_model(*args, **kwargs)

    def initialize_from_config(self, kv_cache_config) -> None:
        with self._maybe_pool("kv_cache"):
            super().initialize_from_config(kv_cache_config)

    # ---------------------------------------------------------------- running
    @token_recover_wrapper
    def execute_model(self, scheduler_output, *args: Any, **kwargs: Any):
        prof = getattr(self, "profiler", None)
        if self._profile_threshold and prof is not None:
            total = getattr(scheduler_output, "total_num_scheduled_tokens", 0)
            if self._profile_steps_left == 0 and total == self._profile_threshold:
                prof.start()
                self._profile_steps_left = self._profile_stop_step
        out = super().execute_model(scheduler_output, *args, **kwargs)
        if self._profile_steps_left > 0:
            self._profile_steps_left -= 1
            if self._profile_steps_left == 0 and prof is not None:
                prof.stop()
        return out

    # token-recovery hooks (ha/monitor.py)
    def stop_device(self) -> None:
        import torch

        from ..parallel import state as pstate
        try:
            torch.cuda.synchronize()
        except Exception as e:
            logger.warning("synchronize during stop_device: %s", e)
        pstate.abort_communicators()

    def restart_device(self) -> None:
        import torch
        torch.cuda.empty_cache()

    def reinit_process_group(self) -> None:
        from ..parallel import state as pstate
        pstate.reinit_communicators()
