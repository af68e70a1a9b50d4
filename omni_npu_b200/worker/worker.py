"""Per-device worker: device and process-group set-up, model loading, memory
profiling, KV-cache creation, graph capture and step execution.

Counterpart of ``NPUWorker`` (omni_npu/worker/npu_worker.py:38-291):
``init_device`` (:77-120), ``determine_available_memory`` (:123-159),
``initialize_from_config`` (:164-179), ``compile_or_warm_up_model`` (:199-202),
``execute_model`` with token-threshold profiling (:229-246) and the profiler
set-up (:248-284).
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch

from .. import ops
from ..config import EngineConfig
from ..engine.scheduler import SchedulerOutput
from ..ha.monitor import token_recover_wrapper
from ..logger import logger
from ..parallel import state as pstate
from .model_runner import ModelRunner


class Worker:
    def __init__(self, config: EngineConfig, local_rank: int = 0, rank: int = 0,
                 distributed_init_method: Optional[str] = None, is_driver_worker: bool = True) -> None:
        self.config = config
        self.local_rank = local_rank
        self.rank = rank
        self.ha_agent = None            # token recovery (ha/monitor.py), off unless enabled
        self.distributed_init_method = distributed_init_method
        self.is_driver_worker = is_driver_worker
        self.device: Optional[torch.device] = None
        self.model_runner: Optional[ModelRunner] = None
        self.profiler = None
        self._profile_steps_left = 0
        self._profile_threshold = int(os.environ.get("PROFILER_TOKEN_THRESHOLD", "0"))
        self._profile_stop_step = int(os.environ.get("PROFILER_STOP_STEP", "5"))

    # -------------------------------------------------------------- set-up
    def init_device(self) -> None:
        if os.environ.get("PROFILING_NAMELIST"):
            from ..utils.trace import apply_namelist
            apply_namelist()        # wrap the functions the name list asks for before anything runs
        want_cuda = self.config.device in ("auto", "cuda") and torch.cuda.is_available()
        if self.config.device == "cuda" and not want_cuda:
            raise RuntimeError("device='cuda' requested but CUDA is not available")
        if want_cuda:
            torch.cuda.set_device(self.local_rank)
            self.device = torch.device("cuda", self.local_rank)
            ops.load_extension(required=True)
            self._init_free, self._init_total = torch.cuda.mem_get_info(self.device)
        else:
            self.device = torch.device("cpu")
        pc = self.config.parallel
        if not pstate.model_parallel_is_initialized():
            pstate.init_distributed(self.device, init_method=self.distributed_init_method)
            pstate.init_model_parallel(pc.tensor_parallel_size, pc.pipeline_parallel_size,
                                       pc.data_parallel_size, self.device,
                                       pcp=pc.prefill_context_parallel_size)
            for key, spec in (pc.layer_parallel_config or {}).items():
                if isinstance(spec, dict) and "tp_size_or_ranks" in spec:
                    pstate.register_layer_group(key, spec["tp_size_or_ranks"])
        if self.device.type == "cuda" and pc.tensor_parallel_size > 1 and self.config.fused_collectives:
            from ..parallel.symm_mem import attach_symmetric_memory
            attach_symmetric_memory(pstate.get_tp_group(), self.device)
        torch.manual_seed(self.config.seed)
        self.model_runner = ModelRunner(self.config, self.device)
        self._init_profiler()

    def load_model(self) -> None:
        if self.config.enable_sleep_mode and self.device.type == "cuda":
            # weights live in the sleepable pool under their own tag: level-1 sleep copies them to
            # pinned host memory and gives their device memory back, wake-up restores them in place
            from .mem_pool import B200MemAllocator
            with B200MemAllocator.get_instance().use_memory_pool(tag="weights"):
                self.model_runner.load_model()
        else:
            self.model_runner.load_model()

    def get_model(self):
        return self.model_runner.get_model()

    def determine_num_blocks(self) -> int:
        n = self.model_runner.determine_num_blocks()
        # every rank of the world must agree on the number of blocks
        world = pstate.get_world_group()
        if world.world_size > 1:
            n = min(world.all_gather_object(n))
        return n

    def get_kv_cache_spec(self):
        return self.model_runner.get_kv_cache_spec()

    def initialize_from_config(self, num_blocks: int) -> None:
        if self.config.kv_transfer is not None and self.config.kv_transfer.kv_connector:
            from ..kv_transfer.connector import create_connector
            self.model_runner.kv_connector = create_connector(self.config, role="worker",
                                                              device=self.device)
        if self.config.enable_sleep_mode and self.device.type == "cuda":
            from .mem_pool import B200MemAllocator
            with B200MemAllocator.get_instance().use_memory_pool(tag="kv_cache"):
                self.model_runner.initialize_kv_cache(num_blocks)
        else:
            self.model_runner.initialize_kv_cache(num_blocks)

    def compile_or_warm_up_model(self) -> None:
        if self.device.type == "cuda":
            # touch every kernel once outside of capture, then capture
            self.model_runner._dummy_run(min(256, self.config.scheduler.max_num_batched_tokens), prefill=True)
            self.model_runner._dummy_run(1, prefill=False)
            torch.cuda.synchronize(self.device)
            ops.check_status(self.device)
        self.model_runner.capture_model()
        # ranks may have drifted by seconds (loading, capture); meet on the host so that the
        # first device-side wait of the serving loop starts with every peer present
        world = pstate.get_world_group()
        if world.world_size > 1:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            world.barrier()

    # ------------------------------------------------------------- running
    def _profile_window_open(self, out: SchedulerOutput) -> None:
        """Token-threshold profiling: a step that schedules exactly ``PROFILER_TOKEN_THRESHOLD``
        tokens starts the profiler for ``PROFILER_STOP_STEP`` steps."""
        if self._profile_threshold and self.profiler is not None:
            if self._profile_steps_left == 0 and out.total_num_scheduled_tokens == self._profile_threshold:
                self.profiler.start()
                self._profile_steps_left = self._profile_stop_step

    def _profile_window_close(self) -> None:
        if self._profile_steps_left > 0:
            self._profile_steps_left -= 1
            if self._profile_steps_left == 0:
                self.profiler.stop()

    @token_recover_wrapper
    def execute_model(self, out: SchedulerOutput) -> List[int]:
        self._profile_window_open(out)
        tokens = self.model_runner.execute_model(out)
        self._profile_window_close()
        return tokens

    def launch_decode(self, out: SchedulerOutput, prev: Optional[dict] = None) -> dict:
        """Decode step launched ahead of its results (asynchronous scheduling): same profiling
        window as ``execute_model``; the step counts when it is launched."""
        self._profile_window_open(out)
        handle = self.model_runner.launch_decode(out, prev)
        self._profile_window_close()
        return handle

    # ------------------------------------------------ token recovery hooks
    def enable_token_recovery(self, env=None) -> None:
        """Start this worker's command endpoint and register it with the coordinator
        (``USE_HA=1``, ``HA_SERVER_IP``, ``HA_PORT``)."""
        from ..ha.common import HAEnv
        from ..ha.monitor import HAWorkerAgent
        env = env or HAEnv.from_environ()
        if env.use_ha and self.ha_agent is None:
            self.ha_agent = HAWorkerAgent(env, self.rank, self.local_rank).start()

    def stop_device(self) -> None:
        """Leave whatever the device is doing: wait (bounded by the communicators' own
        timeouts) for queued work and abort the communicators so peers' collectives end."""
        if self.device.type == "cuda":
            try:
                torch.cuda.synchronize(self.device)
            except Exception as e:
                logger.warning("synchronize during stop_device: %s", e)
        pstate.abort_communicators()

    def restart_device(self) -> None:
        """Drop state that may be inconsistent after a failed step (captured graphs stay
        valid: they hold no communicator handles of torch.distributed)."""
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    def reinit_process_group(self) -> None:
        pstate.reinit_communicators()

    def execute_dummy_batch(self) -> None:
        self.model_runner.execute_dummy_batch()

    def profile(self, is_start: bool = True) -> None:
        if self.profiler is None:
            raise RuntimeError("profiler not enabled: set VLLM_TORCH_PROFILER_DIR")
        self.profiler.start() if is_start else self.profiler.stop()

    def _init_profiler(self) -> None:
        trace_dir = os.environ.get("VLLM_TORCH_PROFILER_DIR")
        if not trace_dir:
            return
        acts = [torch.profiler.ProfilerActivity.CPU]
        if self.device.type == "cuda":
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self.profiler = torch.profiler.profile(
            activities=acts,
            record_shapes=bool(int(os.environ.get("VLLM_TORCH_PROFILER_RECORD_SHAPES", "0"))),
            profile_memory=bool(int(os.environ.get("VLLM_TORCH_PROFILER_WITH_PROFILE_MEMORY", "0"))),
            with_stack=bool(int(os.environ.get("VLLM_TORCH_PROFILER_WITH_STACK", "0"))),
            on_trace_ready=torch.profiler.tensorboard_trace_handler(trace_dir, use_gzip=True))

    def sleep(self, level: int = 1) -> int:
        """Level 1: weights are kept in pinned host memory, the KV cache is discarded; level 2: both
        are discarded.  Returns the device bytes released.
        (reference: sleep-mode pool, omni_npu/worker/npu_mem_pool.py:109-284, wired in
        omni_npu/worker/npu_worker.py:164-179)"""
        from .mem_pool import B200MemAllocator
        return B200MemAllocator.get_instance().sleep(offload_tags=("weights",) if level == 1 else ())

    def wake_up(self, tags=None) -> int:
        from .mem_pool import B200MemAllocator
        return B200MemAllocator.get_instance().wake_up(tags)

    def shutdown(self) -> None:
        if self.model_runner is not None and self.model_runner.kv_connector is not None:
            self.model_runner.kv_connector.close()
