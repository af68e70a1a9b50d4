"""Engine and offline ``LLM`` front end.

``LLMEngine`` ties scheduler and worker together: ``add_request`` / ``step``.
``LLM.generate`` is the offline batch API.  With more than one rank the engine
runs SPMD: every rank executes the same deterministic scheduler over the same
requests, so no per-step control broadcast is needed (ranks only meet inside
the model's collectives); rank 0's outputs are the result.
"""
from __future__ import annotations

import itertools
import time
from typing import Dict, Iterable, List, Optional, Sequence, Union

import torch

from .. import ops
from ..config import EngineConfig, ModelConfig, PRESETS
from ..logger import logger
from ..worker.worker import Worker
from .request import Request, RequestOutput, SamplingParams
from .scheduler import Scheduler, SchedulerOutput


class LLMEngine:
    def __init__(self, config: EngineConfig, local_rank: Optional[int] = None,
                 rank: Optional[int] = None) -> None:
        import os
        self.config = config
        local_rank = int(os.environ.get("LOCAL_RANK", "0")) if local_rank is None else local_rank
        rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.rank = rank
        self.worker = Worker(config, local_rank=local_rank, rank=rank)
        self.worker.init_device()
        self.worker.load_model()
        num_blocks = self.worker.determine_num_blocks()
        self.worker.initialize_from_config(num_blocks)
        self.worker.compile_or_warm_up_model()
        connector = None
        if config.kv_transfer is not None and config.kv_transfer.kv_connector:
            from ..kv_transfer.connector import create_connector
            connector = create_connector(config, role="scheduler")
        reserved = getattr(self.worker.get_model(), "num_reserved_kv_blocks", 0)
        dcp = config.parallel.decode_context_parallel_size
        if dcp > 1:
            mc = config.model
            if not mc.use_mla or mc.use_sparse:
                raise ValueError("decode_context_parallel_size > 1 is supported for latent attention (MLA) "
                                 "models without the sparse indexer")
            if dcp != config.parallel.tensor_parallel_size:
                raise ValueError("decode context parallelism shards the cache over the tensor-parallel group: "
                                 "decode_context_parallel_size must equal tensor_parallel_size")
            if connector is not None or (config.speculative.method and config.speculative.num_speculative_tokens):
                raise ValueError("decode context parallelism is not combined with KV connectors or "
                                 "speculative decoding")
        if config.speculative.method in ("mtp", "deepseek_mtp") and config.speculative.num_speculative_tokens > 1:
            config.scheduler.num_lookahead_tokens = config.speculative.num_speculative_tokens - 1
        self.scheduler = Scheduler(config.scheduler, config.cache, num_blocks, reserved, connector,
                                   context_parallel_size=dcp)
        self._ids = itertools.count()
        self.stats = {"steps": 0, "prefill_steps": 0, "decode_steps": 0, "spec_decode_steps": 0,
                      "h2d_bytes": 0, "d2h_bytes": 0, "output_tokens": 0}
        from ..spec_decode import make_proposer
        self.proposer = make_proposer(config.speculative, self.worker.model_runner)
        # launch decode step n + 1 before reading the tokens of step n (host scheduling and staging then
        # overlap the GPU); on by default, OMNI_B200_ASYNC_SCHED=0 or additional_config["async_scheduling"]
        # = False restores the strictly alternating loop
        import os as _os
        self.async_scheduling = bool(config.additional_config.get(
            "async_scheduling", _os.environ.get("OMNI_B200_ASYNC_SCHED", "1") != "0"))
        self._inflight = None
        # data-parallel replicas (attention DP + experts sharded over DP x TP) step in lock-step
        from ..parallel import state as pstate
        dp = pstate.get_dp_group()
        self.dp_group = dp if dp.world_size > 1 else None
        self.dp_all_idle = False

    @property
    def device(self) -> torch.device:
        return self.worker.device

    def add_request(self, prompt_token_ids: Sequence[int], sampling_params: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None, kv_transfer_params=None,
                    arrival_time: Optional[float] = None) -> str:
        rid = request_id or f"req-{next(self._ids)}"
        self.validate_sampling_params(sampling_params)
        req = Request(rid, prompt_token_ids, sampling_params, self.config.model.eos_token_id,
                      arrival_time, kv_transfer_params)
        self.scheduler.add_request(req)
        return rid

    def validate_sampling_params(self, sp: Optional[SamplingParams]) -> None:
        """Refuse (ValueError) what the sampler cannot honour rather than ignore it."""
        if sp is None:
            return
        runner = self.worker.model_runner
        speculative = self.proposer is not None or runner.mtp is not None
        if speculative and (sp.has_penalties or sp.thinking_token_budget is not None or sp.logprobs):
            raise ValueError("penalties, thinking_token_budget and logprobs are not supported together with "
                             "speculative decoding")
        if sp.structured is not None:
            if speculative:
                raise ValueError("structured outputs are not supported together with speculative decoding")
            if runner.structured is None:
                raise ValueError("structured outputs need a tokenizer (LLM.enable_structured_outputs, or a server "
                                 "started with a tokenizer directory)")
            if runner.pcp_group is not None or self.dp_group is not None:
                raise ValueError("structured outputs are not supported with prefill-context or data parallelism")
            runner.structured.compile(sp.structured)         # a grammar that does not compile is refused here
        if sp.logprobs and (int(sp.logprobs) < 0 or int(sp.logprobs) > 20):
            raise ValueError("logprobs must be between 0 and 20")
        if sp.logprobs and (runner.pcp_group is not None or self.dp_group is not None):
            raise ValueError("logprobs are not supported with prefill-context or data parallelism")
        if sp.prompt_logprobs is not None:
            if not 0 <= int(sp.prompt_logprobs) <= 20:
                raise ValueError("prompt_logprobs must be between 0 and 20")
            if speculative or runner.pcp_group is not None or runner.pp_group is not None or self.dp_group is not None \
                    or runner.kv_connector is not None:
                raise ValueError("prompt_logprobs are not supported with speculative decoding, KV connectors, "
                                 "pipeline, prefill-context or data parallelism")
        if sp.thinking_token_budget is not None and not runner.thinking_processor.enabled:
            raise ValueError("thinking_token_budget needs a reasoning config with think start / end "
                             "token ids (additional_config['reasoning_config'], --reasoning-config)")

    def abort_request(self, request_id: str) -> None:
        self.scheduler.abort_request(request_id)

    def fail_all_requests(self) -> List[RequestOutput]:
        """Abort everything in flight (after a step raised): the requests end with
        finish_reason "abort" and their blocks return to the pool."""
        self._inflight = None
        outs = []
        for req in list(self.scheduler.running) + list(self.scheduler.waiting):
            self.scheduler.abort_request(req.request_id)
            self.worker.model_runner.input_batch.remove_request(req.request_id)
            outs.append(RequestOutput.from_request(req))
        return outs

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished() or self._inflight is not None

    # ---------------------------------------------------- asynchronous decode scheduling
    def _async_ok(self) -> bool:
        """Decode steps may be launched before the previous step's tokens are read when nothing on the
        host needs the token values between steps: no draft proposer, no KV connector, no draft head."""
        runner = self.worker.model_runner
        return (self.async_scheduling and self.proposer is None and self.scheduler.kv_connector is None
                and runner.mtp is None and getattr(self.worker, "ha_agent", None) is None
                and runner.pp_group is None and self.dp_group is None
                and not (runner.pcp_group is not None and runner.pcp_decode_split)
                and not any(runner.needs_host_logits(r) for r in self.scheduler.running))

    def _settle(self) -> List[RequestOutput]:
        """Read back the step in flight and fill its tokens in."""
        if self._inflight is None:
            return []
        out, handle = self._inflight
        self._inflight = None
        runner = self.worker.model_runner
        finished = self.scheduler.resolve_pending(out, runner.collect_decode(handle))
        self.stats["d2h_bytes"] += handle["n"] * 4
        self.stats["output_tokens"] += handle["n"]
        for r in finished:
            runner.input_batch.remove_request(r.request_id)
        return [RequestOutput.from_request(r) for r in finished]

    def _step_async(self) -> List[RequestOutput]:
        early: List[RequestOutput] = []
        if (self._inflight is not None and self.scheduler.cfg.enable_mixed_batches
                and self.scheduler.prompt_work_waiting()):
            # the next step may carry decoding requests beside prompt chunks: their newest tokens
            # (and whether they have just finished) must be known before it is put together
            early = self._settle()
        out = self.scheduler.schedule()
        if out.kind == "decode":
            runner = self.worker.model_runner
            handle = self.worker.launch_decode(out, self._inflight[1] if self._inflight is not None else None)
            self.scheduler.advance_pending(out)
            done = self._settle()                       # the previous step, while this one runs
            self._inflight = (out, handle)
            st = self.stats
            st["steps"] += 1
            st["decode_steps"] += 1
            st["h2d_bytes"] += runner.input_batch.h2d_bytes_last
            interval = self.config.parallel.eplb_step_interval
            if interval > 0 and st["steps"] % interval == 0:
                self.rebalance_experts()                 # weight moves queue behind the step in flight
            return early + done
        # anything but a plain decode step needs the token values on the host first
        done = self._settle()
        return early + done + self._run_scheduled(out)

    def _step_data_parallel(self) -> List[RequestOutput]:
        """One global step of a data-parallel deployment.  Every replica schedules its own
        requests, but the expert-parallel exchanges inside the MoE layers span all replicas, so
        each replica must run exactly one forward pass per global step: replicas agree (one
        small host-side all-reduce) on whether anyone has work; a replica without work runs a
        one-token dummy batch.  ``dp_all_idle`` tells the caller's loop when every replica is
        done.  (reference: dummy batches on idle data-parallel ranks,
        omni_npu/worker/npu_worker.py:213-214, and one engine process per DP rank in
        examples/serve-pd-disaggregate.sh:195-238)"""
        import torch.distributed as dist
        busy = self.scheduler.has_unfinished()
        flag = torch.tensor([int(busy)], dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.dp_group.cpu_group)
        self.dp_all_idle = int(flag.item()) == 0
        if self.dp_all_idle:
            return []
        out = self.scheduler.schedule() if busy else None
        if out is None or out.kind == "idle":
            if out is not None:
                self.worker.model_runner.execute_model(out)      # retire rows, start KV loads
            self.worker.execute_dummy_batch()
            st = self.stats
            st["steps"] += 1
            st["dummy_steps"] = st.get("dummy_steps", 0) + 1
            interval = self.config.parallel.eplb_step_interval
            if interval > 0 and st["steps"] % interval == 0:
                self.rebalance_experts()
            return []
        return self._run_scheduled(out)

    def step(self) -> List[RequestOutput]:
        if self.dp_group is not None:
            return self._step_data_parallel()
        if self._async_ok():
            return self._step_async()
        if self._inflight is not None:                  # the switch was turned off mid-flight
            return self._settle()
        return self._run_scheduled(self.scheduler.schedule())

    def _run_scheduled(self, out: SchedulerOutput) -> List[RequestOutput]:
        if out.kind == "idle":
            # nothing to compute: still let the runner retire rows and start KV loads
            self.worker.model_runner.execute_model(out)
            if self.scheduler.has_unfinished():
                time.sleep(0.001)        # waiting for remote KV
            return []
        tokens = self.worker.execute_model(out)
        if isinstance(tokens, dict):
            return self._after_recovered_step(out, tokens)
        drafts = None
        if self.proposer is not None and any(s.samples for s in out.seqs):
            drafts = self._propose(out, tokens)
        before = sum(len(s.request.output_token_ids) for s in out.seqs)
        finished = self.scheduler.update_from_output(out, tokens, drafts=drafts)
        for idx, entry in (getattr(self.worker.model_runner, "last_logprobs", None) or {}).items():
            out.seqs[idx].request.logprobs.append(entry[:2])        # (log-probability, alternatives); the rank stays behind
        for idx, (first, entries) in (getattr(self.worker.model_runner, "last_prompt_logprobs", None) or {}).items():
            out.seqs[idx].request.prompt_logprobs[first: first + len(entries)] = entries
        st = self.stats
        st["steps"] += 1
        st[out.kind + "_steps"] += 1
        st["h2d_bytes"] += self.worker.model_runner.input_batch.h2d_bytes_last
        st["d2h_bytes"] += self.worker.model_runner.d2h_bytes_last
        st["output_tokens"] += sum(len(s.request.output_token_ids) for s in out.seqs) - before
        for r in finished:
            self.worker.model_runner.input_batch.remove_request(r.request_id)
            if self.worker.model_runner.structured is not None:
                self.worker.model_runner.structured.remove_request(r.request_id)
        interval = self.config.parallel.eplb_step_interval
        if interval > 0 and st["steps"] % interval == 0:
            self.rebalance_experts()
        return [RequestOutput.from_request(r) for r in finished]

    def rebalance_experts(self) -> int:
        """Re-plan the expert placement of every MoE layer from the load measured since the last
        call and move the weights (between steps; every rank reaches this at the same step count,
        so the collectives inside line up).  Returns the number of physical slots that changed."""
        moved = 0
        for m in self.worker.get_model().modules():
            if getattr(m, "eplb", None) is not None and hasattr(m, "rebalance"):
                moved += m.rebalance()
        self.stats["eplb_moves"] = self.stats.get("eplb_moves", 0) + moved
        return moved

    def _after_recovered_step(self, out, verdict: dict) -> List[RequestOutput]:
        """The step failed and the workers recovered (token recovery).  ``recompute``: nothing
        of the step is kept, every scheduled request is recomputed from scratch (its KV may be
        half-written); ``abort``: requests that own a damaged KV block are aborted, the rest
        recomputed."""
        self.stats["recovered_steps"] = self.stats.get("recovered_steps", 0) + 1
        bad = set(verdict.get("bad_blocks") or [])
        finished: List[RequestOutput] = []
        for seq in list(out.seqs):
            req = seq.request
            if req.is_finished:
                continue
            if verdict.get("opt") == "abort" and bad & set(req.block_ids):
                self.scheduler.abort_request(req.request_id)
                self.worker.model_runner.input_batch.remove_request(req.request_id)
                finished.append(RequestOutput.from_request(req))
            else:
                self.scheduler.preempt_for_recompute(req)
                self.worker.model_runner.input_batch.remove_request(req.request_id)
        return finished

    def _propose(self, out, tokens) -> List[List[int]]:
        """Draft tokens for the next step of every sequence that just produced a token.
        Host-side proposers see the token history including this step's tokens."""
        prop = self.proposer
        if getattr(prop, "needs_hidden_states", False):
            return prop.propose(out, tokens)
        drafts: List[List[int]] = []
        for seq, tok in zip(out.seqs, tokens):
            if not seq.samples:
                drafts.append([])
                continue
            new = list(tok) if isinstance(tok, (list, tuple)) else [tok]
            drafts.append(prop.propose_one(seq.request.all_token_ids + [int(t) for t in new]))
        return drafts

    def shutdown(self) -> None:
        self.worker.shutdown()


class LLM:
    """Offline inference front end.

    >>> llm = LLM(model="llama-3-8b")                # preset name, HF directory or ModelConfig
    >>> outs = llm.generate([[1, 2, 3]], SamplingParams(max_tokens=8))
    """

    def __init__(self, model: Union[str, ModelConfig, EngineConfig] = "llama-3-8b", **kw) -> None:
        if isinstance(model, EngineConfig):
            config = model
        else:
            import os
            path = None
            if isinstance(model, ModelConfig):
                mc = model
            elif model in PRESETS:
                mc = PRESETS[model]()
            elif os.path.isdir(model):
                mc, path = ModelConfig.from_pretrained(model, kw.pop("dtype", None)), model
            else:
                raise ValueError(f"unknown model {model!r}: give a preset {sorted(PRESETS)}, a directory or a config")
            config = build_engine_config(mc, model_path=path, **kw)
        self.config = config
        self.engine = LLMEngine(config)
        self.tokenizer = None             # loaded on first use from the model directory (or set by the caller)

    def get_tokenizer(self):
        """The model directory's tokenizer (None when there is none): text prompts are encoded with
        it, outputs get their ``text``, structured outputs are compiled against it."""
        if self.tokenizer is None and self.config.model_path:
            try:
                from transformers import AutoTokenizer
                self.tokenizer = AutoTokenizer.from_pretrained(self.config.model_path)
            except Exception:                          # no tokenizer files beside the weights
                return None
            try:
                self.enable_structured_outputs(self.tokenizer)
            except Exception:                          # the grammar package is optional
                pass
        return self.tokenizer

    def enable_structured_outputs(self, tokenizer) -> None:
        """Give the engine the tokenizer that structured outputs (``SamplingParams.structured``) are
        compiled against; call it on every rank."""
        self.tokenizer = self.tokenizer or tokenizer
        self.engine.worker.model_runner.enable_structured_outputs(tokenizer)

    def start_profile(self) -> None:
        """Start the worker's torch profiler (needs ``VLLM_TORCH_PROFILER_DIR`` at start-up)."""
        self.engine.worker.profile(True)

    def stop_profile(self) -> None:
        self.engine.worker.profile(False)

    def sleep(self, level: int = 1) -> int:
        """Give the device memory of the sleep-mode pool back (needs ``enable_sleep_mode=True``);
        only between requests.  Returns the bytes released."""
        if self.engine.has_unfinished_requests():
            raise RuntimeError("sleep() while requests are running")
        return self.engine.worker.sleep(level)

    def wake_up(self, tags=None) -> int:
        return self.engine.worker.wake_up(tags)

    def generate(self, prompts: Sequence[Union[str, Sequence[int]]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 ) -> List[RequestOutput]:
        """Run the prompts to completion.  A prompt is a list of token ids, or text when the model
        directory has a tokenizer (the outputs then carry ``text`` as well)."""
        tok = self.tokenizer
        if any(isinstance(p, str) for p in prompts):
            tok = self.get_tokenizer()
            if tok is None:
                raise ValueError("text prompts need a tokenizer in the model directory; pass token ids instead")
            prompts = [tok.encode(p) if isinstance(p, str) else p for p in prompts]
        sps = sampling_params if isinstance(sampling_params, (list, tuple)) else [sampling_params] * len(prompts)
        order: Dict[str, int] = {}
        now = time.monotonic()
        for i, (p, sp) in enumerate(zip(prompts, sps)):
            order[self.engine.add_request(p, sp, arrival_time=now)] = i
        results: List[Optional[RequestOutput]] = [None] * len(prompts)
        if self.engine.dp_group is not None:
            # replicas finish at different times; keep stepping (dummy batches) until all are done
            while True:
                for o in self.engine.step():
                    results[order[o.request_id]] = o
                if self.engine.dp_all_idle:
                    break
        while self.engine.has_unfinished_requests():
            for o in self.engine.step():
                results[order[o.request_id]] = o
        if self.engine.device.type == "cuda":
            ops.check_status(self.engine.device)
        if tok is not None:
            for o in results:
                if o is not None:
                    o.text = tok.decode(o.output_token_ids)
        return results  # type: ignore[return-value]


def build_engine_config(model: ModelConfig, model_path: Optional[str] = None, **kw) -> EngineConfig:
    """Keyword-style construction mirroring the usual serving flags
    (tensor_parallel_size, max_num_seqs, block_size, ...)."""
    from ..config import (CacheConfig, CompilationConfig, KVTransferConfig, ParallelConfig,
                          SchedulerConfig, SpeculativeConfig)
    cache = CacheConfig(block_size=kw.pop("block_size", 16),
                        gpu_memory_utilization=kw.pop("gpu_memory_utilization", 0.9),
                        num_gpu_blocks=kw.pop("num_gpu_blocks", None),
                        enable_prefix_caching=kw.pop("enable_prefix_caching", False))
    par = ParallelConfig(tensor_parallel_size=kw.pop("tensor_parallel_size", 1),
                         pipeline_parallel_size=kw.pop("pipeline_parallel_size", 1),
                         data_parallel_size=kw.pop("data_parallel_size", 1),
                         enable_expert_parallel=kw.pop("enable_expert_parallel", False),
                         decode_context_parallel_size=kw.pop("decode_context_parallel_size", 1),
                         prefill_context_parallel_size=kw.pop("prefill_context_parallel_size", 1),
                         sequence_parallel_residual=kw.pop("sequence_parallel_residual", False),
                         num_redundant_experts=kw.pop("num_redundant_experts", 0),
                         eplb_step_interval=kw.pop("eplb_step_interval", 0),
                         layer_parallel_config=kw.pop("layer_parallel_config", {}) or {})
    sched = SchedulerConfig(max_num_seqs=kw.pop("max_num_seqs", 128),
                            max_num_batched_tokens=kw.pop("max_num_batched_tokens", 8192),
                            max_model_len=kw.pop("max_model_len", min(8192, model.max_position_embeddings)),
                            enable_chunked_prefill=kw.pop("enable_chunked_prefill", True),
                            enable_mixed_batches=kw.pop("enable_mixed_batches", False),
                            policy=kw.pop("scheduling_policy", "fcfs"))
    comp = kw.pop("compilation_config", None)
    if isinstance(comp, dict):
        comp = CompilationConfig(cudagraph_mode=comp.get("cudagraph_mode", "FULL_DECODE_ONLY"),
                                 cudagraph_capture_sizes=comp.get("cudagraph_capture_sizes"))
    kvt = kw.pop("kv_transfer_config", None)
    if isinstance(kvt, dict):
        kvt = KVTransferConfig(**kvt)
    spec = kw.pop("speculative_config", None)
    if isinstance(spec, dict):
        spec = SpeculativeConfig(method=spec.get("method"),
                                 num_speculative_tokens=spec.get("num_speculative_tokens", 0),
                                 prompt_lookup_max=spec.get("prompt_lookup_max", 4),
                                 prompt_lookup_min=spec.get("prompt_lookup_min", 2))
    cfg = EngineConfig(model=model, cache=cache, parallel=par, scheduler=sched,
                       compilation=comp or CompilationConfig(), kv_transfer=kvt,
                       speculative=spec or SpeculativeConfig(), model_path=model_path,
                       load_format=kw.pop("load_format", "auto"), seed=kw.pop("seed", 0),
                       device=kw.pop("device", "auto"), enforce_eager=kw.pop("enforce_eager", False),
                       enable_sleep_mode=kw.pop("enable_sleep_mode", False),
                       additional_config=kw.pop("additional_config", {}) or {})
    if kw:
        raise TypeError(f"unknown engine arguments: {sorted(kw)}")
    return cfg
