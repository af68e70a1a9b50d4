"""vLLM worker that runs this package's own model runner.

``B200Worker`` derives from vLLM's ``WorkerBase`` only (not from vLLM's GPU worker and not
from ``GPUModelRunner``): vLLM's engine core keeps its scheduler, KV block manager and
executor, and every per-device step goes through this package's ``Worker`` /
``ModelRunner`` (input batch with one pinned staging copy per step, full-step CUDA-graph
decode, tcgen05 GEMMs, fused collectives, own sampler).  The counterpart in the reference is
``NPUWorker`` + ``NPUModelRunner`` (omni_npu/worker/npu_worker.py:38-291,
omni_npu/worker/npu_model_runner.py:68-623); the reference's runner subclasses
``GPUModelRunner``, this one does not.

What is translated per step:

* vLLM ``SchedulerOutput`` -> ``engine.scheduler.SchedulerOutput``.  The worker keeps one
  ``engine.request.Request`` per live request (tokens, block ids, sampling parameters) and
  updates it from ``scheduled_new_reqs`` / ``scheduled_cached_reqs``.  A step whose sequences
  all feed exactly one token that yields a sample is a *decode* step (CUDA graph); anything
  else (prompt chunks, or prompt chunks mixed with decoding sequences, as vLLM's chunked
  prefill produces) runs as a variable-length *prefill* step.
* the runner's sampled tokens -> vLLM ``ModelRunnerOutput``.

KV cache: ``get_kv_cache_spec`` describes one attention spec per layer so that vLLM's KV
cache manager can size the cache; ``initialize_from_config`` takes the resulting block count
and lets the runner allocate its own paged tensors.  Block 0 is vLLM's null block and is the
only block the runner's dummy runs touch.

vLLM's asynchronous scheduling is supported for plain decode steps: the step is launched without
waiting for the previous step's tokens (they are fed forward on the device, the host books
placeholders) and ``sample_tokens`` returns an ``AsyncModelRunnerOutput`` that the executor
resolves later; any other kind of step first waits for the tokens in flight.

Speculative decoding driven by vLLM's scheduler: the n-gram method and the model's own MTP head.
The worker makes the drafts (a host look-up after every step, or the runner's MTP head running k
times as a chain inside the step) and hands them to vLLM (``take_draft_token_ids``), vLLM schedules
them, the worker verifies 1 + k rows per request in one pass and returns the accepted tokens plus
the one that follows them (the reference patches vLLM's ``EagleProposer`` for graph-mode drafting:
omni_npu/vllm_patches/patches/common/patch_eagle.py).

Log-probabilities of sampled tokens (``SamplingParams.logprobs``) are computed by the runner from
its own logits and handed back as vLLM's ``LogprobsLists``; such steps run as one eager launch.

Structured outputs: vLLM hands the grammar's bitmask to ``sample_tokens``; a step with such requests
is deferred to that call and runs there as one eager launch with the bitmask applied to the logits
rows of the structured requests (``grammar_mask_fn``).

Not supported under vLLM yet (refused with a clear error, never silently wrong): separate draft
models (Eagle heads, draft checkpoints), prompt log-probabilities, LoRA, pooling, pipeline and
context parallelism; structured outputs or log-probabilities together with speculative decoding.
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional

import torch

from .. import compat
from ..logger import logger

if compat.vllm_available():
    from vllm.v1.worker.worker_base import WorkerBase as _WorkerBase
else:                                                     # importable without vLLM (docs, tests)
    class _WorkerBase:                                    # type: ignore[no-redef]
        def __init__(self, vllm_config, local_rank, rank, distributed_init_method, is_driver_worker=False):
            self.vllm_config, self.local_rank, self.rank = vllm_config, local_rank, rank
            self.distributed_init_method, self.is_driver_worker = distributed_init_method, is_driver_worker


# vLLM's names for drafting with the target model's own multi-token-prediction head
MTP_METHODS = ("mtp", "deepseek_mtp")


def engine_config_from_vllm(vllm_config, device_type: str):
    """This package's ``EngineConfig`` for a vLLM ``VllmConfig``."""
    from ..config import ModelConfig
    from ..engine.llm import build_engine_config
    mc_v = vllm_config.model_config
    hf = mc_v.hf_config
    d = hf.to_dict() if hasattr(hf, "to_dict") else dict(hf)
    mc = ModelConfig.from_hf_dict(d, dtype=mc_v.dtype)
    pc, sc, cc = vllm_config.parallel_config, vllm_config.scheduler_config, vllm_config.cache_config
    if pc.pipeline_parallel_size > 1:
        raise ValueError("pipeline parallelism under vLLM is not supported by the B200 worker; "
                         "use the standalone engine (omni_npu_b200.serving.api_server)")
    if int(getattr(pc, "prefill_context_parallel_size", 1) or 1) > 1 or \
            int(getattr(pc, "decode_context_parallel_size", 1) or 1) > 1:
        # vLLM's block manager shards the cache of a context-parallel deployment by tokens; this
        # package's prefill context parallelism keeps the whole cache on every rank and its decode
        # context parallelism has its own block arithmetic (engine/scheduler.py)
        raise ValueError("context parallelism under vLLM is not supported by the B200 worker; "
                         "use the standalone engine (omni_npu_b200.serving.api_server)")
    comp = vllm_config.compilation_config
    sizes = list(getattr(comp, "cudagraph_capture_sizes", None) or [])
    sizes = [s for s in sizes if s <= sc.max_num_seqs] or None
    mode = str(getattr(getattr(comp, "cudagraph_mode", None), "name", "FULL_DECODE_ONLY"))
    eager = bool(mc_v.enforce_eager) or mode == "NONE" or device_type != "cuda"
    load_format = str(getattr(vllm_config.load_config, "load_format", "auto"))
    path = mc_v.model if os.path.isdir(str(mc_v.model)) else None
    ac = dict(getattr(vllm_config, "additional_config", None) or {})
    spec_kw = {}
    vsc = getattr(vllm_config, "speculative_config", None)
    if vsc is not None and str(getattr(vsc, "method", "")) in MTP_METHODS:
        # the runner builds the model's MTP head and drafts with it inside its own steps
        spec_kw["speculative_config"] = {"method": "deepseek_mtp",
                                         "num_speculative_tokens": int(vsc.num_speculative_tokens)}
    cfg = build_engine_config(
        mc, model_path=path, tensor_parallel_size=pc.tensor_parallel_size,
        data_parallel_size=1, enable_expert_parallel=bool(pc.enable_expert_parallel),
        max_num_seqs=sc.max_num_seqs, max_num_batched_tokens=sc.max_num_batched_tokens,
        max_model_len=mc_v.max_model_len, block_size=cc.block_size,
        gpu_memory_utilization=cc.gpu_memory_utilization, enforce_eager=eager,
        compilation_config={"cudagraph_mode": "NONE" if eager else "FULL_DECODE_ONLY",
                            "cudagraph_capture_sizes": sizes},
        load_format="dummy" if load_format == "dummy" or path is None else "auto",
        seed=int(mc_v.seed or 0), device=device_type,
        enable_sleep_mode=bool(getattr(mc_v, "enable_sleep_mode", False)), additional_config=ac, **spec_kw)
    return cfg


def sampling_params_from_vllm(sp):
    """vLLM ``SamplingParams`` -> this package's.  Stop conditions stay with vLLM's scheduler,
    which sees every sampled token; only what shapes the distribution is carried over."""
    from ..engine.request import SamplingParams
    if sp is None:
        return SamplingParams(max_tokens=1 << 30, ignore_eos=True)
    if getattr(sp, "prompt_logprobs", None):
        raise ValueError("prompt_logprobs are not supported by the B200 worker")
    # parameters that vLLM's own sampler would honour through logits processors this worker does not run
    if getattr(sp, "logits_processors", None):
        raise ValueError("sampling parameter logits_processors is not supported by the B200 worker")
    # vLLM tokenizes the banned words when it takes the request in; without that list they cannot be honoured
    bad = getattr(sp, "bad_words_token_ids", None)
    if getattr(sp, "bad_words", None) and not bad:
        raise ValueError("sampling parameter bad_words reached the B200 worker without its token ids")
    want_lp = getattr(sp, "logprobs", None)
    top_k = int(getattr(sp, "top_k", 0) or 0)
    return SamplingParams(
        max_tokens=1 << 30, temperature=float(sp.temperature or 0.0), top_k=top_k if top_k > 0 else 0,
        top_p=float(sp.top_p if sp.top_p is not None else 1.0), seed=sp.seed, ignore_eos=True,
        presence_penalty=float(sp.presence_penalty or 0.0), frequency_penalty=float(sp.frequency_penalty or 0.0),
        repetition_penalty=float(sp.repetition_penalty or 1.0),
        thinking_token_budget=(getattr(sp, "extra_args", None) or {}).get("thinking_token_budget"),
        # vLLM's 0 = the sampled token's log-probability only; the runner keeps at least one alternative
        logprobs=None if want_lp is None else max(1, min(20, int(want_lp))),
        # vLLM's own sampler (and with it its logits processors) is not on this worker's path: the
        # bias and the minimum length are applied by the runner's logits hook instead
        logit_bias={int(k): float(v) for k, v in (getattr(sp, "logit_bias", None) or {}).items()} or None,
        min_tokens=int(getattr(sp, "min_tokens", 0) or 0), min_p=float(getattr(sp, "min_p", 0.0) or 0.0),
        allowed_token_ids=list(getattr(sp, "allowed_token_ids", None) or ()) or None,
        bad_words_token_ids=[list(w) for w in bad] if bad else None,
        stop_token_ids=tuple(int(t) for t in (getattr(sp, "all_stop_token_ids", None) or ())))


def grammar_mask_fn(step_req_ids, structured_req_ids, bitmask):
    """Logits adjustment for one step: row i of the logits belongs to ``step_req_ids[i]``; row j of
    ``bitmask`` (int32 words, bit b of word w = token 32 w + b, set = allowed) to
    ``structured_req_ids[j]``.  Tokens whose bit is clear get -inf; other rows are untouched."""
    import numpy as np
    row_of = {rid: i for i, rid in enumerate(step_req_ids)}
    pairs = [(row_of[rid], j) for j, rid in enumerate(structured_req_ids) if rid in row_of]
    words = np.ascontiguousarray(np.asarray(bitmask, dtype=np.int32))

    def fn(logits: torch.Tensor) -> torch.Tensor:
        if not pairs:
            return logits
        vocab = logits.shape[-1]
        rows = torch.tensor([p[0] for p in pairs], dtype=torch.long, device=logits.device)
        w = torch.from_numpy(words[[p[1] for p in pairs]]).to(logits.device)
        bits = (w.unsqueeze(-1) >> torch.arange(32, device=logits.device, dtype=torch.int32)) & 1
        allowed = bits.reshape(len(pairs), -1)[:, :vocab].bool()
        if allowed.shape[1] < vocab:          # a bitmask narrower than the (padded) vocabulary: the tail is not allowed
            allowed = torch.cat([allowed, allowed.new_zeros(len(pairs), vocab - allowed.shape[1])], dim=1)
        sub = logits.index_select(0, rows).masked_fill(~allowed, float("-inf"))
        return logits.index_copy(0, rows, sub)
    return fn


def logprobs_lists(seqs, sampled, last_logprobs):
    """vLLM's ``LogprobsLists`` for one step: a row per request of the step, [sampled token, top k]
    in the first k + 1 columns (rows of requests that did not ask, or got no token, are zeros)."""
    import numpy as np
    from vllm.v1.outputs import LogprobsLists
    if not last_logprobs:
        return None
    k = max(len(e[1]) for e in last_logprobs.values())
    n = len(seqs)
    ids = np.zeros((n, k + 1), dtype=np.int64)
    lps = np.full((n, k + 1), -np.inf, dtype=np.float32)
    ranks = np.zeros((n,), dtype=np.int64)
    for i, (lp, top, rank) in last_logprobs.items():
        if not sampled[i]:
            continue
        ids[i, 0], lps[i, 0], ranks[i] = sampled[i][0], lp, rank
        for j, (tid, v) in enumerate(top):
            ids[i, 1 + j], lps[i, 1 + j] = tid, v
    return LogprobsLists(ids, lps, ranks)


class StepTranslator:
    """Per-request state of a worker and the translation of one scheduler step."""

    def __init__(self) -> None:
        self.requests: Dict[str, Any] = {}
        self.allow_spec = False          # set by the worker when vLLM's speculative method is one it runs

    def translate(self, so):
        from ..engine.request import Request
        from ..engine.scheduler import ScheduledSeq, SchedulerOutput
        spec = getattr(so, "scheduled_spec_decode_tokens", None) or {}
        if spec and not self.allow_spec:
            raise NotImplementedError("speculative decoding driven by vLLM's scheduler is supported for the "
                                      "n-gram method only")
        out = SchedulerOutput()
        for rid in so.finished_req_ids:
            if self.requests.pop(rid, None) is not None:
                out.finished_req_ids.append(rid)
        for rid in (getattr(so, "preempted_req_ids", None) or ()):
            r = self.requests.get(rid)
            if r is not None:
                r.block_ids = []
                r.num_computed_tokens = 0
                out.preempted.append(rid)
        for new in so.scheduled_new_reqs:
            if new.pooling_params is not None:
                raise NotImplementedError("pooling requests are not supported by the B200 worker")
            if len(new.block_ids) != 1:
                raise NotImplementedError("more than one KV cache group is not supported by the B200 worker")
            toks = new.prompt_token_ids if new.prompt_token_ids is not None else new.prefill_token_ids
            if toks is None:
                raise NotImplementedError("prompt embeddings are not supported by the B200 worker")
            req = Request(new.req_id, toks, sampling_params_from_vllm(new.sampling_params))
            req.block_ids = list(new.block_ids[0])
            req.num_computed_tokens = int(new.num_computed_tokens)
            self.requests[new.req_id] = req
        cached = so.scheduled_cached_reqs
        for i, rid in enumerate(cached.req_ids):
            req = self.requests[rid]
            nb = cached.new_block_ids[i]
            if rid in cached.resumed_req_ids:
                req.block_ids = list(nb[0]) if nb is not None else []
            elif nb is not None:
                req.block_ids.extend(nb[0])
            req.num_computed_tokens = int(cached.num_computed_tokens[i])
            if cached.new_token_ids:                      # pipeline parallelism: tokens come from the scheduler
                known = len(req.output_token_ids)
                want = int(cached.num_output_tokens[i]) if cached.num_output_tokens else known
                extra = cached.new_token_ids[i][-(want - known):] if want > known else []
                req.output_token_ids.extend(int(t) for t in extra)
        seqs: List[ScheduledSeq] = []
        all_decode = True
        has_spec = False
        order = [n.req_id for n in so.scheduled_new_reqs] + list(cached.req_ids)
        for rid in order:
            n = int(so.num_scheduled_tokens.get(rid, 0))
            if n <= 0:
                continue
            req = self.requests[rid]
            start = req.num_computed_tokens
            drafts = [int(t) for t in spec.get(rid, ())]
            if drafts:
                # vLLM scheduled the newest token plus its drafts: n = 1 + drafts (fewer when the
                # token budget cut them short)
                drafts = drafts[: max(0, n - 1)]
                n = 1 + len(drafts)
                seqs.append(ScheduledSeq(req, start, n, True, drafts))
                has_spec = True
                continue
            samples = start + n >= req.num_tokens
            seqs.append(ScheduledSeq(req, start, n, samples))
            if not (n == 1 and samples and start > 0):
                all_decode = False
        out.seqs = seqs
        out.num_tokens = sum(s.num_new_tokens for s in seqs)
        out.kind = "idle" if not seqs else ("decode" if all_decode else "prefill")
        if has_spec:
            out.kind = "spec_decode" if all_decode else "prefill+spec"
        return out

    def commit_pending(self, out) -> List[int]:
        """Book a launched decode step whose tokens are not on the host yet: every sequence gets a
        placeholder (-1) as its newest token.  Returns the placeholder positions for ``resolve``."""
        pos = []
        for seq in out.seqs:
            req = seq.request
            req.num_computed_tokens = seq.start + seq.num_new_tokens
            req.output_token_ids.append(-1)
            pos.append(len(req.output_token_ids) - 1)
        return pos

    @staticmethod
    def resolve(out, pos: List[int], tokens: List[int]) -> List[List[int]]:
        """Fill the placeholders of a launched step with the tokens that arrived."""
        result: List[List[int]] = []
        for seq, p, tok in zip(out.seqs, pos, tokens):
            ids = seq.request.output_token_ids
            if p < len(ids):
                ids[p] = int(tok)
            result.append([int(tok)])
        return result

    def commit(self, out, tokens: List[int]) -> List[List[int]]:
        """Book the step's sampled tokens on the worker's request objects; returns vLLM's
        ``sampled_token_ids`` (an empty list for a prompt chunk that does not end its prompt)."""
        result: List[List[int]] = []
        for seq, tok in zip(out.seqs, tokens):
            req = seq.request
            if isinstance(tok, (list, tuple)):
                # a verification step: the accepted drafts and the token that follows them
                toks = [int(t) for t in tok]
                req.num_computed_tokens = seq.start + len(toks)
                req.output_token_ids.extend(toks)
                result.append(toks)
                continue
            req.num_computed_tokens = seq.start + seq.num_new_tokens
            if seq.samples:
                req.output_token_ids.append(int(tok))
                result.append([int(tok)])
            else:
                result.append([])
        return result


class PendingDecodeOutput:
    """Result of a decode step that was launched without waiting for its tokens (vLLM's
    asynchronous scheduling).  ``get_output`` blocks until the device-to-host copy of the sampled
    tokens has finished, fills the placeholders and builds vLLM's ``ModelRunnerOutput``; it may be
    called from the executor's output thread."""

    def __init__(self, worker: "B200Worker", out, handle: dict, pos: List[int]) -> None:
        self.worker, self.out, self.handle, self.pos = worker, out, handle, pos
        self._result = None

    def tokens_on_host(self) -> None:
        if self._result is None:
            import threading
            with self.worker._resolve_lock:
                if self._result is None:
                    tokens = self.worker.model_runner.collect_decode(self.handle)
                    self._result = StepTranslator.resolve(self.out, self.pos, tokens)

    def get_output(self):
        from vllm.v1.outputs import ModelRunnerOutput
        self.tokens_on_host()
        req_ids = [s.request.request_id for s in self.out.seqs]
        return ModelRunnerOutput(req_ids=req_ids, req_id_to_index={r: i for i, r in enumerate(req_ids)},
                                 sampled_token_ids=self._result, logprobs=None, prompt_logprobs_dict={},
                                 pooler_output=[])


if compat.vllm_available():
    from vllm.v1.outputs import AsyncModelRunnerOutput as _AsyncBase

    class PendingDecodeOutput(PendingDecodeOutput, _AsyncBase):  # type: ignore[no-redef]
        pass


class B200Worker(_WorkerBase):  # type: ignore[misc, valid-type]
    def __init__(self, vllm_config, local_rank: int, rank: int, distributed_init_method: str,
                 is_driver_worker: bool = False, **kwargs: Any) -> None:
        super().__init__(vllm_config=vllm_config, local_rank=local_rank, rank=rank,
                         distributed_init_method=distributed_init_method, is_driver_worker=is_driver_worker)
        self.inner = None                      # this package's Worker
        self.engine_config = None
        self.translator = StepTranslator()
        self.ha_agent = None
        self._kv_bytes_per_block = 0
        self.steps = {"decode": 0, "prefill": 0}
        import threading
        self._resolve_lock = threading.Lock()
        self._inflight: Optional[PendingDecodeOutput] = None     # decode step launched ahead of its tokens
        self._stashed = None                                     # output of execute_model, handed out by sample_tokens
        self._deferred = None                                    # a step that waits for its grammar bitmask
        self.async_scheduling = bool(getattr(vllm_config.scheduler_config, "async_scheduling", False))
        # speculative decoding driven by vLLM's scheduler: the n-gram method runs here (drafts are
        # looked up on the host after every step and handed to vLLM through take_draft_token_ids;
        # vLLM schedules them, this worker verifies them in one pass of 1 + k rows per request)
        self.proposer = None
        self._drafts = None
        self._step_drafts = None
        sc = getattr(vllm_config, "speculative_config", None)
        self.mtp_drafts = False          # drafts come from the runner's MTP head (its chain of k steps)
        if sc is not None:
            method = str(getattr(sc, "method", "") or "")
            if method == "ngram":
                from ..spec_decode.ngram_proposer import NgramProposer
                self.proposer = NgramProposer(int(sc.num_speculative_tokens),
                                              int(getattr(sc, "prompt_lookup_min", None) or 2),
                                              int(getattr(sc, "prompt_lookup_max", None) or 4))
            elif method in MTP_METHODS:
                self.mtp_drafts = True
            else:
                raise NotImplementedError(f"speculative method {method!r} under vLLM's scheduler is not supported by "
                                          "the B200 worker (n-gram look-up and the model's MTP head are)")
            self.translator.allow_spec = True

    # ---------------------------------------------------------------- set-up
    def init_device(self) -> None:
        from vllm.platforms import current_platform
        from .worker import Worker
        device_type = "cuda" if current_platform.device_type == "cuda" and torch.cuda.is_available() else "cpu"
        if device_type == "cuda":
            os.environ.pop("NCCL_ASYNC_ERROR_HANDLING", None)
            self.device = torch.device("cuda", self.local_rank)
            torch.cuda.set_device(self.device)
        else:
            self.device = torch.device("cpu")
        # vLLM's own groups (executor message queues, process titles and any vLLM layer that
        # asks for them) on the default process group; this package's groups are built on the
        # same default group below
        from vllm.v1.worker.gpu_worker import init_worker_distributed_environment
        init_worker_distributed_environment(self.vllm_config, self.rank, self.distributed_init_method,
                                            self.local_rank, current_platform.dist_backend)
        self.engine_config = engine_config_from_vllm(self.vllm_config, device_type)
        try:
            from ..models import config_loader
            mc = self.vllm_config.model_config
            config_loader.load_model_extra_config(
                mc.hf_config, enforce_eager=bool(mc.enforce_eager),
                enable_chunked_prefill=bool(getattr(self.scheduler_config, "enable_chunked_prefill", True)),
                enable_eplb=bool(getattr(self.parallel_config, "enable_eplb", False)),
                additional_config=getattr(self.vllm_config, "additional_config", None))
            config_loader.apply_to_runtime()
        except Exception as e:                             # a missing plan is not fatal: defaults apply
            logger.debug("deployment plan not applied: %s", e)
        self.inner = Worker(self.engine_config, local_rank=self.local_rank, rank=self.rank,
                            distributed_init_method=self.distributed_init_method,
                            is_driver_worker=self.is_driver_worker)
        self.inner.init_device()
        self.model_runner = self.inner.model_runner
        self.ha_agent = self.inner.ha_agent
        logger.info("B200 worker rank %d on %s: own model runner (%s), tp=%d", self.rank, self.device,
                    type(self.model_runner).__name__, self.engine_config.parallel.tensor_parallel_size)

    def load_model(self, *, load_dummy_weights: bool = False) -> None:
        if load_dummy_weights:
            self.engine_config.load_format = "dummy"
        self.inner.load_model()

    def get_model(self):
        return self.inner.get_model()

    def get_supported_tasks(self):
        return ("generate",)

    def update_max_model_len(self, max_model_len: int) -> None:
        self.model_config.max_model_len = max_model_len

    # -------------------------------------------------------------- KV cache
    def get_kv_cache_spec(self) -> Dict[str, Any]:
        """One attention spec per layer, sized like the runner's own cache layout, so that vLLM's
        block count times ``page_size_bytes`` is what the runner will allocate."""
        from vllm.v1.kv_cache_interface import FullAttentionSpec, MLAAttentionSpec, SinkFullAttentionSpec
        spec = self.model_runner.get_kv_cache_spec()
        mc = self.engine_config.model
        self._kv_bytes_per_block = spec.bytes_per_block
        per_layer = spec.bytes_per_block // spec.num_layers
        esz = mc.dtype.itemsize
        out: Dict[str, Any] = {}
        for i in range(spec.num_layers):
            name = f"model.layers.{i}.self_attn.attn"
            if spec.kind == "gqa":
                # per-block shapes of the runner's own caches: k [heads, block, D], v [heads, block, Dv]
                hk, _, dk = spec.shapes["k"]
                dv = spec.shapes["v"][-1]
                # Static attention sinks: the model keeps its learned sink tokens in the blocks right
                # after the null block; vLLM's sink manager takes exactly those out of its free
                # queue (reference: SinkFullAttentionSpec and the manager that pops the sink blocks,
                # omni_npu/vllm_patches/patches/models/pangu72b-vl/patch_kv_cache_interface.py:88-141,
                # .../pangu_sink_swa_mla/patch_single_type_kv_cache_manager.py:26-62)
                reserved = int(getattr(self.inner.get_model(), "num_reserved_kv_blocks", 0))
                kw = dict(block_size=spec.block_size, num_kv_heads=int(hk), head_size=int(dk),
                          head_size_v=int(dv), dtype=mc.dtype)
                if reserved > 1:
                    s = SinkFullAttentionSpec(sink_len=(reserved - 1) * spec.block_size, **kw)
                else:
                    s = FullAttentionSpec(**kw)
            else:
                width = per_layer // (spec.block_size * esz)      # latent + rope (+ index key) columns
                s = MLAAttentionSpec(block_size=spec.block_size, num_kv_heads=1, head_size=width, dtype=mc.dtype)
            if s.page_size_bytes != per_layer:
                raise RuntimeError(f"KV spec of layer {i} is {s.page_size_bytes} bytes per block, the runner "
                                   f"allocates {per_layer}")
            out[name] = s
        return out

    def get_cache_block_size_bytes(self) -> int:
        return self._kv_bytes_per_block or self.model_runner.get_kv_cache_spec().bytes_per_block

    @torch.inference_mode()
    def determine_available_memory(self) -> int:
        """Bytes this rank can give to the KV cache: the requested share of the device minus what
        is in use after loading and minus the activation peak of the largest prefill step."""
        cc = self.cache_config
        explicit = getattr(cc, "kv_cache_memory_bytes", None)
        if explicit:
            return int(explicit)
        if self.device.type != "cuda":
            spec = self.model_runner.get_kv_cache_spec()
            want = self.engine_config.scheduler.max_num_seqs * self.engine_config.scheduler.max_model_len
            return max(64, 2 * want // spec.block_size + 8) * spec.bytes_per_block
        peak = self.model_runner.profile_run()
        free, total = torch.cuda.mem_get_info(self.device)
        budget = int(total * cc.gpu_memory_utilization) - (total - free) - peak
        logger.info("KV cache budget %.2f GiB (activation peak %.2f GiB)", budget / 2**30, peak / 2**30)
        if budget <= 0:
            raise RuntimeError("no device memory left for the KV cache; lower max_num_batched_tokens or raise "
                               "gpu_memory_utilization")
        return budget

    def initialize_from_config(self, kv_cache_config) -> None:
        num_blocks = int(kv_cache_config.num_blocks)
        self.cache_config.num_gpu_blocks = num_blocks
        self.inner.initialize_from_config(num_blocks)
        logger.info("KV cache: %d blocks of %d tokens", num_blocks, self.engine_config.cache.block_size)

    def initialize_cache(self, num_gpu_blocks: int, num_cpu_blocks: int) -> None:
        self.cache_config.num_gpu_blocks = num_gpu_blocks
        self.cache_config.num_cpu_blocks = num_cpu_blocks

    def compile_or_warm_up_model(self):
        from vllm.v1.worker.worker_base import CompilationTimes
        self.inner.compile_or_warm_up_model()
        return CompilationTimes(language_model=float(self.model_runner.timings.get("capture_s", 0.0)), encoder=0.0)

    # ---------------------------------------------------------------- running
    @torch.inference_mode()
    def execute_model(self, scheduler_output):
        from vllm.v1.outputs import EMPTY_MODEL_RUNNER_OUTPUT, ModelRunnerOutput
        out = self.translator.translate(scheduler_output)
        if getattr(scheduler_output, "has_structured_output_requests", False) and out.kind != "idle":
            # the grammar bitmask of this step arrives with sample_tokens(): the whole step (forward
            # pass and sampling are one launch sequence here) runs there, with the bitmask applied to
            # the logits before sampling
            if out.kind in ("spec_decode", "prefill+spec") or self.mtp_drafts:
                raise NotImplementedError("structured outputs together with speculative decoding are not "
                                          "supported by the B200 worker")
            self._deferred = out
            return None
        if out.kind == "idle":
            self.inner.execute_model(out)                 # retire rows of finished requests
            return EMPTY_MODEL_RUNNER_OUTPUT
        runner = self.model_runner
        if (self.async_scheduling and out.kind == "decode" and runner.mtp is None and self.proposer is None
                and not any(runner.needs_host_logits(s.request) for s in out.seqs)):
            # vLLM scheduled this step before the previous one's tokens were read: launch it without
            # waiting; token values missing on the host are fed forward on the device
            prev = self._inflight
            handle = self.inner.launch_decode(out, prev.handle if prev is not None and prev._result is None else None)
            pending = PendingDecodeOutput(self, out, handle, self.translator.commit_pending(out))
            self._inflight = pending
            self.steps["decode"] = self.steps.get("decode", 0) + 1
            self.steps["launched_ahead"] = self.steps.get("launched_ahead", 0) + 1
            self._stashed = pending
            return None
        if self._inflight is not None:
            self._inflight.tokens_on_host()               # anything else stages token values on the host
            self._inflight = None
        tokens = self._run(out)
        sampled = self.translator.commit(out, tokens)
        req_ids = [s.request.request_id for s in out.seqs]
        if self.proposer is not None:
            # drafts for the next step of every request that got a token in this one
            self._drafts = (req_ids, [self.proposer.propose_one(s.request.all_token_ids) if toks else []
                                      for s, toks in zip(out.seqs, sampled)])
        elif self.mtp_drafts:
            # the MTP head ran inside the step (on the hidden states of the accepted positions)
            got = self._step_drafts or [[] for _ in out.seqs]
            self._drafts = (req_ids, [[int(t) for t in d] if toks else [] for d, toks in zip(got, sampled)])
        self._stashed = ModelRunnerOutput(req_ids=req_ids, req_id_to_index={r: i for i, r in enumerate(req_ids)},
                                          sampled_token_ids=sampled,
                                          logprobs=logprobs_lists(out.seqs, sampled, runner.last_logprobs),
                                          prompt_logprobs_dict={}, pooler_output=[])
        return None

    # a mixed step is split when it carries at least this many decoding sequences
    MIXED_SPLIT_MIN_DECODES = int(os.environ.get("OMNI_B200_MIXED_SPLIT_MIN", "8"))
    # models whose attention layers take the decoding rows of a mixed step through the decode kernel
    # (grouped-query attention) run such a step as ONE pass; 0 = always two launches
    MIXED_ONE_PASS = os.environ.get("OMNI_B200_MIXED_ONE_PASS", "1") != "0"

    def _gqa_only(self) -> bool:
        if getattr(self, "_gqa_only_cached", None) is None:
            from ..attention.gqa import GQAAttention
            from ..attention.mla import MLAAttention
            mods = list(self.get_model().modules())
            other = any(isinstance(m, MLAAttention) or type(m).__name__ == "PanguSinkAttention" for m in mods)
            self._gqa_only_cached = any(type(m) is GQAAttention for m in mods) and not other
        return self._gqa_only_cached

    def _run(self, out) -> List[int]:
        """Run one translated step.  vLLM's chunked prefill schedules prompt chunks together with
        decoding sequences.  One-token rows are a poor fit for the variable-length prefill
        attention (a 128-row query tile per sequence and head, the KV of a group read once per
        query head), so a mixed step with enough decoding sequences runs as two launches: the
        decoding sequences through the decode path (CUDA graph, split-KV attention), the prompt
        chunks through the prefill path."""
        from ..engine.scheduler import SchedulerOutput
        self._step_drafts = None
        if any(s.request.sampling_params.logprobs for s in out.seqs):
            if out.kind in ("spec_decode", "prefill+spec") or self.mtp_drafts:
                raise NotImplementedError("logprobs together with speculative decoding are not supported by the "
                                          "B200 worker")
            # one launch, so that the step's log-probabilities line up with its sequences
            self.steps[out.kind] = self.steps.get(out.kind, 0) + 1
            return self.inner.execute_model(out)
        if self.mtp_drafts:
            return self._run_mtp(out)
        if out.kind == "prefill+spec":
            # verification rows and prompt chunks in one vLLM step: two launches
            ver = [i for i, s in enumerate(out.seqs) if s.spec_token_ids or (s.num_new_tokens == 1 and s.samples
                                                                              and s.start > 0)]
            pre = [i for i in range(len(out.seqs)) if i not in set(ver)]
            first = SchedulerOutput(kind="spec_decode", seqs=[out.seqs[i] for i in ver],
                                    num_tokens=sum(out.seqs[i].num_new_tokens for i in ver),
                                    preempted=out.preempted, finished_req_ids=out.finished_req_ids,
                                    step_index=out.step_index)
            second = SchedulerOutput(kind="prefill", seqs=[out.seqs[i] for i in pre],
                                     num_tokens=sum(out.seqs[i].num_new_tokens for i in pre),
                                     step_index=out.step_index)
            tokens = [0] * len(out.seqs)
            for idx, part in ((ver, first), (pre, second)):
                if idx:
                    for i, t in zip(idx, self.inner.execute_model(part)):
                        tokens[i] = t
            self.steps["mixed"] = self.steps.get("mixed", 0) + 1
            self.steps["spec_decode"] = self.steps.get("spec_decode", 0) + 1
            return tokens
        if out.kind == "prefill":
            dec = [i for i, s in enumerate(out.seqs) if s.num_new_tokens == 1 and s.samples and s.start > 0]
            if self.MIXED_ONE_PASS and 0 < len(dec) < len(out.seqs) and self._gqa_only():
                # one forward pass over all rows: the decoding sequences first (their rows go through
                # the decode attention kernel), the prompt chunks behind them; the GEMMs see one batch,
                # so the weights stream once instead of once per launch
                pre = [i for i in range(len(out.seqs)) if i not in set(dec)]
                order = dec + pre
                one = SchedulerOutput(kind="prefill", seqs=[out.seqs[i] for i in order], num_tokens=out.num_tokens,
                                      preempted=out.preempted, finished_req_ids=out.finished_req_ids,
                                      step_index=out.step_index, num_decode_seqs=len(dec))
                tokens = [0] * len(out.seqs)
                for i, t in zip(order, self.inner.execute_model(one)):
                    tokens[i] = t
                self.steps["mixed"] = self.steps.get("mixed", 0) + 1
                self.steps["mixed_one_pass"] = self.steps.get("mixed_one_pass", 0) + 1
                return tokens
            if self.MIXED_SPLIT_MIN_DECODES <= len(dec) < len(out.seqs):
                pre = [i for i in range(len(out.seqs)) if i not in set(dec)]
                first = SchedulerOutput(kind="decode", seqs=[out.seqs[i] for i in dec], num_tokens=len(dec),
                                        preempted=out.preempted, finished_req_ids=out.finished_req_ids,
                                        step_index=out.step_index)
                second = SchedulerOutput(kind="prefill", seqs=[out.seqs[i] for i in pre],
                                         num_tokens=sum(out.seqs[i].num_new_tokens for i in pre),
                                         step_index=out.step_index)
                tokens: List[int] = [0] * len(out.seqs)
                for idx, part in ((dec, first), (pre, second)):
                    for i, t in zip(idx, self.inner.execute_model(part)):
                        tokens[i] = t
                self.steps["mixed"] = self.steps.get("mixed", 0) + 1
                return tokens
        self.steps[out.kind] = self.steps.get(out.kind, 0) + 1
        return self.inner.execute_model(out)

    def _run_mtp(self, out) -> List[int]:
        """A step of a deployment that drafts with the MTP head: verification rows (and decoding rows
        without drafts) run as one verification pass, prompt chunks as a prefill pass; each pass leaves
        the head's drafts for its sequences in ``runner.last_drafts``."""
        from ..engine.scheduler import SchedulerOutput
        runner = self.model_runner
        n = len(out.seqs)
        ver = [i for i, s in enumerate(out.seqs) if s.spec_token_ids]
        rest = [i for i in range(n) if i not in set(ver)]
        tokens: List[Any] = [0] * n
        drafts: List[List[int]] = [[] for _ in range(n)]
        parts = []
        if ver:
            parts.append((ver, SchedulerOutput(kind="spec_decode", seqs=[out.seqs[i] for i in ver],
                                               num_tokens=sum(out.seqs[i].num_new_tokens for i in ver),
                                               preempted=out.preempted, finished_req_ids=out.finished_req_ids,
                                               step_index=out.step_index)))
        if rest:
            all_dec = all(out.seqs[i].num_new_tokens == 1 and out.seqs[i].samples and out.seqs[i].start > 0
                          for i in rest)
            parts.append((rest, SchedulerOutput(kind="decode" if all_dec else "prefill",
                                                seqs=[out.seqs[i] for i in rest],
                                                num_tokens=sum(out.seqs[i].num_new_tokens for i in rest),
                                                preempted=[] if ver else out.preempted,
                                                finished_req_ids=[] if ver else out.finished_req_ids,
                                                step_index=out.step_index)))
        for idx, part in parts:
            got = self.inner.execute_model(part)
            last = list(getattr(runner, "last_drafts", None) or [])
            for j, i in enumerate(idx):
                tokens[i] = got[j]
                if j < len(last):
                    drafts[i] = list(last[j])
            self.steps[part.kind] = self.steps.get(part.kind, 0) + 1
        self._step_drafts = drafts
        return tokens

    def sample_tokens(self, grammar_output=None):
        """Second half of vLLM's two-call step: the forward pass and the sampling both ran in
        ``execute_model`` (structured-output bitmasks are refused there), this hands the result out."""
        if self._deferred is not None:
            self._run_deferred(grammar_output)
        out, self._stashed = self._stashed, None
        if out is None:
            raise RuntimeError("sample_tokens called without a preceding execute_model")
        return out

    def _run_deferred(self, grammar_output) -> None:
        """A step with structured-output requests: run it now, with the grammar's bitmask (one row
        of ceil(vocab / 32) int32 words per structured request, bit set = token allowed) applied to
        the logits rows of those requests (reference: vLLM's ``apply_grammar_bitmask``)."""
        from vllm.v1.outputs import ModelRunnerOutput
        out, self._deferred = self._deferred, None
        runner = self.model_runner
        if self._inflight is not None:
            self._inflight.tokens_on_host()
            self._inflight = None
        if grammar_output is not None and len(grammar_output.structured_output_request_ids):
            runner.extra_logits_fn = grammar_mask_fn([s.request.request_id for s in out.seqs],
                                                     list(grammar_output.structured_output_request_ids),
                                                     grammar_output.grammar_bitmask)
        try:
            self.steps[out.kind] = self.steps.get(out.kind, 0) + 1
            self.steps["structured"] = self.steps.get("structured", 0) + 1
            tokens = self.inner.execute_model(out)          # one launch: logits rows line up with out.seqs
        finally:
            runner.extra_logits_fn = None
        sampled = self.translator.commit(out, tokens)
        req_ids = [s.request.request_id for s in out.seqs]
        self._stashed = ModelRunnerOutput(req_ids=req_ids, req_id_to_index={r: i for i, r in enumerate(req_ids)},
                                          sampled_token_ids=sampled,
                                          logprobs=logprobs_lists(out.seqs, sampled, runner.last_logprobs),
                                          prompt_logprobs_dict={}, pooler_output=[])

    def take_draft_token_ids(self):
        """Drafts proposed after the last step, in vLLM's container (None without a proposer)."""
        drafts, self._drafts = self._drafts, None
        if drafts is None:
            return None
        from vllm.v1.outputs import DraftTokenIds
        return DraftTokenIds(req_ids=list(drafts[0]), draft_token_ids=[list(d) for d in drafts[1]])

    def execute_dummy_batch(self) -> None:
        self.inner.execute_dummy_batch()

    def profile(self, is_start: bool = True, profile_prefix: Optional[str] = None) -> None:
        self.inner.profile(is_start)

    def check_health(self) -> None:
        from .. import ops
        if self.device is not None and self.device.type == "cuda":
            ops.check_status(self.device)

    # ------------------------------------------------------------------ LoRA
    def add_lora(self, lora_request) -> bool:
        raise NotImplementedError("LoRA is not supported by the B200 worker")

    def remove_lora(self, lora_id: int) -> bool:
        return False

    def pin_lora(self, lora_id: int) -> bool:
        return False

    def list_loras(self) -> set:
        return set()

    # -------------------------------------------------------------- sleep mode
    def sleep(self, level: int = 1) -> None:
        self.inner.sleep(level)

    def wake_up(self, tags: Optional[list] = None) -> None:
        self.inner.wake_up(tags)

    # token-recovery hooks (ha/monitor.py)
    def stop_device(self) -> None:
        self.inner.stop_device()

    def restart_device(self) -> None:
        self.inner.restart_device()

    def reinit_process_group(self) -> None:
        self.inner.reinit_process_group()

    def shutdown(self) -> None:
        if self.inner is not None:
            try:
                self.inner.shutdown()
            except Exception as e:                         # pragma: no cover - best effort at exit
                logger.warning("worker shutdown: %s", e)
