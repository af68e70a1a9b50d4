"""Continuous-batching scheduler with chunked prefill and recompute preemption.

A step is either a *prefill* step (one or more prompt chunks, run eagerly) or
a *decode* step (one new token for every running sequence, run from a CUDA
graph).  Prefill has priority while there is room for more running sequences.
KV-connector hooks mirror the life cycle the reference drives through vLLM's
scheduler (omni_npu/connector/llmdatadist_connector_v1.py:233-291,457-576):
a consumer request first waits for its remote KV, a producer request parks its
blocks after finishing so they can still be pulled.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict, List, Optional, Tuple

from ..config import CacheConfig, SchedulerConfig
from .block_manager import BlockPool
from .request import Request, RequestStatus


@dataclass
class ScheduledSeq:
    request: Request
    start: int             # tokens already in the KV cache before this step
    num_new_tokens: int    # tokens computed in this step
    samples: bool          # whether this step yields an output token for the request
    spec_token_ids: List[int] = field(default_factory=list)   # draft tokens verified in this step


@dataclass
class SchedulerOutput:
    kind: str = "idle"                      # "prefill" | "decode" | "spec_decode" | "idle"
    seqs: List[ScheduledSeq] = field(default_factory=list)
    num_tokens: int = 0
    # mixed batches: the first num_decode_seqs entries of a "prefill" step are decoding requests
    # that ride along with one token each
    num_decode_seqs: int = 0
    preempted: List[str] = field(default_factory=list)
    finished_req_ids: List[str] = field(default_factory=list)
    kv_connector_metadata: Any = None
    step_index: int = 0
    pending_pos: List[int] = field(default_factory=list)   # asynchronous scheduling: output index of each placeholder

    @property
    def total_num_scheduled_tokens(self) -> int:
        return self.num_tokens


class Scheduler:
    def __init__(self, sched_cfg: SchedulerConfig, cache_cfg: CacheConfig, num_blocks: int,
                 num_reserved_blocks: int = 0, kv_connector=None, context_parallel_size: int = 1) -> None:
        self.cfg = sched_cfg
        # With decode context parallelism every rank stores 1 / world of a sequence's tokens
        # (token p on rank p % world), so one block id covers block_size * world tokens.
        self.block_size = cache_cfg.block_size * max(1, context_parallel_size)
        # automatic prefix caching: full blocks are findable by the hash of their token prefix and
        # shared between requests (not together with a KV connector, whose blocks are pulled by id)
        self.pool = BlockPool(num_blocks, self.block_size, num_reserved_blocks,
                              prefix_caching=bool(getattr(cache_cfg, "enable_prefix_caching", False))
                              and kv_connector is None)
        self.prefix_stats = {"requests": 0, "hit_tokens": 0}
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.requests: Dict[str, Request] = {}
        self.kv_connector = kv_connector
        self._finished_since_last: List[str] = []
        self._step = 0
        self.spec_stats = {"drafted": 0, "accepted": 0}
        self.num_preemptions = 0          # over the life of the scheduler (finished requests leave ``requests``)
        self.kv_load_failures = 0

    # ------------------------------------------------------------------ intake
    def add_request(self, req: Request) -> None:
        if req.num_prompt_tokens >= self.cfg.max_model_len:
            raise ValueError(f"prompt of {req.num_prompt_tokens} tokens exceeds max_model_len "
                             f"{self.cfg.max_model_len}")
        usable = self.pool.num_blocks - self.pool.num_reserved
        if self.pool.blocks_needed(req.num_prompt_tokens) > usable:
            raise ValueError(f"prompt of {req.num_prompt_tokens} tokens does not fit the KV cache "
                             f"({usable} blocks of {self.block_size} tokens)")
        self.requests[req.request_id] = req
        if self.cfg.policy == "priority":
            # keep the queue ordered by (priority, arrival): behind every request that is at least as urgent
            key = (req.sampling_params.priority, req.arrival_time)
            pos = len(self.waiting)
            while pos > 0 and (self.waiting[pos - 1].sampling_params.priority,
                               self.waiting[pos - 1].arrival_time) > key \
                    and self.waiting[pos - 1].status != RequestStatus.PREEMPTED:
                pos -= 1
            self.waiting.insert(pos, req)
        else:
            self.waiting.append(req)

    def abort_request(self, request_id: str) -> None:
        req = self.requests.get(request_id)
        if req is None or req.is_finished:
            return
        req.status = RequestStatus.FINISHED_ABORTED
        req.finish_time = time.monotonic()
        if req in self.running:
            self.running.remove(req)
        elif req in self.waiting:
            self.waiting.remove(req)
        self._release(req)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    @property
    def num_unfinished(self) -> int:
        return len(self.waiting) + len(self.running)

    # ---------------------------------------------------------------- blocks
    def _ensure_blocks(self, req: Request, total_tokens: int) -> bool:
        look = getattr(self.cfg, "num_lookahead_tokens", 0)
        if look:
            # slots for a draft head's chain of extra steps (never past the longest sequence allowed)
            total_tokens = max(total_tokens, min(total_tokens + look, self.cfg.max_model_len))
        need = self.pool.blocks_needed(total_tokens, len(req.block_ids))
        if need == 0:
            return True
        if not self.pool.can_allocate(need):
            return False
        req.block_ids.extend(self.pool.allocate(need))
        return True

    # ------------------------------------------------------------ prefix caching
    def _attach_cached_prefix(self, req: Request) -> bool:
        """Give a request that starts from nothing the cached blocks of its longest known prefix
        (whole blocks, and never the whole sequence: the last token is always computed)."""
        from .block_manager import chain_block_hashes
        bs = self.block_size
        usable = (req.num_tokens - 1) // bs
        # a request that wants the log-probabilities of its prompt has to run every prompt row
        if usable <= 0 or req.sampling_params.prompt_logprobs is not None:
            return False
        toks = req.all_token_ids
        req._block_hashes = chain_block_hashes(toks, bs, getattr(req, "_block_hashes", None), upto_blocks=usable)
        hit = self.pool.match_prefix(req._block_hashes[:usable])
        self.prefix_stats["requests"] += 1
        if not hit:
            return False
        self.pool.acquire(hit)
        req.block_ids = list(hit)
        req.num_computed_tokens = len(hit) * bs
        req._registered_blocks = len(hit)
        self.prefix_stats["hit_tokens"] += len(hit) * bs
        return True

    def _detach_cached_prefix(self, req: Request) -> None:
        self.prefix_stats["hit_tokens"] -= len(req.block_ids) * self.block_size
        self.pool.free(req.block_ids)
        req.block_ids = []
        req.num_computed_tokens = 0
        req._registered_blocks = 0

    def _register_full_blocks(self, req: Request) -> None:
        """Make the blocks that this request has filled with settled tokens findable by content."""
        if not self.pool.prefix_caching:
            return
        bs = self.block_size
        nfull = min(req.num_computed_tokens, req.num_tokens) // bs
        done = getattr(req, "_registered_blocks", 0)
        if nfull <= done or nfull > len(req.block_ids):
            return
        from .block_manager import chain_block_hashes
        hashes = chain_block_hashes(req.all_token_ids, bs, getattr(req, "_block_hashes", None), upto_blocks=nfull)
        req._block_hashes = hashes
        upto = min(len(hashes), nfull)
        for i in range(done, upto):
            self.pool.register(req.block_ids[i], hashes[i])
        req._registered_blocks = max(done, upto)

    def prompt_work_waiting(self) -> bool:
        """Whether this step could hold prompt tokens: a running request with an unfinished prompt
        (or recompute), or a waiting request and a free sequence slot."""
        for req in self.running:
            remaining = req.num_tokens - req.num_computed_tokens
            if remaining > 1 or (remaining == 1 and not req.output_token_ids):
                return True
        return bool(self.waiting) and len(self.running) < self.cfg.max_num_seqs

    def _release(self, req: Request) -> None:
        delay = None
        if self.kv_connector is not None and req.status != RequestStatus.FINISHED_ABORTED:
            delay, params = self.kv_connector.request_finished(req, req.block_ids)
            if params is not None:
                req.kv_transfer_params = params
        if delay:
            self.pool.park(req.request_id, req.block_ids, delay)
        else:
            self.pool.free(req.block_ids)
        req.block_ids = []
        self._finished_since_last.append(req.request_id)
        self.requests.pop(req.request_id, None)      # a long-running server must not keep every request it ever saw

    def _preempt_one(self, protect: Request) -> Optional[Request]:
        """Evict the most recently admitted running request (recompute later); under the priority
        policy the least urgent one (highest priority value, latest arrival)."""
        order = list(reversed(self.running))
        if self.cfg.policy == "priority":
            order = sorted(self.running, key=lambda r: (r.sampling_params.priority, r.arrival_time), reverse=True)
        for victim in order:
            if victim is protect:
                continue
            self.running.remove(victim)
            self.pool.free(victim.block_ids)
            victim.block_ids = []
            victim.num_computed_tokens = 0
            victim._registered_blocks = 0
            victim.status = RequestStatus.PREEMPTED
            victim.num_preemptions += 1
            self.num_preemptions += 1
            self.waiting.appendleft(victim)
            return victim
        return None

    def preempt_for_recompute(self, req: Request) -> None:
        """Send a running request back to the head of the waiting queue; its KV is dropped
        and recomputed from its tokens (prompt + outputs so far)."""
        if req in self.running:
            self.running.remove(req)
        self.pool.free(req.block_ids)
        req.block_ids = []
        req.num_computed_tokens = 0
        req._registered_blocks = 0
        req.spec_token_ids = []
        req.status = RequestStatus.PREEMPTED
        req.num_preemptions += 1
        self.num_preemptions += 1
        if req not in self.waiting:
            self.waiting.appendleft(req)

    # -------------------------------------------------------------- schedule
    def schedule(self) -> SchedulerOutput:
        self._step += 1
        out = SchedulerOutput(step_index=self._step)
        self.pool.expire_parked()
        if self.kv_connector is not None:
            for rid in self.kv_connector.take_released_requests():
                self.pool.release_parked(rid)

        budget = self.cfg.max_num_batched_tokens
        # 0) mixed batches: the decoding requests come first, one token each, when prompt work is
        # waiting.  No eviction on their behalf: a rider that finds no block sits this step out.
        riders: List[ScheduledSeq] = []
        if self.cfg.enable_mixed_batches and self.prompt_work_waiting():
            for req in self.running:
                if budget <= 1:
                    break
                if req.num_tokens - req.num_computed_tokens != 1 or not req.output_token_ids:
                    continue
                if req.spec_token_ids:             # drafts are verified in decode steps only
                    riders = []
                    break
                if not self._ensure_blocks(req, req.num_tokens):
                    continue
                riders.append(ScheduledSeq(req, req.num_computed_tokens, 1, True))
                budget -= 1
            if not riders:
                budget = self.cfg.max_num_batched_tokens
        # 1) unfinished prompt chunks of running requests, then new admissions
        prefill: List[ScheduledSeq] = []
        for req in list(self.running):
            if req not in self.running:            # evicted below to make room for an earlier request
                continue
            remaining = req.num_tokens - req.num_computed_tokens
            if remaining > 1 or (remaining == 1 and not req.output_token_ids):
                n = min(remaining, budget)
                if n <= 0:
                    break
                if not self.cfg.enable_chunked_prefill and n < remaining:
                    break
                # A half-computed prompt must never reach the decode branch (it would sample from
                # an incomplete context).  When its next chunk finds no blocks, later-admitted
                # requests are evicted for it; if it is itself the latest one, it goes back to the
                # waiting queue and is recomputed when blocks are free again.
                fits = self._ensure_blocks(req, req.num_computed_tokens + n)
                while not fits:
                    victim = self.running[-1]
                    if victim is req:
                        if len(self.running) == 1 and not prefill:
                            raise RuntimeError("KV cache too small for a single sequence")
                        self.preempt_for_recompute(req)
                        out.preempted.append(req.request_id)
                        break
                    self.preempt_for_recompute(victim)
                    out.preempted.append(victim.request_id)
                    for s in prefill:
                        if s.request is victim:
                            budget += s.num_new_tokens
                    prefill = [s for s in prefill if s.request is not victim]
                    fits = self._ensure_blocks(req, req.num_computed_tokens + n)
                if not fits:
                    continue
                prefill.append(ScheduledSeq(req, req.num_computed_tokens, n, n == remaining))
                budget -= n
        # nothing is admitted in a step that had to evict: the evicted request sits at the head of
        # the queue and would take the freed blocks straight back
        while (self.waiting and budget > 0 and len(self.running) < self.cfg.max_num_seqs
               and not out.preempted):
            req = self.waiting[0]
            if req.status == RequestStatus.WAITING_FOR_REMOTE_KVS:
                done = False
                if self.kv_connector is not None:
                    try:
                        done = self.kv_connector.is_load_finished(req)
                    except ConnectionError as e:
                        # the producer is gone or the pull failed: compute the prompt here instead
                        # (the blocks already allocated for the remote KV are simply filled locally)
                        self.kv_load_failures += 1
                        req.num_external_tokens = 0
                        req.kv_transfer_params = None
                        req.num_computed_tokens = 0
                        done = True
                        import logging
                        logging.getLogger("omni_npu_b200").warning("%s: falling back to local prefill", e)
                if done:
                    req.status = RequestStatus.WAITING
                else:
                    # keep order simple: look at the next request instead
                    self.waiting.rotate(-1)
                    if all(r.status == RequestStatus.WAITING_FOR_REMOTE_KVS for r in self.waiting):
                        break
                    continue
            if (self.kv_connector is not None and req.num_computed_tokens == 0
                    and req.num_external_tokens == 0 and req.kv_transfer_params):
                ext, is_async = self.kv_connector.get_num_new_matched_tokens(req, 0)
                if ext > 0:
                    if not self._ensure_blocks(req, ext):
                        break
                    req.num_external_tokens = ext
                    self.kv_connector.update_state_after_alloc(req, req.block_ids, ext)
                    if is_async:
                        req.status = RequestStatus.WAITING_FOR_REMOTE_KVS
                        continue
            if req.num_external_tokens and req.num_computed_tokens == 0:
                # remote KV covers the prompt except (at least) its last token
                req.num_computed_tokens = min(req.num_external_tokens, req.num_tokens - 1)
            attached = (self.pool.prefix_caching and req.num_computed_tokens == 0 and not req.block_ids
                        and self._attach_cached_prefix(req))
            remaining = req.num_tokens - req.num_computed_tokens
            n = min(remaining, budget)
            # admit only when the whole prompt would fit now: a prompt admitted chunk by chunk into
            # a nearly full cache is evicted half-way and recomputed over and over
            if ((n < remaining and not self.cfg.enable_chunked_prefill)
                    or not self.pool.can_allocate(self.pool.blocks_needed(req.num_tokens, len(req.block_ids)))
                    or not self._ensure_blocks(req, req.num_computed_tokens + n)):
                if attached:
                    self._detach_cached_prefix(req)
                break
            self.waiting.popleft()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            prefill.append(ScheduledSeq(req, req.num_computed_tokens, n, n == remaining))
            budget -= n
        if prefill:
            # a rider whose request was evicted for a prompt chunk above is dropped
            riders = [s for s in riders if s.request in self.running]
            out.kind = "prefill"
            out.seqs = riders + prefill
            out.num_decode_seqs = len(riders)
            out.num_tokens = sum(s.num_new_tokens for s in out.seqs)
            self._finish_output(out)
            return out

        # 2) decode: one token for every running request, plus its draft tokens to verify
        decode: List[ScheduledSeq] = []
        i = 0
        while i < len(self.running):
            req = self.running[i]
            if req.num_tokens - req.num_computed_tokens > 1:
                i += 1                 # prompt (or recompute) not finished: never sampled from here
                continue
            # drafts must leave room for the bonus token inside max_model_len and the budget
            room = min(self.cfg.max_model_len - req.num_tokens - 1,
                       req.sampling_params.max_tokens - len(req.output_token_ids) - 1)
            drafts = req.spec_token_ids[: max(0, room)] if req.spec_token_ids else []
            while not self._ensure_blocks(req, req.num_tokens + len(drafts)):
                victim = self._preempt_one(protect=req)
                if victim is None:
                    raise RuntimeError("KV cache too small for a single sequence")
                out.preempted.append(victim.request_id)
                victim.spec_token_ids = []
                decode = [s for s in decode if s.request is not victim]
            if req in self.running:
                decode.append(ScheduledSeq(req, req.num_computed_tokens, 1 + len(drafts), True, list(drafts)))
            i = self.running.index(req) + 1
        if decode:
            spec = any(s.spec_token_ids for s in decode)
            out.kind = "spec_decode" if spec else "decode"
            out.seqs = decode
            out.num_tokens = sum(s.num_new_tokens for s in decode)
        self._finish_output(out)
        return out

    # ------------------------------------------------ decode steps settled one step late
    # With asynchronous scheduling the host launches decode step n + 1 before it has read the tokens
    # of step n: the token VALUES are fed forward on the device, the host only needs the COUNTS to
    # build the next step.  ``advance_pending`` does the bookkeeping of a launched step with
    # placeholder tokens; ``resolve_pending`` fills the values in when they arrive.
    PENDING_TOKEN = -1

    def advance_pending(self, out: SchedulerOutput, now: Optional[float] = None) -> None:
        now = time.monotonic() if now is None else now
        out.pending_pos = []
        done: List[Request] = []
        for seq in out.seqs:
            req = seq.request
            req.num_computed_tokens = seq.start + seq.num_new_tokens
            req.spec_token_ids = []
            self._register_full_blocks(req)
            req.append_output(self.PENDING_TOKEN, now)
            out.pending_pos.append(len(req.output_token_ids) - 1)
            if len(req.output_token_ids) >= req.sampling_params.max_tokens or req.num_tokens >= self.cfg.max_model_len:
                # ends by length whatever the token turns out to be
                req.status = RequestStatus.FINISHED_LENGTH_CAPPED
                req.finish_time = now
                done.append(req)
        for req in done:
            self.running.remove(req)
            self._release(req)

    def resolve_pending(self, out: SchedulerOutput, tokens: List[int], now: Optional[float] = None) -> List[Request]:
        """Tokens of a step accounted by ``advance_pending``.  A request whose token ends it (EOS,
        stop token) finishes now; the placeholder a later launched step already appended for it is
        dropped and that step's token for it is ignored.  Returns the requests this step finished."""
        now = time.monotonic() if now is None else now
        finished: List[Request] = []
        for seq, tok, pos in zip(out.seqs, tokens, out.pending_pos):
            req = seq.request
            if pos >= len(req.output_token_ids):
                continue                      # the request ended at an earlier token: surplus step
            if req.status == RequestStatus.FINISHED_ABORTED:
                continue
            req.output_token_ids[pos] = int(tok)
            sp = req.sampling_params
            stop = ((not sp.ignore_eos and req.eos_token_id is not None and int(tok) == req.eos_token_id)
                    or int(tok) in sp.stop_token_ids)
            if stop:
                del req.output_token_ids[pos + 1:]
                was_running = not req.is_finished
                req.status = RequestStatus.FINISHED_STOPPED
                req.finish_time = now
                if was_running:
                    if req in self.running:
                        self.running.remove(req)
                    elif req in self.waiting:          # preempted in the meantime
                        self.waiting.remove(req)
                    self._release(req)
                finished.append(req)
            elif req.is_finished and pos == len(req.output_token_ids) - 1:
                finished.append(req)          # ended by length in advance_pending; this was its last token
        return finished

    def _finish_output(self, out: SchedulerOutput) -> None:
        out.finished_req_ids, self._finished_since_last = self._finished_since_last, []
        if self.kv_connector is not None:
            out.kv_connector_metadata = self.kv_connector.build_connector_meta(out)

    # ---------------------------------------------------------------- update
    def update_from_output(self, out: SchedulerOutput, sampled: List, now: Optional[float] = None,
                           drafts: Optional[List[List[int]]] = None) -> List[Request]:
        """Apply one step's results.  ``sampled[i]`` belongs to ``out.seqs[i]``: one token,
        or (after a verification step) the list of tokens the step settled.  ``drafts[i]``
        are the draft tokens proposed for the request's next step.  Returns requests that
        finished in this step."""
        finished: List[Request] = []
        now = time.monotonic() if now is None else now
        for idx, (seq, tok) in enumerate(zip(out.seqs, sampled)):
            req = seq.request
            if req.is_finished:
                continue
            toks = list(tok) if isinstance(tok, (list, tuple)) else [tok]
            if seq.spec_token_ids:
                # the KV entries of the accepted drafts (and of the token before them) are valid;
                # the last emitted token has none yet
                req.num_computed_tokens = seq.start + len(toks)
                self.spec_stats["drafted"] += len(seq.spec_token_ids)
                self.spec_stats["accepted"] += len(toks) - 1
            else:
                req.num_computed_tokens = seq.start + seq.num_new_tokens
            req.spec_token_ids = []
            self._register_full_blocks(req)
            if not seq.samples:
                continue
            done = False
            for t in toks:
                req.append_output(t, now)
                if req.check_stop() or req.num_tokens >= self.cfg.max_model_len:
                    if not req.is_finished:
                        req.status = RequestStatus.FINISHED_LENGTH_CAPPED
                        req.finish_time = now
                    done = True
                    break
            if done:
                finished.append(req)
            elif drafts is not None and idx < len(drafts) and drafts[idx]:
                req.spec_token_ids = [int(t) for t in drafts[idx]]
        for req in finished:
            self.running.remove(req)
            self._release(req)
        return finished
