"""OpenAI-compatible HTTP front end of the standalone engine.

    python -m omni_npu_b200.serving.api_server --model llama-3-8b --port 8000 \
        --max-num-seqs 128 --tensor-parallel-size 1 [--kv-transfer-config '{...}'] \
        [--reasoning-parser pangu] [--tool-call-parser pangu] [--reasoning-config '{...}']

Endpoints: ``POST /v1/completions`` (token ids or text when a tokenizer directory is
given), ``POST /v1/chat/completions``, ``GET /v1/models``, ``GET /health``,
``GET /metrics`` (Prometheus text).  One engine thread runs ``LLMEngine.step`` in a loop;
request handlers enqueue requests and wait for their outputs (streaming sends one
server-sent event per engine step that produced tokens for the request).

The reference serves through ``vllm serve`` with its platform plugin
(examples/serve-single-instance.sh:100-187); this module is the same surface for the
standalone engine, including the request field ``thinking_token_budget``
(omni_npu/vllm_patches/patches/common/patch_think_limit.py) and ``kv_transfer_params`` for
prefill/decode disaggregation.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import threading
import time
import uuid
from typing import Any, Dict, List, Optional

from ..engine.request import RequestOutput, SamplingParams
from ..logger import logger
from ..sample.structured import structured_spec_from_body


class EngineLoop:
    """Owns the engine; a background thread steps it while there is work."""

    def __init__(self, llm, follower: bool = False) -> None:
        self.llm = llm
        self.engine = llm.engine
        # Ranks of one replica (tensor x pipeline parallel) run the same deterministic scheduler, so they
        # must see the same requests in the same order between the same steps.  HTTP arrives at rank 0
        # only: before every step it broadcasts what arrived since the last one (``_run_leader``), the
        # other ranks apply it and step when told (``run_follower``).
        from ..parallel import state as pstate
        world = pstate.get_world_group()
        self.group = world if world.world_size > 1 else None
        if getattr(self.engine, "dp_group", None) is not None:
            # one server per data-parallel rank: nothing to replicate when the replica is a single rank
            self.group = None
        if self.group is None and getattr(self.engine, "dp_group", None) is not None and \
                pstate.get_tp_group().world_size * pstate.get_pp_group().world_size > 1:
            raise NotImplementedError("the API server replicates requests inside ONE replica: start one server "
                                      "per data-parallel rank with tensor_parallel_size * pipeline_parallel_size == 1, "
                                      "or use data_parallel_size == 1")
        self._new: List[tuple] = []
        self._aborts: List[str] = []
        self.tokenizer = None                 # set by build_app: stop strings are matched on decoded text
        self.lock = threading.Lock()
        self.wake = threading.Event()
        self.waiters: Dict[str, Dict[str, Any]] = {}
        self.running = True
        self.thread = None
        if not follower:
            self.thread = threading.Thread(target=self._run if self.group is None else self._run_leader, daemon=True)
            self.thread.start()
        self.counters = {"requests": 0, "finished": 0, "output_tokens": 0, "steps": 0}

    def submit(self, prompt_ids: List[int], sp: SamplingParams, kv_transfer_params=None,
               stop: Optional[List[str]] = None) -> str:
        """``stop``: strings that end the request when they appear in its decoded output (needs
        ``self.tokenizer``); the answer's text is cut before the first of them."""
        self.engine.validate_sampling_params(sp)        # ValueError -> HTTP 400, before anything is queued
        if stop and self.tokenizer is None:
            raise ValueError("stop strings need a tokenizer (use stop_token_ids on a server without one)")
        rid = f"cmpl-{uuid.uuid4().hex}"
        slot = {"event": threading.Event(), "output": None, "seen": 0, "queue": [], "request": None,
                "stop": [s for s in (stop or []) if s], "text": None}
        with self.lock:
            self.waiters[rid] = slot
            if self.group is None:
                self.engine.add_request(prompt_ids, sp, request_id=rid, kv_transfer_params=kv_transfer_params)
                slot["request"] = self.engine.scheduler.requests[rid]
            else:                                   # added on every rank by the next broadcast
                self._new.append((rid, list(prompt_ids), sp, kv_transfer_params))
            self.counters["requests"] += 1
        self.wake.set()
        return rid

    def abort(self, rid: str) -> None:
        with self.lock:
            if self.group is None:
                self.engine.abort_request(rid)
            else:
                self._aborts.append(rid)
            self.waiters.pop(rid, None)

    def _run(self) -> None:
        # data-parallel replicas step together even when this one is idle (its dummy batches keep
        # the expert-parallel exchanges of the busy replicas going)
        lock_step = getattr(self.engine, "dp_group", None) is not None
        while self.running:
            if not lock_step and not self.engine.has_unfinished_requests():
                self.wake.wait(0.05)
                self.wake.clear()
                continue
            if lock_step and getattr(self.engine, "dp_all_idle", False):
                self.wake.wait(0.002)
                self.wake.clear()
            with self.lock:
                self._publish(self._safe_step())

    def _find_stop(self, ids: List[int], seen: int, stops: List[str]):
        """(tokens to keep, text before the stop string) when a stop string shows up in the decoded
        output, else None.  Only prefixes that end in the newly arrived tokens are decoded."""
        first = max(1, seen + 1)
        for k in range(first, len(ids) + 1):
            text = self.tokenizer.decode(ids[:k])
            hits = [text.find(s) for s in stops if s in text]
            if hits:
                return k - 1, text[: min(hits)]
        return None

    def _safe_step(self):
        """One engine step.  An exception must not end the loop thread (every waiter would hang):
        the requests in flight are failed with finish_reason "abort" and the loop goes on."""
        try:
            return self.engine.step()
        except Exception:
            logger.exception("engine step failed: aborting the requests in flight")
            self.counters["failed_steps"] = self.counters.get("failed_steps", 0) + 1
            return self.engine.fail_all_requests()

    def _publish(self, outs) -> None:
        """After a step (lock held): hand new tokens to streaming waiters, finished outputs to all."""
        self.counters["steps"] += 1
        for rid, slot in self.waiters.items():
            req = slot["request"]
            if req is None:
                continue
            ids = req.output_token_ids
            ready = len(ids)
            while ready > 0 and ids[ready - 1] < 0:     # tokens of a step still in flight
                ready -= 1
            if ready > slot["seen"]:
                new_ids = ids[slot["seen"]:ready]
                if slot["stop"] and slot["output"] is None:
                    cut = self._find_stop(ids[:ready], slot["seen"], slot["stop"])
                    if cut is not None:
                        keep, text = cut
                        # the request ends here: answer now, drop what came after the stop string
                        out = RequestOutput.from_request(req)
                        out.output_token_ids = list(ids[:keep])
                        out.finished, out.finish_reason = True, "stop"
                        out.text = text                       # what the routes answer with instead of decoding
                        slot["queue"].extend(ids[slot["seen"]:keep])
                        slot["seen"] = ready
                        slot["output"] = out
                        slot["event"].set()
                        if self.group is None:
                            self.engine.abort_request(rid)
                        else:
                            self._aborts.append(rid)
                        continue
                slot["queue"].extend(new_ids)
                slot["seen"] = ready
        for o in outs:
            slot = self.waiters.get(o.request_id)
            if slot is not None and slot["output"] is None:
                slot["output"] = o
                slot["event"].set()
            self.counters["finished"] += 1
            self.counters["output_tokens"] += len(o.output_token_ids)

    # ------------------------------------------------ more than one rank per replica
    KEEPALIVE_S = 5.0        # idle leaders still broadcast, so followers never sit in a receive for long

    def _apply(self, new, aborts) -> None:
        for rid, prompt_ids, sp, kvp in new:
            self.engine.add_request(prompt_ids, sp, request_id=rid, kv_transfer_params=kvp)
            slot = self.waiters.get(rid)
            if slot is not None:
                slot["request"] = self.engine.scheduler.requests[rid]
        for rid in aborts:
            self.engine.abort_request(rid)

    def _run_leader(self) -> None:
        last = time.monotonic()
        while self.running:
            with self.lock:
                new, aborts, self._new, self._aborts = self._new, self._aborts, [], []
            busy = bool(new or aborts) or self.engine.has_unfinished_requests()
            if not busy and time.monotonic() - last < self.KEEPALIVE_S:
                self.wake.wait(0.05)
                self.wake.clear()
                continue
            last = time.monotonic()
            self.group.broadcast_object({"new": new, "aborts": aborts, "step": busy, "stop": False}, src=0)
            with self.lock:
                self._apply(new, aborts)
                if busy:
                    self._publish(self._safe_step())
        self.group.broadcast_object({"new": [], "aborts": [], "step": False, "stop": True}, src=0)

    def run_follower(self) -> None:
        """Loop of every rank but the first: apply what rank 0 received, step when it steps."""
        while True:
            msg = self.group.broadcast_object(None, src=0)
            if msg["stop"]:
                return
            self._apply(msg["new"], msg["aborts"])
            if msg["step"]:
                try:
                    self.engine.step()
                except Exception:               # the leader fails the same step the same way
                    logger.exception("engine step failed on a follower rank")
                    self.engine.fail_all_requests()

    def wait(self, rid: str, timeout: Optional[float] = None):
        slot = self.waiters[rid]
        slot["event"].wait(timeout)
        out = slot["output"]
        if out is not None:
            self.waiters.pop(rid, None)
        return out

    def shutdown(self) -> None:
        self.running = False
        self.wake.set()
        if self.thread is not None:
            self.thread.join(timeout=5)


def _logprobs_from_body(body: Dict[str, Any]) -> Optional[int]:
    """Completions: ``logprobs: n``.  Chat: ``logprobs: true`` with ``top_logprobs: n`` (n = 0: the
    sampled token's log-probability only, asked for as 1 alternative here)."""
    lp, top = body.get("logprobs"), body.get("top_logprobs")
    if lp is True:
        return max(1, int(top or 0))
    if lp in (None, False) and not top:
        return None
    return max(1, int(top if top else lp))


def bad_words_token_ids(words, tokenizer) -> Optional[list]:
    """Token sequences of the words a request bans: each word as it is written at the start of a text
    and as it is written after a space (most vocabularies spell the two differently)."""
    if not words:
        return None
    if tokenizer is None:
        raise ValueError("bad_words needs a tokenizer; this server has none")
    seqs = []
    for w in words:
        for text in (w.lstrip(), " " + w.lstrip()):
            ids = [int(t) for t in tokenizer.encode(text, add_special_tokens=False)]
            if ids and ids not in seqs:
                seqs.append(ids)
    return seqs or None


def sampling_from_body(body: Dict[str, Any], tokenizer=None) -> SamplingParams:
    stop_ids = body.get("stop_token_ids") or ()
    return SamplingParams(max_tokens=int(body.get("max_tokens") or body.get("max_completion_tokens") or 16),
                          temperature=float(body.get("temperature", 1.0 if body.get("top_p") else 0.0) or 0.0),
                          top_k=int(body.get("top_k") or 0), top_p=float(body.get("top_p") or 1.0),
                          seed=body.get("seed"), ignore_eos=bool(body.get("ignore_eos", False)),
                          stop_token_ids=tuple(stop_ids),
                          presence_penalty=float(body.get("presence_penalty") or 0.0),
                          frequency_penalty=float(body.get("frequency_penalty") or 0.0),
                          repetition_penalty=float(body.get("repetition_penalty") or 1.0),
                          thinking_token_budget=body.get("thinking_token_budget"),
                          logprobs=_logprobs_from_body(body),
                          prompt_logprobs=(int(body["prompt_logprobs"]) if body.get("prompt_logprobs") is not None else None),
                          structured=structured_spec_from_body(body),
                          priority=int(body.get("priority") or 0), min_tokens=int(body.get("min_tokens") or 0),
                          min_p=float(body.get("min_p") or 0.0), allowed_token_ids=body.get("allowed_token_ids") or None,
                          bad_words_token_ids=bad_words_token_ids(body.get("bad_words"), tokenizer),
                          logit_bias={int(k): float(v) for k, v in (body.get("logit_bias") or {}).items()} or None)


def build_app(llm, tokenizer=None, model_name: str = "model", reasoning_parser=None, tool_parser=None):
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

    app = FastAPI()
    loop = EngineLoop(llm)
    loop.tokenizer = tokenizer
    app.state.engine_loop = loop

    def encode(prompt) -> List[int]:
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], int):
            return prompt
        if tokenizer is None:
            raise HTTPException(400, "this server has no tokenizer: send 'prompt' as a list of token ids")
        return tokenizer.encode(prompt)

    def decode(ids: List[int]) -> str:
        return tokenizer.decode(ids) if tokenizer is not None else ""

    @app.get("/health")
    def health():
        return {"status": "ok"}

    @app.post("/start_profile")
    async def start_profile():
        llm.start_profile()
        return {"status": "profiling"}

    @app.post("/stop_profile")
    async def stop_profile():
        llm.stop_profile()
        return {"status": "stopped"}

    @app.post("/sleep")
    async def sleep(level: int = 1):
        try:
            return {"status": "asleep", "released_bytes": llm.sleep(level)}
        except RuntimeError as e:
            return JSONResponse({"error": str(e)}, status_code=409)

    @app.post("/wake_up")
    async def wake_up():
        return {"status": "awake", "mapped_bytes": llm.wake_up()}

    @app.get("/ping")
    def ping():
        return PlainTextResponse("pong")

    @app.get("/version")
    def version():
        from .. import __version__ as v
        return {"version": v}

    @app.post("/tokenize")
    async def tokenize(body: Dict[str, Any]):
        """Token ids of ``prompt`` (or of ``messages`` through the chat template)."""
        if tokenizer is None:
            raise HTTPException(400, "this server has no tokenizer")
        if body.get("messages") is not None:
            if not hasattr(tokenizer, "apply_chat_template"):
                raise HTTPException(400, "the tokenizer has no chat template")
            ids = tokenizer.apply_chat_template(body["messages"], tokenize=True,
                                                add_generation_prompt=bool(body.get("add_generation_prompt", True)))
        else:
            ids = tokenizer.encode(body.get("prompt") or "")
        return {"tokens": list(ids), "count": len(ids), "max_model_len": llm.config.scheduler.max_model_len}

    @app.post("/detokenize")
    async def detokenize(body: Dict[str, Any]):
        if tokenizer is None:
            raise HTTPException(400, "this server has no tokenizer")
        return {"prompt": tokenizer.decode([int(t) for t in body.get("tokens") or []])}

    @app.get("/v1/models")
    def models():
        return {"object": "list", "data": [{"id": model_name, "object": "model"}]}

    @app.get("/metrics")
    def metrics():
        c, e = loop.counters, llm.engine.stats
        sch = llm.engine.scheduler
        lines = [f"omni_b200_requests_total {c['requests']}", f"omni_b200_requests_finished_total {c['finished']}",
                 f"omni_b200_output_tokens_total {c['output_tokens']}", f"omni_b200_engine_steps_total {e['steps']}",
                 f"omni_b200_prefill_steps_total {e.get('prefill_steps', 0)}",
                 f"omni_b200_decode_steps_total {e.get('decode_steps', 0)}",
                 f"omni_b200_spec_decode_steps_total {e.get('spec_decode_steps', 0)}",
                 f"omni_b200_running_requests {len(sch.running)}",
                 f"omni_b200_waiting_requests {len(sch.waiting)}",
                 f"omni_b200_kv_cache_usage {sch.pool.usage:.6f}",
                 f"omni_b200_kv_blocks_free {sch.pool.num_free}",
                 f"omni_b200_preemptions_total {sch.num_preemptions}",
                 f"omni_b200_prefix_cache_queries_total {sch.prefix_stats['requests']}",
                 f"omni_b200_prefix_cache_hit_tokens_total {sch.prefix_stats['hit_tokens']}",
                 f"omni_b200_spec_draft_tokens_total {sch.spec_stats['drafted']}",
                 f"omni_b200_spec_accepted_tokens_total {sch.spec_stats['accepted']}",
                 f"omni_b200_failed_steps_total {c.get('failed_steps', 0)}"]
        return PlainTextResponse("\n".join(lines) + "\n")

    def _submit(ids, body) -> str:
        stop = body.get("stop")
        stop = [stop] if isinstance(stop, str) else list(stop or [])
        try:
            return loop.submit(ids, sampling_from_body(body, tokenizer), body.get("kv_transfer_params"), stop=stop)
        except ValueError as e:
            raise HTTPException(400, str(e))

    def _text(out) -> str:
        """The answer's text: cut before a stop string when one ended the request."""
        cut = getattr(out, "text", None)
        return cut if cut is not None else decode(out.output_token_ids)

    async def _finish(rid: str):
        while True:
            out = await asyncio.to_thread(loop.wait, rid, 0.5)
            if out is not None:
                return out

    async def _stream(rid: str, make_chunk):
        slot = loop.waiters[rid]
        while True:
            await asyncio.sleep(0.005)
            with loop.lock:
                toks, slot["queue"] = slot["queue"], []
            if toks:
                yield "data: " + json.dumps(make_chunk(toks, None)) + "\n\n"
            if slot["event"].is_set():
                out = loop.wait(rid, 0)
                with loop.lock:
                    rest = slot["queue"]
                if rest:
                    yield "data: " + json.dumps(make_chunk(rest, None)) + "\n\n"
                yield "data: " + json.dumps(make_chunk([], out.finish_reason or "stop")) + "\n\n"
                yield "data: [DONE]\n\n"
                return

    def _n_choices(body) -> int:
        n = int(body.get("n") or 1)
        if n < 1 or n > 16:
            raise HTTPException(400, "n must be between 1 and 16")
        if n > 1 and body.get("stream"):
            raise HTTPException(400, "streaming answers one choice (n = 1)")
        return n

    def _completion_choice(index: int, out) -> Dict[str, Any]:
        lp = None
        if out.logprobs is not None:
            # the completions form: parallel lists over the output tokens
            lp = {"tokens": [decode([t]) if tokenizer is not None else str(t) for t in out.output_token_ids],
                  "token_ids": out.output_token_ids, "token_logprobs": [e[0] for e in out.logprobs],
                  "top_logprobs": [{(decode([i]) if tokenizer is not None else str(i)): v for i, v in e[1]}
                                   for e in out.logprobs]}
        if out.prompt_logprobs is not None:
            # one entry per prompt token: null for the first, else {token: log-probability} of the token and its alternatives
            name = (lambda i: decode([i])) if tokenizer is not None else str
            extra = {"prompt_logprobs": [None if e is None else {name(t): e[0], **{name(i): v for i, v in e[1]}}
                                         for t, e in zip(out.prompt_token_ids, out.prompt_logprobs)]}
        else:
            extra = {}
        return {**extra, "index": index, "text": _text(out), "token_ids": out.output_token_ids, "logprobs": lp,
                "finish_reason": out.finish_reason or "stop"}

    @app.post("/v1/completions")
    async def completions(body: Dict[str, Any]):
        ids = encode(body.get("prompt"))
        n = _n_choices(body)
        if n > 1:
            # n independent requests (each draws from its own default seed, or from seed + index)
            rids = [_submit(ids, dict(body, seed=body["seed"] + i) if body.get("seed") is not None else body)
                    for i in range(n)]
            outs = [await _finish(r) for r in rids]
            done = sum(len(o.output_token_ids) for o in outs)
            return JSONResponse({
                "id": rids[0], "object": "text_completion", "created": int(time.time()), "model": model_name,
                "choices": [_completion_choice(i, o) for i, o in enumerate(outs)],
                "usage": {"prompt_tokens": len(ids), "completion_tokens": done, "total_tokens": len(ids) + done}})
        rid = _submit(ids, body)
        created = int(time.time())
        if body.get("stream"):
            def chunk(toks, finish):
                return {"id": rid, "object": "text_completion", "created": created, "model": model_name,
                        "choices": [{"index": 0, "text": decode(toks), "token_ids": toks, "finish_reason": finish}]}
            return StreamingResponse(_stream(rid, chunk), media_type="text/event-stream")
        out = await _finish(rid)
        return JSONResponse({
            "id": rid, "object": "text_completion", "created": created, "model": model_name,
            "choices": [_completion_choice(0, out)],
            "usage": {"prompt_tokens": len(ids), "completion_tokens": len(out.output_token_ids),
                      "total_tokens": len(ids) + len(out.output_token_ids)},
            "kv_transfer_params": out.kv_transfer_params})

    @app.post("/v1/chat/completions")
    async def chat(body: Dict[str, Any]):
        msgs = body.get("messages") or []
        if tokenizer is not None and hasattr(tokenizer, "apply_chat_template"):
            ids = tokenizer.apply_chat_template(msgs, add_generation_prompt=True, tokenize=True)
        elif msgs and isinstance(msgs[-1].get("content"), list) and all(isinstance(t, int) for t in msgs[-1]["content"]):
            ids = msgs[-1]["content"]                      # token ids in the last message (no tokenizer)
        else:
            raise HTTPException(400, "chat needs a tokenizer with a chat template")
        rid = _submit(ids, body)
        if body.get("stream"):
            # chat.completion.chunk events: the role first, then the text of the new tokens as they
            # arrive (reasoning / tool-call parsing needs the whole text and applies to the plain answer)
            created = int(time.time())
            state = {"first": True}

            def chunk(toks, finish):
                delta: Dict[str, Any] = {"content": decode(toks)} if toks else {}
                if state["first"]:
                    delta["role"] = "assistant"
                    state["first"] = False
                return {"id": rid, "object": "chat.completion.chunk", "created": created, "model": model_name,
                        "choices": [{"index": 0, "delta": delta, "token_ids": toks, "finish_reason": finish}]}
            return StreamingResponse(_stream(rid, chunk), media_type="text/event-stream")
        out = await _finish(rid)
        text = _text(out)
        message: Dict[str, Any] = {"role": "assistant", "content": text}
        if reasoning_parser is not None:
            reasoning, content = reasoning_parser.extract_reasoning(text)
            message["reasoning_content"], message["content"] = reasoning, content
        if tool_parser is not None and body.get("tools"):
            info = tool_parser.extract_tool_calls(message["content"] or "")
            if getattr(info, "tools_called", False):
                import dataclasses
                message["tool_calls"] = [dataclasses.asdict(tc) if dataclasses.is_dataclass(tc) else tc
                                         for tc in info.tool_calls]
                message["content"] = info.content
        return JSONResponse({
            "id": rid, "object": "chat.completion", "created": int(time.time()), "model": model_name,
            "choices": [{"index": 0, "message": message, "finish_reason": out.finish_reason or "stop",
                         # the chat form: one entry per output token with its alternatives
                         "logprobs": None if out.logprobs is None else {"content": [
                             {"token": decode([t]) if tokenizer is not None else str(t), "token_id": t, "logprob": e[0],
                              "top_logprobs": [{"token": decode([i]) if tokenizer is not None else str(i),
                                                "token_id": i, "logprob": v} for i, v in e[1]]}
                             for t, e in zip(out.output_token_ids, out.logprobs)]}}],
            "usage": {"prompt_tokens": len(ids), "completion_tokens": len(out.output_token_ids),
                      "total_tokens": len(ids) + len(out.output_token_ids)}})

    return app


def make_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser("omni_npu_b200.serving.api_server")
    ap.add_argument("--model", default="llama-3-8b", help="preset name or HF directory")
    ap.add_argument("--served-model-name", default=None)
    ap.add_argument("--tokenizer", default=None, help="HF tokenizer directory (default: the model directory)")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--pipeline-parallel-size", type=int, default=1)
    ap.add_argument("--prefill-context-parallel-size", type=int, default=1,
                    help="split the tokens of prefill steps over this many ranks (grouped-query attention models)")
    ap.add_argument("--data-parallel-size", type=int, default=1)
    ap.add_argument("--enable-expert-parallel", action="store_true")
    ap.add_argument("--max-num-seqs", type=int, default=128)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--max-model-len", type=int, default=8192)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--enforce-eager", action="store_true")
    ap.add_argument("--no-enable-chunked-prefill", dest="enable_chunked_prefill", action="store_false")
    ap.add_argument("--scheduling-policy", default="fcfs", choices=["fcfs", "priority"],
                    help="priority: requests carry a 'priority' field, lower values first")
    ap.add_argument("--enable-prefix-caching", action="store_true",
                    help="reuse the KV blocks of a cached token prefix for new requests")
    ap.add_argument("--enable-mixed-batches", action="store_true",
                    help="decoding requests ride along in the prefill steps of other requests")
    ap.add_argument("--compilation-config", type=json.loads, default=None)
    ap.add_argument("--kv-transfer-config", type=json.loads, default=None)
    ap.add_argument("--speculative-config", type=json.loads, default=None)
    ap.add_argument("--additional-config", type=json.loads, default=None)
    ap.add_argument("--reasoning-parser", default=None)
    ap.add_argument("--tool-call-parser", default=None)
    ap.add_argument("--reasoning-config", type=json.loads, default=None)
    ap.add_argument("--enable-kv-rmsnorm-rope-cache", action="store_true", default=True)
    ap.add_argument("--load-format", default="auto")
    ap.add_argument("--seed", type=int, default=0)
    return ap


def main(argv=None) -> None:
    import os

    import uvicorn

    from ..engine.llm import LLM
    from .parsers import get_reasoning_parser, get_tool_parser
    args = make_parser().parse_args(argv)
    kw = dict(tensor_parallel_size=args.tensor_parallel_size, data_parallel_size=args.data_parallel_size,
              pipeline_parallel_size=args.pipeline_parallel_size,
              prefill_context_parallel_size=args.prefill_context_parallel_size,
              enable_expert_parallel=args.enable_expert_parallel, max_num_seqs=args.max_num_seqs,
              max_num_batched_tokens=args.max_num_batched_tokens, max_model_len=args.max_model_len,
              block_size=args.block_size, gpu_memory_utilization=args.gpu_memory_utilization,
              enforce_eager=args.enforce_eager, enable_chunked_prefill=args.enable_chunked_prefill,
              enable_mixed_batches=args.enable_mixed_batches,
              enable_prefix_caching=args.enable_prefix_caching, scheduling_policy=args.scheduling_policy,
              compilation_config=args.compilation_config, kv_transfer_config=args.kv_transfer_config,
              speculative_config=args.speculative_config, additional_config=args.additional_config,
              load_format=args.load_format, seed=args.seed)
    if args.reasoning_config:
        kw["additional_config"] = dict(kw["additional_config"] or {}, reasoning_config=args.reasoning_config)
    llm = LLM(model=args.model, **kw)
    tokenizer = None
    tok_dir = args.tokenizer or (args.model if os.path.isdir(args.model) else None)
    if tok_dir:
        try:
            from transformers import AutoTokenizer
            tokenizer = AutoTokenizer.from_pretrained(tok_dir)
        except Exception as e:
            logger.warning("no tokenizer loaded from %s (%s): token-id requests only", tok_dir, e)
    if tokenizer is not None:
        try:
            llm.enable_structured_outputs(tokenizer)        # on every rank: each one masks its own logits
        except Exception as e:
            logger.warning("structured outputs are off (%s)", e)
    if int(os.environ.get("RANK", "0")) != 0 and args.data_parallel_size == 1:
        EngineLoop(llm, follower=True).run_follower()       # requests arrive through rank 0
        return
    if args.data_parallel_size > 1:
        args.port += int(os.environ.get("RANK", "0"))      # one server per data-parallel rank: port + rank
    if args.reasoning_config and tokenizer is not None:
        # marker strings given instead of token ids: resolve them now that there is a tokenizer
        proc = llm.engine.worker.model_runner.thinking_processor
        if proc.cfg is not None and not proc.enabled:
            proc.cfg.initialize_token_ids(tokenizer)
            proc.__init__(proc.cfg, device=proc.device)
    rp = get_reasoning_parser(args.reasoning_parser)(tokenizer) if args.reasoning_parser and tokenizer else None
    tp = get_tool_parser(args.tool_call_parser)(tokenizer) if args.tool_call_parser and tokenizer else None
    app = build_app(llm, tokenizer, args.served_model_name or os.path.basename(str(args.model)), rp, tp)
    uvicorn.run(app, host=args.host, port=args.port, log_level="info")


if __name__ == "__main__":
    main()
