"""Requests, sampling parameters and per-request outputs."""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple


@dataclass
class SamplingParams:
    max_tokens: int = 16
    temperature: float = 0.0           # 0 = greedy
    top_k: int = 0                     # 0 / -1 = off
    top_p: float = 1.0
    seed: Optional[int] = None
    ignore_eos: bool = False
    stop_token_ids: Sequence[int] = ()
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    thinking_token_budget: Optional[int] = None
    logprobs: Optional[int] = None
    # log-probabilities of the prompt's own tokens (each given the tokens before it) with this many
    # most likely alternatives; 0 asks for the prompt tokens' values alone
    prompt_logprobs: Optional[int] = None
    # added to the logits of the named tokens before sampling ({token id: bias}, as in the OpenAI API)
    logit_bias: Optional[Dict[int, float]] = None
    # the end-of-sequence and stop tokens cannot be sampled before this many output tokens
    min_tokens: int = 0
    # tokens whose probability (after temperature) is below min_p x the largest one cannot be sampled
    min_p: float = 0.0
    # when given, only these tokens can be sampled
    allowed_token_ids: Optional[Sequence[int]] = None
    # token sequences that must not appear in the output: once the output ends with all but the last
    # token of one of them, that last token cannot be sampled
    bad_words_token_ids: Optional[Sequence[Sequence[int]]] = None
    # scheduling priority under SchedulerConfig.policy == "priority": lower values are admitted first
    # and preempted last (ties: earlier arrival first)
    priority: int = 0
    # structured output: {"choice": [...]} | {"json_schema": ...} | {"json_object": True} | {"regex": ...} |
    # {"grammar": ebnf} (sample/structured.py); needs a tokenizer given to the engine
    structured: Optional[Dict[str, Any]] = None
    extra_args: Dict[str, Any] = field(default_factory=dict)

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-5

    @property
    def has_penalties(self) -> bool:
        return (self.presence_penalty != 0.0 or self.frequency_penalty != 0.0
                or self.repetition_penalty != 1.0)


class RequestStatus(enum.IntEnum):
    WAITING = 0
    WAITING_FOR_REMOTE_KVS = 1
    RUNNING = 2
    PREEMPTED = 3
    FINISHED_STOPPED = 4
    FINISHED_LENGTH_CAPPED = 5
    FINISHED_ABORTED = 6

    @property
    def finished(self) -> bool:
        return self >= RequestStatus.FINISHED_STOPPED


class Request:
    __slots__ = ("request_id", "prompt_token_ids", "sampling_params", "output_token_ids", "status",
                 "block_ids", "num_computed_tokens", "arrival_time", "first_token_time",
                 "finish_time", "kv_transfer_params", "eos_token_id", "num_preemptions",
                 "spec_token_ids", "client_index", "num_external_tokens", "_block_hashes",
                 "_registered_blocks", "logprobs", "prompt_logprobs")

    def __init__(self, request_id: str, prompt_token_ids: Sequence[int],
                 sampling_params: Optional[SamplingParams] = None,
                 eos_token_id: Optional[int] = None, arrival_time: Optional[float] = None,
                 kv_transfer_params: Optional[Dict[str, Any]] = None) -> None:
        self.request_id = request_id
        self.prompt_token_ids: List[int] = list(prompt_token_ids)
        self.sampling_params = sampling_params or SamplingParams()
        self.output_token_ids: List[int] = []
        self.status = RequestStatus.WAITING
        self.block_ids: List[int] = []
        self.num_computed_tokens = 0
        self.arrival_time = time.monotonic() if arrival_time is None else arrival_time
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None
        self.kv_transfer_params = kv_transfer_params
        self.eos_token_id = eos_token_id
        self.num_preemptions = 0
        self.spec_token_ids: List[int] = []
        self.client_index = 0
        self.num_external_tokens = 0
        # prefix caching: content hashes of the full blocks hashed so far, and how many of this
        # request's blocks are registered with the pool under their hash
        self._block_hashes: Optional[List[bytes]] = None
        self._registered_blocks = 0
        # one entry per output token when sampling_params.logprobs is set:
        # (log-probability of the token, [(token id, log-probability), ...] of the most likely tokens)
        self.logprobs: List[Tuple[float, List[Tuple[int, float]]]] = []
        # one entry per prompt token when sampling_params.prompt_logprobs is set (None for the first
        # token, which has nothing before it), same shape as an entry of ``logprobs``
        self.prompt_logprobs: Optional[List[Optional[Tuple[float, List[Tuple[int, float]]]]]] = (
            [None] * len(self.prompt_token_ids) if self.sampling_params.prompt_logprobs is not None else None)

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def all_token_ids(self) -> List[int]:
        return self.prompt_token_ids + self.output_token_ids

    @property
    def is_finished(self) -> bool:
        return self.status.finished

    def token_at(self, i: int) -> int:
        n = len(self.prompt_token_ids)
        return self.prompt_token_ids[i] if i < n else self.output_token_ids[i - n]

    def append_output(self, token: int, now: Optional[float] = None) -> None:
        if not self.output_token_ids:
            self.first_token_time = time.monotonic() if now is None else now
        self.output_token_ids.append(int(token))

    def check_stop(self) -> bool:
        """Update status if the last token ends the request; returns finished."""
        sp = self.sampling_params
        last = self.output_token_ids[-1]
        if not sp.ignore_eos and self.eos_token_id is not None and last == self.eos_token_id:
            self.status = RequestStatus.FINISHED_STOPPED
        elif last in sp.stop_token_ids:
            self.status = RequestStatus.FINISHED_STOPPED
        elif len(self.output_token_ids) >= sp.max_tokens:
            self.status = RequestStatus.FINISHED_LENGTH_CAPPED
        if self.status.finished:
            self.finish_time = time.monotonic()
            return True
        return False


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: List[int]
    output_token_ids: List[int]
    finished: bool
    finish_reason: Optional[str] = None
    ttft: Optional[float] = None           # seconds from arrival to first token
    tpot: Optional[float] = None           # mean seconds per output token after the first
    kv_transfer_params: Optional[Dict[str, Any]] = None
    logprobs: Optional[List[Tuple[float, List[Tuple[int, float]]]]] = None    # per output token, when asked for
    text: Optional[str] = None             # decoded output, when a tokenizer is at hand
    prompt_logprobs: Optional[List[Optional[Tuple[float, List[Tuple[int, float]]]]]] = None   # per prompt token

    @classmethod
    def from_request(cls, r: Request) -> "RequestOutput":
        reason = None
        if r.status == RequestStatus.FINISHED_STOPPED:
            reason = "stop"
        elif r.status == RequestStatus.FINISHED_LENGTH_CAPPED:
            reason = "length"
        elif r.status == RequestStatus.FINISHED_ABORTED:
            reason = "abort"
        ttft = (r.first_token_time - r.arrival_time) if r.first_token_time is not None else None
        tpot = None
        if r.finish_time is not None and r.first_token_time is not None and len(r.output_token_ids) > 1:
            tpot = (r.finish_time - r.first_token_time) / (len(r.output_token_ids) - 1)
        return cls(r.request_id, list(r.prompt_token_ids), list(r.output_token_ids), r.is_finished,
                   reason, ttft, tpot, r.kv_transfer_params,
                   list(r.logprobs[: len(r.output_token_ids)]) if r.sampling_params.logprobs else None,
                   prompt_logprobs=list(r.prompt_logprobs) if r.prompt_logprobs is not None else None)
