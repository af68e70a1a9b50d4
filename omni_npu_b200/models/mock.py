"""Mock models: run the serving stack without (or around) the real network.

``mock_model_class_factory(base)`` derives a class from any model class of this package
and overrides ``forward`` / ``compute_logits`` / ``load_weights`` according to
environment switches (read once, at construction):

``RANDOM_MODE=1``            skip the network: hidden states are a cheap deterministic
                             function of (token, position), logits come from the real LM
                             head (or are pseudo-random with ``MOCK_COMPUTE_LOGITS=1``);
``CAPTURE_MODE=1``           run the real network and record, for every sequence prefix
                             that produced logits, the top tokens and their logits into
                             ``$MOCK_CAPTURE_DIR/$MOCK_CAPTURE_FILE.json`` (file-locked, so
                             several ranks / instances can share it);
``REPLAY_MODE=1``            do not run the network; answer every prefix from the capture
                             file (unknown prefixes fall back to random mode);
``KV_CACHE_MODE=1``          with replay: also fill the KV-cache slots of the step with
                             pseudo-random values, so a prefill instance has "KV" to ship
                             to a decode instance in PD-disaggregation tests;
``FORWARD_TIME=<ms>`` /      sleep this long per forward pass, or as long as the captured
``SIMULATE_ELAPSED_TIME=1``  run took (never inside CUDA-graph capture);
``PREFILL_PROCESS=1``        this instance is the prefill side (suffix ``p`` on the file).

The prefix of a sequence is tracked from the step inputs alone (token ids, query
offsets, block tables), keyed by the first KV block of the sequence, which is unique
while the request lives.

Same purpose and switches as the reference's capture/replay mock
(omni_npu/v1/models/mock/mock.py:92-260,1112-1337); ``NO_NPU_MOCK`` there corresponds
to simply running this package with ``device="cpu"``.
"""
from __future__ import annotations

import hashlib
import json
import os
import time
from typing import Dict, List, Optional

import torch

from ..attention.metadata import get_forward_context
from ..logger import logger

_TOPN = 4


def _env_int(name: str, default: int = 0) -> int:
    try:
        return int(os.getenv(name, str(default)))
    except ValueError:
        return default


def _prefix_key(tokens: List[int]) -> str:
    h = hashlib.sha1()
    h.update(len(tokens).to_bytes(4, "little"))
    h.update(b"".join(int(t).to_bytes(4, "little", signed=True) for t in tokens))
    return h.hexdigest()


class MockModel:
    """Marker base of every class made by :func:`mock_model_class_factory`."""


def mock_model_class_factory(base_class: type) -> type:
    class Mock(base_class, MockModel):  # type: ignore[misc, valid-type]
        def __init__(self, engine_config, device=None) -> None:
            super().__init__(engine_config, device)
            self.random_mode = _env_int("RANDOM_MODE")
            self.capture_mode = _env_int("CAPTURE_MODE")
            self.replay_mode = _env_int("REPLAY_MODE")
            self.kv_cache_mode = _env_int("KV_CACHE_MODE")
            self.prefill_process = _env_int("PREFILL_PROCESS")
            self.forward_time_ms = _env_int("FORWARD_TIME")
            self.simulate_elapsed_time = _env_int("SIMULATE_ELAPSED_TIME")
            self.mock_compute_logits = _env_int("MOCK_COMPUTE_LOGITS", 0)
            cap_dir = os.getenv("MOCK_CAPTURE_DIR", "./mock_capture")
            name = os.getenv("MOCK_CAPTURE_FILE", "mock_cache") + ("p" if self.prefill_process else "")
            self.capture_path = os.path.join(cap_dir, name + ".json")
            self.lock_path = os.path.join(cap_dir, os.getenv("MOCK_CAPTURE_FILE_LOCK", ".lock"))
            self.records: Dict[str, dict] = {}
            self._history: Dict[int, List[int]] = {}        # first block id -> token prefix
            self._pending_keys: List[Optional[str]] = []
            self._pending_elapsed = 0.0
            self.base_forward_calls = 0
            if self.capture_mode and self.replay_mode:
                raise ValueError("CAPTURE_MODE and REPLAY_MODE are mutually exclusive")
            if self.capture_mode or self.replay_mode:
                os.makedirs(cap_dir, exist_ok=True)
            if self.replay_mode:
                self._read_records()
                logger.info("mock model: replaying %d recorded prefixes from %s", len(self.records),
                            self.capture_path)

        # ---------------------------------------------------------------- files
        def _read_records(self) -> None:
            if os.path.exists(self.capture_path):
                with open(self.capture_path) as f:
                    self.records = json.load(f)

        def _flush_records(self, new: Dict[str, dict]) -> None:
            from filelock import FileLock
            with FileLock(self.lock_path):
                merged = {}
                if os.path.exists(self.capture_path):
                    with open(self.capture_path) as f:
                        merged = json.load(f)
                merged.update(new)
                tmp = self.capture_path + ".tmp"
                with open(tmp, "w") as f:
                    json.dump(merged, f)
                os.replace(tmp, self.capture_path)

        # ------------------------------------------------------------- prefixes
        def _track(self, input_ids: torch.Tensor, md) -> List[Optional[str]]:
            """Extend the per-sequence token prefixes with this step's inputs; returns the
            prefix key of every sequence (None for padded rows of a graph batch)."""
            n = md.num_actual_seqs if md.num_actual_seqs is not None else md.num_seqs
            ids = input_ids.tolist()
            if md.is_prefill:
                cu = md.cu_q[: md.num_seqs + 1].tolist()
            else:
                q = max(1, md.q_len)
                cu = [i * q for i in range(md.num_seqs + 1)]
            lens = md.seq_lens[: md.num_seqs].tolist()
            first_blocks = md.block_tables[: md.num_seqs, 0].tolist()
            keys: List[Optional[str]] = []
            for b in range(md.num_seqs):
                if b >= n:
                    keys.append(None)
                    continue
                new = ids[cu[b]: cu[b + 1]]
                start = lens[b] - len(new)
                hist = self._history.get(first_blocks[b])
                if hist is None or start == 0 or len(hist) < start:
                    hist = [] if start == 0 else [-1] * start      # unknown earlier tokens (e.g. remote KV)
                hist = hist[:start] + new
                self._history[first_blocks[b]] = hist
                keys.append(_prefix_key(hist))
            return keys

        # --------------------------------------------------------------- forward
        def _cheap_hidden(self, input_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
            h = self.config.hidden_size
            base = (input_ids.to(torch.float32) * 0.013 + positions.to(torch.float32) * 0.007).unsqueeze(1)
            ramp = torch.arange(h, device=input_ids.device, dtype=torch.float32).unsqueeze(0)
            return torch.sin(base * (1.0 + ramp * 0.01)).to(self.config.dtype)

        def _fill_kv(self, md, kv_caches) -> None:
            slots = md.slot_mapping[: md.num_tokens].long()
            slots = slots[slots >= 0]
            if slots.numel() == 0:
                return
            for cache in kv_caches:
                for t in (cache if isinstance(cache, (tuple, list)) else (cache,)):
                    flat = t.view(-1, *t.shape[2:]) if t.dim() >= 3 else t
                    vals = torch.sin(slots.to(torch.float32)).view(-1, *([1] * (flat.dim() - 1)))
                    flat[slots] = vals.to(flat.dtype).expand(-1, *flat.shape[1:])

        def forward(self, input_ids, positions, inputs_embeds=None):
            capturing = input_ids.is_cuda and torch.cuda.is_current_stream_capturing()
            ctx = get_forward_context()
            md = ctx.attn_metadata if ctx is not None else None
            track = (self.capture_mode or self.replay_mode) and md is not None and not capturing
            self._pending_keys = self._track(input_ids, md) if track else []
            t0 = time.perf_counter()
            if self.random_mode or self.replay_mode:
                hidden = self._cheap_hidden(input_ids, positions)
                if self.kv_cache_mode and md is not None and ctx.kv_caches:
                    self._fill_kv(md, ctx.kv_caches)
            else:
                self.base_forward_calls += 1
                hidden = super().forward(input_ids, positions, inputs_embeds)
            if not capturing:
                if self.capture_mode and input_ids.is_cuda:
                    torch.cuda.synchronize()
                self._pending_elapsed = time.perf_counter() - t0
                wait = self.forward_time_ms / 1e3
                if self.replay_mode and self.simulate_elapsed_time and self._pending_keys:
                    rec = [self.records.get(k) for k in self._pending_keys if k]
                    wait = max([r.get("elapsed", 0.0) for r in rec if r] or [wait])
                if wait > 0:
                    time.sleep(wait)
            return hidden

        def compute_logits(self, hidden):
            keys = self._pending_keys
            if self.replay_mode and keys:
                logits = torch.full((hidden.shape[0], self.config.vocab_size), -30.0, dtype=torch.float32,
                                    device=hidden.device)
                for row, key in enumerate(keys[: hidden.shape[0]]):
                    rec = self.records.get(key) if key else None
                    if rec is None:
                        logits[row, (row * 7919 + 13) % self.config.vocab_size] = 0.0
                        continue
                    idx = torch.tensor(rec["ids"], device=hidden.device)
                    logits[row, idx] = torch.tensor(rec["logits"], dtype=torch.float32, device=hidden.device)
                return logits
            if self.mock_compute_logits:
                v = self.config.vocab_size
                ramp = torch.arange(v, device=hidden.device, dtype=torch.float32).unsqueeze(0)
                return torch.sin(hidden[:, :1].float() * 50.0 + ramp * 0.37)
            logits = super().compute_logits(hidden)
            if self.capture_mode and keys:
                top = torch.topk(logits.float(), _TOPN, dim=-1)
                vals, ids = top.values.tolist(), top.indices.tolist()
                new = {}
                for row, key in enumerate(keys[: logits.shape[0]]):
                    if key:
                        new[key] = {"ids": ids[row], "logits": vals[row], "elapsed": self._pending_elapsed}
                if new:
                    self.records.update(new)
                    self._flush_records(new)
            return logits

        def load_weights(self, weights):
            if self.random_mode or self.replay_mode:
                return set()            # nothing of the checkpoint is needed
            return super().load_weights(weights)

    Mock.__name__ = "Mock" + base_class.__name__
    Mock.__qualname__ = Mock.__name__
    return Mock


def _default_base():
    from .llama import LlamaForCausalLM
    return LlamaForCausalLM


class _LazyMock:
    """``MockModelForCausalLM`` resolves its base on first use so that importing this
    module does not import every model family."""
    _cls = None

    def __call__(self, engine_config, device=None):
        if _LazyMock._cls is None:
            base = os.getenv("MOCK_BASE_ARCH")
            if base:
                from .registry import resolve_model_cls
                _LazyMock._cls = mock_model_class_factory(resolve_model_cls(base))
            else:
                _LazyMock._cls = mock_model_class_factory(_default_base())
        return _LazyMock._cls(engine_config, device)


MockModelForCausalLM = _LazyMock()
