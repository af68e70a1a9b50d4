"""Persistent per-request rows and per-step input staging.

Each running request owns a row of host-side numpy arrays (block table, number
of computed tokens, sampling parameters).  A step's device inputs are built with
vectorised numpy operations into ONE pinned int32 staging buffer laid out as

    [ input_ids | positions | slot_mapping | seq_lens | cu_q | temperature(f32 bits)
      | top_k | top_p(f32 bits) | block_table rows ]

and shipped with a single host-to-device copy.  For every CUDA-graph batch size
the section offsets are fixed, so the captured graph reads the same device
addresses at every replay.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..engine.request import Request


@dataclass
class StepLayout:
    """Offsets (in int32 elements) of each section for a given (tokens, seqs) capacity."""
    T: int
    S: int
    max_blocks: int
    ids: int = 0
    pos: int = 0
    slot: int = 0
    seq_lens: int = 0
    cu_q: int = 0
    temp: int = 0
    top_k: int = 0
    top_p: int = 0
    seeds: int = 0
    logits_idx: int = 0
    next_ids: int = 0
    bt: int = 0
    total: int = 0

    @classmethod
    def make(cls, T: int, S: int, max_blocks: int) -> "StepLayout":
        lay = cls(T, S, max_blocks)
        off = 0
        for name, n in (("ids", T), ("pos", T), ("slot", T), ("seq_lens", S), ("cu_q", S + 1),
                        ("temp", S), ("top_k", S), ("top_p", S), ("seeds", 2 * S),
                        ("logits_idx", S), ("next_ids", T), ("bt", S * max_blocks)):
            off = (off + 3) // 4 * 4           # 16-byte aligned sections
            setattr(lay, name, off)
            off += n
        lay.total = (off + 3) // 4 * 4
        return lay


def default_seed(request_id: str, base_seed: int = 0) -> int:
    """Sampling seed of a request that gave none.  Tensor-parallel ranks are separate processes
    and each samples on its own, so the value must not depend on the process: Python's ``hash``
    of a string is salted per process, a CRC of the request id (mixed with the engine seed) is
    the same everywhere."""
    import zlib
    data = request_id.encode("utf-8")
    lo = zlib.crc32(data)
    hi = zlib.crc32(data[::-1] + b"#", base_seed & 0xFFFFFFFF)
    return ((hi << 32) | lo) & 0x7FFFFFFFFFFFFFFF


class InputBatch:
    def __init__(self, max_num_seqs: int, max_model_len: int, block_size: int,
                 max_num_batched_tokens: int, device: torch.device, cp_world: int = 1, cp_rank: int = 0) -> None:
        self.max_num_seqs = max_num_seqs
        self.block_size = block_size
        # decode context parallelism: token p of a sequence is stored on rank p % cp_world at local
        # position p // cp_world; other ranks get slot -1 for it (the cache-write kernels skip those)
        self.cp_world, self.cp_rank = max(1, cp_world), cp_rank
        self.max_blocks = (max_model_len + block_size * self.cp_world - 1) // (block_size * self.cp_world)
        self.device = device
        self.num_rows = 0
        self.rows: List[Optional[Request]] = [None] * max_num_seqs
        self.row_of: Dict[str, int] = {}
        self.block_table = np.zeros((max_num_seqs, self.max_blocks), dtype=np.int32)
        self.num_blocks = np.zeros(max_num_seqs, dtype=np.int32)
        self.temperature = np.zeros(max_num_seqs, dtype=np.float32)
        self.top_k = np.zeros(max_num_seqs, dtype=np.int32)
        self.top_p = np.ones(max_num_seqs, dtype=np.float32)
        self.seeds = np.zeros(max_num_seqs, dtype=np.int64)
        self.base_seed = 0              # engine seed, mixed into the default per-request seeds
        cap_T = max(max_num_batched_tokens, max_num_seqs)
        self.capacity = StepLayout.make(cap_T, max_num_seqs, self.max_blocks)
        pin = device.type == "cuda"
        self.host = torch.zeros(self.capacity.total, dtype=torch.int32, pin_memory=pin)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.capacity.total, dtype=torch.int32, device=device)
        self.h2d_bytes_last = 0
        self._upload_event = None
        self._upload_pending = False

    # ------------------------------------------------------------------ rows
    def add_request(self, req: Request) -> int:
        row = self.row_of.get(req.request_id)
        if row is None:
            row = self.num_rows
            if row >= self.max_num_seqs:
                raise RuntimeError("input batch is full")
            self.num_rows += 1
            self.rows[row] = req
            self.row_of[req.request_id] = row
            self.num_blocks[row] = 0
            sp = req.sampling_params
            self.temperature[row] = sp.temperature
            self.top_k[row] = sp.top_k if sp.top_k and sp.top_k > 0 else 0
            self.top_p[row] = sp.top_p
            self.seeds[row] = sp.seed if sp.seed is not None else default_seed(req.request_id, self.base_seed)
        self.sync_blocks(row, req)
        return row

    def sync_blocks(self, row: int, req: Request) -> None:
        have, want = int(self.num_blocks[row]), len(req.block_ids)
        if want > have:
            self.block_table[row, have:want] = req.block_ids[have:want]
            self.num_blocks[row] = want
        elif want < have:                        # request was preempted and re-admitted
            self.block_table[row, :want] = req.block_ids
            self.num_blocks[row] = want

    def remove_request(self, request_id: str) -> None:
        row = self.row_of.pop(request_id, None)
        if row is None:
            return
        last = self.num_rows - 1
        if row != last:
            moved = self.rows[last]
            self.rows[row] = moved
            self.row_of[moved.request_id] = row
            self.block_table[row] = self.block_table[last]
            for arr in (self.num_blocks, self.temperature, self.top_k, self.top_p, self.seeds):
                arr[row] = arr[last]
        self.rows[last] = None
        self.num_rows = last

    # ----------------------------------------------------------------- staging
    def layout_for(self, T: int, S: int) -> StepLayout:
        return StepLayout.make(T, S, self.max_blocks)

    def views(self, lay: StepLayout, buf: torch.Tensor) -> Dict[str, torch.Tensor]:
        """Typed views into ``buf`` (host or device) for a layout."""
        T, S, mb = lay.T, lay.S, lay.max_blocks
        return {
            "ids": buf[lay.ids: lay.ids + T],
            "pos": buf[lay.pos: lay.pos + T],
            "slot": buf[lay.slot: lay.slot + T],
            "seq_lens": buf[lay.seq_lens: lay.seq_lens + S],
            "cu_q": buf[lay.cu_q: lay.cu_q + S + 1],
            "temp": buf[lay.temp: lay.temp + S].view(torch.float32),
            "top_k": buf[lay.top_k: lay.top_k + S],
            "top_p": buf[lay.top_p: lay.top_p + S].view(torch.float32),
            "seeds": buf[lay.seeds: lay.seeds + 2 * S].view(torch.int64),
            "logits_idx": buf[lay.logits_idx: lay.logits_idx + S],
            "next_ids": buf[lay.next_ids: lay.next_ids + T],
            "bt": buf[lay.bt: lay.bt + S * mb].view(S, mb),
        }

    def _slots(self, row, pos: np.ndarray) -> np.ndarray:
        """Cache slots of positions ``pos`` of the request(s) in ``row`` (an index or an index array
        matching ``pos``)."""
        bs = self.block_size
        if self.cp_world == 1:
            return self.block_table[row, pos // bs] * bs + pos % bs
        lp = pos // self.cp_world
        slot = self.block_table[row, lp // bs] * bs + lp % bs
        return np.where(pos % self.cp_world == self.cp_rank, slot, -1).astype(np.int32)

    def upload(self, lay: StepLayout) -> None:
        """One H2D copy of the staged step (pinned host -> device).  The copy is asynchronous:
        the staging buffer must not be rewritten until it has run (``wait_upload``)."""
        self.dev[: lay.total].copy_(self.host[: lay.total], non_blocking=True)
        self.h2d_bytes_last = lay.total * 4
        if self.device.type == "cuda":
            if self._upload_event is None:
                self._upload_event = torch.cuda.Event()
            self._upload_event.record()
            self._upload_pending = True

    def wait_upload(self) -> None:
        """Block until the last ``upload`` has read the staging buffer.  Every ``stage_*`` call
        starts with it: with a long queue ahead of the copy (for instance the zero-fill of a large
        KV cache right before the warm-up steps) the host would otherwise overwrite the buffer
        before the device has copied it, and the earlier step would run on the later step's
        inputs."""
        if self._upload_pending:
            self._upload_event.synchronize()
            self._upload_pending = False

    def _fill_sampling(self, lay: StepLayout, rows: np.ndarray, n: int, token_index=None) -> None:
        """Sampling parameters of the step's rows.  The random stream of a row is keyed by the
        request's seed mixed with the index of the token being sampled (``token_index``: output tokens
        the request has so far), so a seeded request draws the same tokens whenever it runs and
        whatever else the engine has done."""
        h = self.host_np
        h[lay.temp: lay.temp + n] = self.temperature[rows].view(np.int32)
        h[lay.top_k: lay.top_k + n] = self.top_k[rows]
        h[lay.top_p: lay.top_p + n] = self.top_p[rows].view(np.int32)
        seeds = self.seeds[rows]
        if token_index is not None and n:
            idx = np.asarray(token_index, dtype=np.uint64) + np.uint64(1)
            with np.errstate(over="ignore"):
                seeds = ((seeds.astype(np.uint64) + idx * np.uint64(0x9E3779B97F4A7C15))
                         & np.uint64(0x7FFFFFFFFFFFFFFF)).astype(np.int64)
        h[lay.seeds: lay.seeds + 2 * n] = seeds.view(np.int32)
        if lay.S > n:
            h[lay.temp + n: lay.temp + lay.S] = 0
            h[lay.top_k + n: lay.top_k + lay.S] = 0
            h[lay.top_p + n: lay.top_p + lay.S] = np.float32(1.0).view(np.int32)

    def stage_decode(self, lay: StepLayout, reqs: Sequence[Request], q_len: int = 1) -> np.ndarray:
        """Stage a decode step for ``reqs`` (one new token each) padded to lay.S
        sequences.  Returns the row indices used."""
        self.wait_upload()
        n = len(reqs)
        bs = self.block_size
        h = self.host_np
        rows = np.fromiter((self.row_of[r.request_id] for r in reqs), dtype=np.int64, count=n)
        for r, row in zip(reqs, rows):
            if len(r.block_ids) != self.num_blocks[row]:
                self.sync_blocks(int(row), r)
        pos = np.fromiter((r.num_tokens - 1 for r in reqs), dtype=np.int32, count=n)
        ids = np.fromiter((r.output_token_ids[-1] if r.output_token_ids else r.prompt_token_ids[-1]
                           for r in reqs), dtype=np.int32, count=n)
        h[lay.ids: lay.ids + n] = ids
        h[lay.pos: lay.pos + n] = pos
        h[lay.slot: lay.slot + n] = self._slots(rows, pos)
        h[lay.seq_lens: lay.seq_lens + n] = pos + 1
        if lay.S > n:
            # padded sequences: length 1 over block 0, results discarded
            h[lay.ids + n: lay.ids + lay.T] = 0
            h[lay.pos + n: lay.pos + lay.T] = 0
            h[lay.slot + n: lay.slot + lay.T] = -1
            h[lay.seq_lens + n: lay.seq_lens + lay.S] = 1
        h[lay.cu_q: lay.cu_q + lay.S + 1] = np.arange(lay.S + 1, dtype=np.int32) * q_len
        h[lay.logits_idx: lay.logits_idx + lay.S] = np.arange(lay.S, dtype=np.int32)
        h[lay.next_ids: lay.next_ids + lay.T] = -1
        self._fill_sampling(lay, rows, n, [len(r.output_token_ids) for r in reqs])
        bt = h[lay.bt: lay.bt + lay.S * lay.max_blocks].reshape(lay.S, lay.max_blocks)
        bt[:n] = self.block_table[rows]
        if lay.S > n:
            bt[n:] = 0
        return rows

    def stage_spec_decode(self, lay: StepLayout, seqs) -> Tuple[np.ndarray, int]:
        """Stage a verification step: every sequence feeds its last token followed by its
        draft tokens (ScheduledSeq.spec_token_ids) at positions start .. start + k.
        Returns (rows, max_q_len)."""
        self.wait_upload()
        h = self.host_np
        bs = self.block_size
        n = len(seqs)
        rows = np.empty(n, dtype=np.int64)
        off = 0
        max_q = 0
        cu = h[lay.cu_q: lay.cu_q + n + 1]
        cu[0] = 0
        for i, s in enumerate(seqs):
            req = s.request
            row = self.add_request(req)
            rows[i] = row
            q = 1 + len(s.spec_token_ids)
            max_q = max(max_q, q)
            last = req.output_token_ids[-1] if req.output_token_ids else req.prompt_token_ids[-1]
            h[lay.ids + off] = last
            if q > 1:
                h[lay.ids + off + 1: lay.ids + off + q] = s.spec_token_ids
            p = np.arange(s.start, s.start + q, dtype=np.int32)
            h[lay.pos + off: lay.pos + off + q] = p
            h[lay.slot + off: lay.slot + off + q] = self._slots(row, p)
            h[lay.seq_lens + i] = s.start + q
            off += q
            cu[i + 1] = off
            h[lay.logits_idx + i] = off - 1
        self._fill_sampling(lay, rows, n, [len(s.request.output_token_ids) for s in seqs])
        bt = h[lay.bt: lay.bt + lay.S * lay.max_blocks].reshape(lay.S, lay.max_blocks)
        bt[:n] = self.block_table[rows]
        # successor of fed token j of sequence i = element (i, j) of the [n, max_q] matrix of
        # verified tokens the step produces (staged as a flat index into that matrix)
        off = 0
        for i, s in enumerate(seqs):
            q = 1 + len(s.spec_token_ids)
            h[lay.next_ids + off: lay.next_ids + off + q] = i * max_q + np.arange(q, dtype=np.int32)
            off += q
        return rows, max_q

    def stage_prefill(self, lay: StepLayout, seqs) -> Tuple[np.ndarray, int]:
        """Stage a prefill step.  ``seqs`` are ScheduledSeq (request, start,
        num_new_tokens).  Returns (rows, max_q_len)."""
        self.wait_upload()
        h = self.host_np
        bs = self.block_size
        n = len(seqs)
        rows = np.empty(n, dtype=np.int64)
        off = 0
        max_q = 0
        cu = h[lay.cu_q: lay.cu_q + n + 1]
        cu[0] = 0
        for i, s in enumerate(seqs):
            req = s.request
            row = self.add_request(req)
            rows[i] = row
            q = s.num_new_tokens
            max_q = max(max_q, q)
            toks = req.prompt_token_ids[s.start: s.start + q]
            if len(toks) < q:                     # recomputation after preemption reaches into outputs
                toks = req.all_token_ids[s.start: s.start + q]
            h[lay.ids + off: lay.ids + off + q] = toks
            p = np.arange(s.start, s.start + q, dtype=np.int32)
            h[lay.pos + off: lay.pos + off + q] = p
            h[lay.slot + off: lay.slot + off + q] = self._slots(row, p)
            h[lay.seq_lens + i] = s.start + q
            # successors inside the chunk, then the token after it if the request already has it
            h[lay.next_ids + off: lay.next_ids + off + q - 1] = toks[1:]
            nxt = s.start + q
            h[lay.next_ids + off + q - 1] = req.token_at(nxt) if nxt < req.num_tokens else -1
            off += q
            cu[i + 1] = off
            h[lay.logits_idx + i] = off - 1
        self._fill_sampling(lay, rows, n, [len(s.request.output_token_ids) for s in seqs])
        bt = h[lay.bt: lay.bt + lay.S * lay.max_blocks].reshape(lay.S, lay.max_blocks)
        bt[:n] = self.block_table[rows]
        return rows, max_q
