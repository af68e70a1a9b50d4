"""Model check of the push all-reduce protocol on CPU threads.

The device kernel (csrc/comm/ll_protocol.cuh, allreduce_ll_kernel) is modelled operation by
operation with one Python thread per rank and NumPy buffers: data words double as flags
(a sentinel value means "not arrived"), the receive buffer has three slots used round robin
by epoch, a call re-arms the slot of the PREVIOUS call (all its readers are done: every rank
needed this rank's push of the current epoch to leave it) using the fill count it recorded.
Random delays reorder the ranks; message sizes change from call to call.  A rank that races a
full call ahead must never overwrite data a slower rank has not consumed, nor read stale data.
"""
import random
import threading
import time

import numpy as np

SENTINEL = np.float32(-1.2345e30)


class Rank(threading.Thread):
    def __init__(self, rank, world, recv, calls, results, errors, seed):
        super().__init__(daemon=True)
        self.rank, self.world, self.recv, self.calls = rank, world, recv, calls
        self.results, self.errors = results, errors
        self.rng = random.Random(seed)
        self.meta = [0, 0, 0, 0]          # epoch, fill count of slot 0..2

    def jitter(self):
        if self.rng.random() < 0.3:
            time.sleep(self.rng.random() * 0.002)

    def all_reduce(self, x):
        n = len(x)
        epoch = self.meta[0] + 1
        slot = epoch % 3
        for dst in range(self.world):                       # push: plain stores into every rank's buffer
            self.jitter()
            self.recv[dst][slot, self.rank, :n] = x
        out = np.zeros(n, np.float32)
        for src in range(self.world):                       # data-carried flags: wait per element
            deadline = time.time() + 5.0
            row = self.recv[self.rank][slot, src]
            while (row[:n] == SENTINEL).any():
                if time.time() > deadline:
                    raise TimeoutError(f"rank {self.rank} epoch {epoch}: source {src} never arrived")
                time.sleep(0)
            out += row[:n]
        prev = (epoch + 2) % 3                               # slot of the previous call
        self.recv[self.rank][prev, :, : self.meta[1 + prev]] = SENTINEL
        self.meta[1 + slot] = n
        self.meta[0] = epoch
        return out

    def run(self):
        try:
            for i, n in enumerate(self.calls):
                x = np.full(n, float(self.rank + 1) * (i + 1), np.float32)
                got = self.all_reduce(x)
                want = sum(float(r + 1) * (i + 1) for r in range(self.world))
                if not np.allclose(got, want):
                    raise AssertionError(f"rank {self.rank} call {i}: {got[:4]} != {want}")
                self.jitter()
            self.results[self.rank] = True
        except Exception as e:                               # pragma: no cover - reported by the test
            self.errors.append(e)


def _run(world, calls, seed):
    cap = max(calls)
    recv = [np.full((3, world, cap), SENTINEL, np.float32) for _ in range(world)]
    results, errors = {}, []
    ranks = [Rank(r, world, recv, calls, results, errors, seed * 31 + r) for r in range(world)]
    for t in ranks:
        t.start()
    for t in ranks:
        t.join(timeout=30)
    assert not errors, errors
    assert len(results) == world
    # at rest only the last call's slot holds data; the two other slots are armed again
    last = len(calls) % 3
    for r in range(world):
        for s in range(3):
            if s != last and s != (len(calls) + 2) % 3:
                assert (recv[r][s] == SENTINEL).all()


def test_push_all_reduce_protocol_with_racing_ranks():
    rng = random.Random(0)
    for seed in range(4):
        calls = [rng.choice([1, 7, 64, 200]) for _ in range(40)]
        _run(world=2 + seed % 3, calls=calls, seed=seed)


def test_small_call_after_large_call_rearms_the_large_fill():
    _run(world=3, calls=[200, 3, 200, 1, 1, 1, 200], seed=9)
