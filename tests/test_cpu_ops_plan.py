"""Host restatement of the balanced cut of the decode attention (ops.decode_balanced_plan): every
tile of every (sequence, kv head) item is covered exactly once, a CTA leaves at most two partial
pieces, and the slots that the merge kernel derives for an item are the ones the CTAs wrote."""
import random

import pytest

from omni_npu_b200 import ops


def _merge_slots(seq_lens, hk, ctas, b, kvh, tile=64):
    """What gqa_decode_merge_balanced_kernel computes for one item: None = a single CTA held it."""
    nb = [max(1, -(-n // tile)) for n in seq_lens]
    total = sum(nb) * hk
    per = max(2, -(-total // ctas))
    x0 = sum(nb[:b]) * hk + kvh * nb[b]
    c0, c1 = x0 // per, (x0 + nb[b] - 1) // per
    if c0 == c1:
        return None
    first = 2 * c0 + (0 if x0 == c0 * per else 1)
    return [first] + [2 * c for c in range(c0 + 1, c1 + 1)]


@pytest.mark.parametrize("seed", range(6))
def test_balanced_plan_covers_every_tile_once_and_matches_the_merge(seed):
    rng = random.Random(seed)
    n_seqs = rng.choice([1, 3, 40, 128, 300])
    hk = rng.choice([1, 2, 4, 8])
    ctas = rng.choice([7, 296, 444])
    seq_lens = [rng.choice([0, 1, 63, 64, 65, rng.randint(1, 5000)]) for _ in range(n_seqs)]
    plan = ops.decode_balanced_plan(seq_lens, hk, ctas)
    assert len(plan) == ctas
    covered = {}
    written = {}
    loads = []
    for c, segs in enumerate(plan):
        partial = [s for s in segs if s[4] >= 0]
        assert len(partial) <= 2
        assert len({s[4] for s in partial}) == len(partial)
        loads.append(sum(s[3] for s in segs))
        for i, (b, kvh, t, n, slot) in enumerate(segs):
            assert n >= 1 and 0 <= kvh < hk
            if slot >= 0:
                assert slot == 2 * c + (0 if i == 0 else 1)
                written.setdefault((b, kvh), []).append(slot)
            for tt in range(t, t + n):
                assert (b, kvh, tt) not in covered
                covered[(b, kvh, tt)] = c
    nb = [max(1, -(-n // 64)) for n in seq_lens]
    assert len(covered) == sum(nb) * hk
    assert max(loads) <= max(2, -(-sum(nb) * hk // ctas))
    for b in range(n_seqs):
        for kvh in range(hk):
            assert _merge_slots(seq_lens, hk, ctas, b, kvh) == written.get((b, kvh))


def test_only_plain_decode_sized_cluster_split_products_go_to_the_library(monkeypatch):
    assert ops.library_small_m(128, True, True)
    assert ops.library_small_m(64, True, True) and ops.library_small_m(256, True, True)
    assert not ops.library_small_m(32, True, True)        # small batches keep batch-invariant numerics
    assert not ops.library_small_m(8192, True, True)      # prefill
    assert not ops.library_small_m(128, False, True)      # gate_up, LM head: no cluster split-K plan
    assert not ops.library_small_m(128, True, False)      # bias / residual / SwiGLU / scales / forced tiles
    monkeypatch.setattr(ops, "SMALL_M_GEMM", "own")
    assert not ops.library_small_m(128, True, True)
