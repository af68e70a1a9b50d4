"""Device-resident sampler state: penalty cache, draft-probability cache, sparse rejection sampling."""
import torch

from omni_npu_b200.sample.rejection_sampler import SparseRejectionSampler
from omni_npu_b200.sample.sampler import apply_penalties
from omni_npu_b200.sample.sampler_cache import PenaltyCache, ProbCache


def _dense_state(prompt, outputs, v):
    pm = torch.zeros(v, dtype=torch.bool)
    pm[torch.tensor(prompt)] = True
    cnt = torch.zeros(v)
    for t in outputs:
        cnt[t] += 1
    return pm, cnt


def test_penalty_cache_tracks_requests_incrementally_and_by_stable_slots():
    v = 32
    pc = PenaltyCache(4, v, "cpu")
    hist = {"a": ([1, 2, 3], [5, 5, 7]), "b": ([9], []), "c": ([4, 4, 30], [4])}
    for rid, (prompt, _) in hist.items():
        pc.add_request(rid, prompt)
    for rid, (_, outs) in hist.items():
        pc.sync_from_history(rid, outs)
    # one more step: only the new token is added
    hist["a"][1].append(7)
    hist["b"][1].append(9)
    pc.sync_from_history("a", hist["a"][1])
    pc.record(pc.slot_index(["b"]), torch.tensor([9]))
    pc.synced["b"] = 1
    logits = torch.randn(3, v)
    order = ["c", "a", "b"]                                   # batch order differs from admission order
    pres, freq, rep = torch.tensor([0.5, 0.0, 1.0]), torch.tensor([0.1, 0.7, 0.0]), torch.tensor([1.3, 1.0, 2.0])
    got = pc.apply(logits, pc.slot_index(order), pres, freq, rep)
    pm = torch.stack([_dense_state(*hist[r], v)[0] for r in order])
    cnt = torch.stack([_dense_state(*hist[r], v)[1] for r in order])
    assert torch.allclose(got, apply_penalties(logits, pm, cnt, pres, freq, rep))
    # a finished request frees its slot; the next one starts clean in it
    pc.remove_request("a")
    s = pc.add_request("d", [0])
    assert int(pc.output_counts[s].sum()) == 0 and pc.prompt_mask[s].nonzero().flatten().tolist() == [0]
    # rejected draft tokens are taken back
    slots = pc.slot_index(["c"])
    before = pc.output_counts[slots[0]].clone()
    toks = torch.tensor([[11, 12]])
    pc.record(slots, toks[:, 0])
    pc.record(slots, toks[:, 1])
    pc.revert(slots, toks, torch.tensor([[True, False]]))
    after = pc.output_counts[slots[0]]
    assert int(after[11] - before[11]) == 1 and int(after[12] - before[12]) == 0
    # a recomputed request (history shorter than what was counted) is rebuilt from its list
    pc.synced["c"] = 3                                       # [4] plus the two recorded above
    pc.sync_from_history("c", [4])
    assert int(pc.output_counts[slots[0]].sum()) == 1


def test_sparse_rejection_sampling_keeps_the_target_distribution():
    """Drafts drawn from the top-3 of a draft distribution that differs from the target: the
    first emitted token must follow the target distribution, and acceptance must actually happen."""
    torch.manual_seed(0)
    v, k, b = 8, 3, 200000
    target = torch.tensor([0.30, 0.05, 0.20, 0.10, 0.15, 0.02, 0.08, 0.10])
    draft = torch.tensor([0.10, 0.40, 0.25, 0.05, 0.05, 0.05, 0.05, 0.05])
    pc = ProbCache(b, 1, k, "cpu")
    for i in range(b):
        pc.slots.slot_of[str(i)] = i
    slots = torch.arange(b)
    drafted = pc.update(slots, 0, draft.expand(b, v))
    assert set(drafted.unique().tolist()) <= {1, 2, 0}          # the top-3 of the draft distribution
    bonus = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 1.0])
    probs = torch.stack([target, bonus]).expand(b, 2, v)
    out, num = SparseRejectionSampler(pc)(probs, slots)
    emp = torch.bincount(out[:, 0], minlength=v).float() / b
    assert torch.allclose(emp, target, atol=4e-3), emp
    acc = (num == 2)
    assert 0.2 < acc.float().mean() < 0.9
    assert bool((out[acc, 1] == 7).all()) and bool((out[~acc, 1] == -1).all())
    # rows without a computed draft distribution reject their drafts and still sample the target
    pc.computed[: b // 2] = False
    out2, num2 = SparseRejectionSampler(pc)(probs, slots)
    assert bool((num2[: b // 2] == 1).all())
    emp2 = torch.bincount(out2[: b // 2, 0], minlength=v).float() / (b // 2)
    assert torch.allclose(emp2, target, atol=6e-3), emp2
