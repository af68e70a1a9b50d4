"""Sampler semantics on CPU: greedy rows, top-k / top-p support sets, distribution of the
exponential-race sampler, penalties."""
import torch

from omni_npu_b200.ops import ref
from omni_npu_b200.sample.sampler import Sampler, apply_penalties


def test_zero_temperature_rows_are_greedy_and_mixed_batches_keep_rows_apart():
    torch.manual_seed(0)
    logits = torch.randn(6, 50)
    s = Sampler(device=torch.device("cpu"))
    temp = torch.tensor([0.0, 0.0, 1.0, 0.0, 2.0, 0.0])
    out = s(logits, temp, torch.zeros(6, dtype=torch.int32), torch.ones(6))
    greedy = logits.argmax(-1).to(torch.int32)
    assert torch.equal(out[temp == 0], greedy[temp == 0])
    assert out.dtype == torch.int32 and out.shape == (6,)


def test_top_k_and_top_p_restrict_the_support():
    logits = torch.tensor([[4.0, 3.0, 2.0, 1.0, 0.0, -1.0]]).repeat(3, 1)
    masked = ref.apply_top_k_top_p(logits, torch.tensor([2, 0, 6], dtype=torch.int32), None)
    assert torch.isfinite(masked[0]).sum() == 2 and torch.isfinite(masked[1]).sum() == 6      # 0 = no limit
    probs = logits[0].softmax(-1)
    p = float(probs[0] + probs[1]) - 1e-4                       # nucleus just below the mass of the top two
    masked = ref.apply_top_k_top_p(logits[:1], None, torch.tensor([p]))
    assert torch.isfinite(masked[0]).nonzero().flatten().tolist() == [0, 1]
    masked = ref.apply_top_k_top_p(logits[:1], None, torch.tensor([1e-6]))                     # always >= 1 token
    assert torch.isfinite(masked[0]).nonzero().flatten().tolist() == [0]
    tie = torch.tensor([[1.0, 1.0, 0.0]])
    assert torch.isfinite(ref.apply_top_k_top_p(tie, torch.tensor([1], dtype=torch.int32), None)[0]).sum() == 2


def test_exponential_race_follows_the_softmax_distribution():
    g = torch.Generator().manual_seed(1)
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).repeat(20000, 1)
    tok = ref.sample(logits, torch.full((20000,), 1.5), None, None, g)
    freq = torch.bincount(tok.long(), minlength=4).float() / 20000
    want = (logits[0] / 1.5).softmax(-1)
    assert (freq - want).abs().max() < 0.015
    # top-k = 2: only two tokens ever, renormalised
    tok = ref.sample(logits, torch.ones(20000), torch.full((20000,), 2, dtype=torch.int32), None, g)
    freq = torch.bincount(tok.long(), minlength=4).float() / 20000
    assert freq[2:].sum() == 0 and abs(float(freq[0]) - float(torch.tensor([2.0, 1.0]).softmax(-1)[0])) < 0.015


def test_penalties_follow_the_openai_definitions():
    logits = torch.tensor([[2.0, -2.0, 1.0, 0.5]])
    counts = torch.tensor([[2.0, 1.0, 0.0, 0.0]])
    prompt = torch.tensor([[False, False, True, False]])
    out = apply_penalties(logits.clone(), prompt, counts, presence=torch.tensor([0.5]), frequency=torch.tensor([0.25]),
                          repetition=torch.tensor([2.0]))
    # token 0: positive logit halved, then - 2 * 0.25 - 0.5; token 1: negative doubled, - 0.25 - 0.5
    assert torch.allclose(out[0], torch.tensor([2.0 / 2 - 0.5 - 0.5, -2.0 * 2 - 0.25 - 0.5, 1.0 / 2, 0.5]))
    same = apply_penalties(logits.clone(), None, torch.zeros(1, 4), torch.zeros(1), torch.zeros(1), torch.ones(1))
    assert torch.equal(same, logits)
