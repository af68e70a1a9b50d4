"""Speculative decoding on CPU: verification rule, rejection sampler, n-gram proposer and
the whole engine path (drafts scheduled, verified, KV positions rolled back)."""
import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.config import ModelConfig
from omni_npu_b200.engine.llm import LLM
from omni_npu_b200.ops import ref
from omni_npu_b200.sample.rejection_sampler import RejectionSampler, SpecDecodeMetadata, parse_output
from omni_npu_b200.sample.sampler import Sampler
from omni_npu_b200.spec_decode import NgramProposer


def test_spec_verify_rule():
    md = SpecDecodeMetadata.make([[5, 6, 7], [], [9, 9]], "cpu")
    assert md.cu_num_draft_tokens.tolist() == [0, 3, 3, 5] and md.max_spec_len == 3
    assert md.target_logits_indices.tolist() == [0, 1, 2, 5, 6] and md.bonus_logits_indices.tolist() == [3, 4, 7]
    target = torch.tensor([5, 6, 1, 9, 9], dtype=torch.int32)      # request 0 rejects its 3rd draft
    bonus = torch.tensor([40, 41, 42], dtype=torch.int32)
    toks, num = ref.spec_verify(md.draft_token_ids, target, bonus, md.cu_num_draft_tokens, md.max_spec_len)
    assert parse_output(toks, num) == [[5, 6, 1], [41], [9, 9, 42]]
    assert toks[0].tolist() == [5, 6, 1, -1] and toks[1].tolist() == [41, -1, -1, -1]


def test_rejection_sampler_greedy_matches_sequential_argmax():
    torch.manual_seed(0)
    v = 50
    drafts = [[3, 4], [7]]
    md = SpecDecodeMetadata.make(drafts, "cpu")
    logits = torch.randn(5, v)
    logits[0, 3] = 10.0       # request 0: first draft right,
    logits[1, 9] = 10.0       # second wrong -> emits 9 and stops
    logits[3, 7] = 10.0       # request 1: draft right, bonus = argmax(row 4)
    rs = RejectionSampler(Sampler(None, torch.device("cpu")))
    z = torch.zeros(2)
    toks, num = rs(md, None, logits, z, torch.zeros(2, dtype=torch.int32), torch.ones(2))
    assert parse_output(toks, num) == [[3, 9], [7, int(logits[4].argmax())]]


def test_rejection_sampler_strict_accepts_identical_distributions():
    torch.manual_seed(1)
    v = 20
    md = SpecDecodeMetadata.make([[2, 5]], "cpu")
    logits = torch.randn(3, v)
    probs = torch.softmax(logits[:2], -1)
    rs = RejectionSampler(Sampler(None, torch.device("cpu")))
    toks, num = rs(md, probs, logits, torch.ones(1), torch.zeros(1, dtype=torch.int32), torch.ones(1), strict=True)
    assert int(num[0]) == 3 and toks[0, :2].tolist() == [2, 5]      # p == q: always accepted


def test_ngram_proposer():
    p = NgramProposer(3, 2, 4)
    assert p.propose_one([1, 2, 3, 4, 5, 9, 9, 2, 3, 4]) == [5, 9, 9]
    assert p.propose_one([1, 2, 3]) == []
    assert p.propose_one([4, 8, 4, 8, 4, 8]) == [4, 8]      # most recent match wins, continuation clipped by the end


def _tiny():
    return ModelConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
                       intermediate_size=128, vocab_size=97, max_position_embeddings=512, dtype=torch.float32)


def test_engine_with_ngram_speculation_matches_plain_greedy():
    """Greedy decoding must give the same tokens with and without speculation; repetitive
    prompts make the n-gram proposer hit so that accepted AND rejected drafts both occur."""
    g = torch.Generator().manual_seed(5)
    base = torch.randint(0, 97, (6,), generator=g).tolist()
    prompts = [base * 4, torch.randint(0, 97, (19,), generator=g).tolist(), (base[:3] * 7)[:20]]
    sp = SamplingParams(max_tokens=24, ignore_eos=True)
    kw = dict(device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256,
              block_size=8, num_gpu_blocks=128, seed=3)
    plain = LLM(model=_tiny(), **kw)
    want = [o.output_token_ids for o in plain.generate(prompts, sp)]
    spec = LLM(model=_tiny(), speculative_config={"method": "ngram", "num_speculative_tokens": 3,
                                                  "prompt_lookup_min": 1}, **kw)
    got = [o.output_token_ids for o in spec.generate(prompts, sp)]
    assert got == want
    st = spec.engine.scheduler.spec_stats
    assert st["drafted"] > 0 and spec.engine.stats["spec_decode_steps"] > 0
    assert all(len(t) == 24 for t in got)
    # fewer model steps than tokens when drafts are accepted
    if st["accepted"]:
        assert spec.engine.stats["steps"] < plain.engine.stats["steps"]


def test_engine_with_mtp_head_matches_plain_greedy():
    """A randomly initialised MTP head drafts mostly wrong tokens; verification must keep the
    output identical to plain greedy decoding, and the head's own KV-cache layer must exist."""
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 97, (n,), generator=g).tolist() for n in (9, 30, 17)]
    sp = SamplingParams(max_tokens=16, ignore_eos=True)
    kw = dict(device="cpu", max_num_seqs=4, max_num_batched_tokens=24, max_model_len=128,
              block_size=8, num_gpu_blocks=96, seed=3)
    plain = LLM(model=_tiny(), **kw)
    want = [o.output_token_ids for o in plain.generate(prompts, sp)]
    spec = LLM(model=_tiny(), speculative_config={"method": "mtp", "num_speculative_tokens": 1}, **kw)
    runner = spec.engine.worker.model_runner
    assert runner.mtp is not None and len(runner.kv_caches) == 3        # 2 layers + 1 MTP layer
    got = [o.output_token_ids for o in spec.generate(prompts, sp)]
    assert got == want
    st = spec.engine.scheduler.spec_stats
    assert st["drafted"] > 0 and spec.engine.stats["spec_decode_steps"] > 0


def test_engine_with_mtp_chain_of_three_drafts_matches_plain_greedy():
    """k = 3: the head runs as a chain of three steps (its own hidden state and draft feed the next
    step one position further), the scheduler keeps two slots of look-ahead allocated, verification
    steps check up to three drafts.  Output identical to plain greedy decoding; with the MTP layer
    made a copy of the logic that produced the target's next token the drafts are also accepted."""
    g = torch.Generator().manual_seed(12)
    prompts = [torch.randint(0, 97, (n,), generator=g).tolist() for n in (9, 30, 17, 5)]
    sp = SamplingParams(max_tokens=20, ignore_eos=True)
    kw = dict(device="cpu", max_num_seqs=4, max_num_batched_tokens=24, max_model_len=128,
              block_size=8, num_gpu_blocks=96, seed=3)
    plain = LLM(model=_tiny(), **kw)
    want = [o.output_token_ids for o in plain.generate(prompts, sp)]
    spec = LLM(model=_tiny(), speculative_config={"method": "mtp", "num_speculative_tokens": 3}, **kw)
    runner = spec.engine.worker.model_runner
    assert runner.mtp_k == 3 and spec.engine.scheduler.cfg.num_lookahead_tokens == 2
    got = [o.output_token_ids for o in spec.generate(prompts, sp)]
    assert got == want
    st = spec.engine.scheduler.spec_stats
    assert st["drafted"] >= 3 * spec.engine.stats["spec_decode_steps"] > 0
    assert spec.engine.scheduler.pool.num_free == 96             # look-ahead blocks are released too


def test_mtp_checkpoint_names():
    from omni_npu_b200.config import EngineConfig, SpeculativeConfig
    from omni_npu_b200.models.llama import LlamaForCausalLM
    from omni_npu_b200.parallel import state
    state.ensure_initialized(torch.device("cpu"))
    cfg = EngineConfig(model=_tiny(), speculative=SpeculativeConfig("mtp", 1), device="cpu")
    m = LlamaForCausalLM(cfg, device="cpu")
    r = m.mtp.rewrite_name
    assert r("model.layers.1.mlp.down_proj.weight") is None                 # target layer
    assert r("model.layers.2.enorm.weight") == "layers.0.enorm.weight"
    assert r("model.layers.2.shared_head.norm.weight") == "layers.0.shared_head_norm.weight"
    assert r("model.layers.2.self_attn.o_proj.weight") == "layers.0.mtp_block.self_attn.o_proj.weight"
    assert r("model.layers.2.embed_tokens.weight") == "__shared_embedding__"
    assert r("model.layers.3.enorm.weight") is None                         # beyond the MTP layers
    w = torch.full((64,), 2.0)
    loaded = m.load_weights([("model.layers.2.hnorm.weight", w), ("model.norm.weight", w)])
    assert "mtp.layers.0.hnorm.weight" in loaded and torch.equal(m.mtp.layers[0].hnorm.weight.data, w)
