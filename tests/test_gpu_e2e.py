"""End-to-end on the GPU: the engine (CUDA kernels, CUDA graphs) against the CPU
reference path of the same engine."""
import pytest
import torch

from omni_npu_b200 import SamplingParams, ops
from omni_npu_b200.config import ModelConfig
from omni_npu_b200.engine.llm import LLM, build_engine_config

pytestmark = pytest.mark.gpu


def _small_cfg():
    return ModelConfig(hidden_size=512, num_layers=2, num_heads=8, num_kv_heads=2, head_dim=64,
                       intermediate_size=1024, vocab_size=2048, rope_theta=10000.0,
                       max_position_embeddings=2048, dtype=torch.bfloat16)


def test_engine_cuda_graph_and_eager_agree():
    cfg = _small_cfg()
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (48, 5, 130, 64, 17)]
    sp = SamplingParams(max_tokens=24, ignore_eos=True)
    outs = {}
    for name, eager in (("graph", False), ("eager", True)):
        llm = LLM(model=cfg, device="cuda", max_num_seqs=8, max_num_batched_tokens=256, max_model_len=512,
                  num_gpu_blocks=256, enforce_eager=eager, seed=3)
        outs[name] = [o.output_token_ids for o in llm.generate(prompts, sp)]
        assert ops.launch_count() > 0
        del llm
    assert outs["graph"] == outs["eager"]


def _step_logits(llm, prompts, max_tokens=1):
    """Logits of every sampling step of ``generate`` (rows in scheduling order), captured through
    the runner's logits hook.  Returns (list of [n, V] fp32 CPU tensors, generated tokens)."""
    runner = llm.engine.worker.model_runner
    grabbed = []

    def hook(seqs):
        def fn(logits):
            grabbed.append(logits[: len(seqs)].float().cpu().clone())
            return logits
        return fn
    real = runner._make_logits_fn
    runner._make_logits_fn = hook
    try:
        outs = llm.generate(prompts, SamplingParams(max_tokens=max_tokens, ignore_eos=True))
    finally:
        runner._make_logits_fn = real
    return grabbed, [o.output_token_ids for o in outs]


def _pair_on_cpu(gpu_llm, cfg, **kw):
    cpu = LLM(model=cfg, device="cpu", **kw)
    cpu.engine.worker.get_model().load_state_dict(
        {k: v.cpu() for k, v in gpu_llm.engine.worker.get_model().state_dict().items()})
    return cpu


def _assert_logits_close(got, want, max_rel, min_cos):
    assert len(got) == len(want) and len(got) > 0
    for a, b in zip(got, want):
        assert a.shape == b.shape
        rel = (a - b).abs().max() / b.abs().max().clamp_min(1e-6)
        cos = torch.nn.functional.cosine_similarity(a, b, dim=-1).min()
        assert rel <= max_rel and cos >= min_cos, (float(rel), float(cos))


def test_engine_logits_match_cpu_reference_path():
    """Same weights through the CUDA kernels (prefill and eager decode steps) and through the fp32
    CPU ops: the logits of the prompt's last position and of three decode steps agree within bf16
    tolerance (3e-2 of the logit range, as the reference's attention tests use)."""
    cfg = _small_cfg()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 2048, (40,), generator=g).tolist() for _ in range(3)]
    kw = dict(max_num_seqs=4, max_num_batched_tokens=128, max_model_len=256, num_gpu_blocks=64, seed=5)
    gpu = LLM(model=cfg, device="cuda", enforce_eager=True, **kw)
    cpu = _pair_on_cpu(gpu, cfg, **kw)
    # teacher forcing: both engines continue from the CPU path's tokens, so later steps stay comparable
    want, toks = _step_logits(cpu, prompts, max_tokens=1)
    got, _ = _step_logits(gpu, prompts, max_tokens=1)
    _assert_logits_close(got, want, 3e-2, 0.999)
    longer = [p + t for p, t in zip(prompts, toks)]
    want, _ = _step_logits(cpu, longer, max_tokens=1)
    got, _ = _step_logits(gpu, longer, max_tokens=1)
    _assert_logits_close(got, want, 3e-2, 0.999)


def _tiny_deepseek(sparse: bool):
    kw = dict(architecture="DeepseekV3ForCausalLM", model_type="deepseek_v3", hidden_size=512, num_layers=3,
              num_heads=16, num_kv_heads=16, head_dim=192, intermediate_size=1024, vocab_size=2048,
              rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=2048, rope_neox=False,
              num_experts=16, num_experts_per_tok=4, moe_intermediate_size=256, num_shared_experts=1,
              first_k_dense=1, use_mla=True, q_lora_rank=256, kv_lora_rank=512, qk_nope_head_dim=128,
              qk_rope_head_dim=64, v_head_dim=128, scoring_func="sigmoid", norm_topk_prob=True,
              n_group=4, topk_group=2, router_bias=True, routed_scaling_factor=2.5)
    if sparse:
        # 8 index heads: dense torch indexer (the kernel wants a multiple of 16); 16 heads: tcgen05 indexer
        kw.update(architecture="DeepseekV32ForCausalLM", index_topk=64, index_n_heads=16 if sparse == "kernel" else 8,
                  index_head_dim=128)
    return ModelConfig(**kw)


@pytest.mark.parametrize("sparse", [False, True, "kernel"])
def test_deepseek_mla_moe_engine_runs_and_paths_agree(sparse):
    """MLA + MoE model on the GPU: graph decode and eager decode give the same tokens."""
    cfg = _tiny_deepseek(sparse)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (70, 9, 130)]
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    outs = []
    for eager in (False, True):
        llm = LLM(model=cfg, device="cuda", max_num_seqs=4, max_num_batched_tokens=256, max_model_len=512,
                  num_gpu_blocks=128, enforce_eager=eager, seed=9)
        outs.append([o.output_token_ids for o in llm.generate(prompts, sp)])
        ops.check_status()
        if eager:
            # and against the fp32 CPU path of the same model: logits at the end of the prompts (a
            # routing near-tie may pick another expert in bf16, hence the looser bound than for a
            # dense model)
            kw = dict(max_num_seqs=4, max_num_batched_tokens=256, max_model_len=512, num_gpu_blocks=128, seed=9)
            cpu = _pair_on_cpu(llm, cfg, **kw)
            want, _ = _step_logits(cpu, prompts)
            got, _ = _step_logits(llm, prompts)
            _assert_logits_close(got, want, 8e-2, 0.99)
        del llm
    if sparse == "kernel":
        # top-k selection over index scores: a last-bit difference between a decode step padded to a
        # captured batch size and the unpadded one can swap two keys at the selection boundary, after
        # which a greedy continuation of a random-init model may part ways; the first tokens must
        # agree exactly, the whole continuation nearly
        for a, b in zip(outs[0], outs[1]):
            assert a[:5] == b[:5]
            assert sum(x == y for x, y in zip(a, b)) >= 0.6 * len(a)
    else:
        assert outs[0] == outs[1]


def test_deepseek_weight_prefetch_hints_do_not_change_results():
    """The L2 weight prefetcher wired into the decoder layers (hints on a side stream, also inside
    the captured decode graphs): same tokens, and hints were issued."""
    cfg = _tiny_deepseek(False)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (40, 9)]
    sp = SamplingParams(max_tokens=8, ignore_eos=True)
    outs = {}
    for on in (False, True):
        llm = LLM(model=cfg, device="cuda", max_num_seqs=4, max_num_batched_tokens=256, max_model_len=512,
                  num_gpu_blocks=128, seed=9, additional_config={"weight_prefetch": on})
        outs[on] = [o.output_token_ids for o in llm.generate(prompts, sp)]
        pf = llm.engine.worker.get_model().prefetcher
        assert (pf is not None and pf.requested_bytes > 0) if on else pf is None
        ops.check_status()
        del llm
    assert outs[True] == outs[False]


def test_qwen3_moe_engine_runs():
    cfg = ModelConfig(architecture="Qwen3MoeForCausalLM", model_type="qwen3_moe", hidden_size=512, num_layers=2,
                      num_heads=8, num_kv_heads=2, head_dim=128, intermediate_size=1024, vocab_size=2048,
                      rms_norm_eps=1e-6, max_position_embeddings=2048, qk_norm=True, num_experts=16,
                      num_experts_per_tok=4, moe_intermediate_size=128, norm_topk_prob=True)
    llm = LLM(model=cfg, device="cuda", max_num_seqs=4, max_num_batched_tokens=256, max_model_len=512,
              num_gpu_blocks=128, seed=4)
    prompts = [[5, 6, 7] * 20, [9] * 7]
    outs = llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    assert all(len(o.output_token_ids) == 8 for o in outs)
    ops.check_status()
    kw = dict(max_num_seqs=4, max_num_batched_tokens=256, max_model_len=512, num_gpu_blocks=128, seed=4)
    cpu = _pair_on_cpu(llm, cfg, **kw)
    want, _ = _step_logits(cpu, prompts)
    got, _ = _step_logits(llm, prompts)
    _assert_logits_close(got, want, 8e-2, 0.99)


@pytest.mark.parametrize("eager", [False, True])
def test_asynchronous_decode_scheduling_gives_the_same_tokens(eager):
    """Decode step n + 1 is launched before the tokens of step n are read (values fed forward on the device);
    tokens must equal the synchronous engine's, with CUDA graphs and without, including EOS stops."""
    cfg = _small_cfg()
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (48, 5, 130, 64, 17, 33, 90, 12, 7, 21)]
    sps = [SamplingParams(max_tokens=m, ignore_eos=False) for m in (24, 3, 17, 1, 30, 9, 12, 24, 2, 11)]
    base = LLM(model=cfg, device="cuda", max_num_seqs=8, max_num_batched_tokens=256, max_model_len=512,
               num_gpu_blocks=256, enforce_eager=eager, seed=3)
    free = [o.output_token_ids for o in base.generate(prompts, [SamplingParams(max_tokens=30, ignore_eos=True)] * 10)]
    del base
    cfg.eos_token_id = free[4][10]                      # request 4 stops on this token at step 11 at the latest
    outs = {}
    for mode in (False, True):
        llm = LLM(model=cfg, device="cuda", max_num_seqs=8, max_num_batched_tokens=256, max_model_len=512,
                  num_gpu_blocks=256, enforce_eager=eager, seed=3, additional_config={"async_scheduling": mode})
        outs[mode] = [(o.output_token_ids, o.finish_reason) for o in llm.generate(prompts, sps)]
        ops.check_status()
        assert llm.engine.scheduler.pool.num_free == 256
        del llm
    assert outs[True] == outs[False]
    assert outs[True][4][1] == "stop" and len(outs[True][4][0]) <= 11


def test_mtp_chain_of_three_drafts_under_cuda_graphs():
    """A draft head run as a chain of three steps inside the step: the captured decode graphs
    (target model + head + chain) give the tokens of the eager path, drafts are scheduled and
    verified, and every block (the look-ahead ones included) goes back to the pool."""
    cfg = _small_cfg()
    g = torch.Generator().manual_seed(8)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (48, 5, 130, 17)]
    sp = SamplingParams(max_tokens=20, ignore_eos=True)
    outs = {}
    for eager in (False, True):
        llm = LLM(model=cfg, device="cuda", max_num_seqs=4, max_num_batched_tokens=256, max_model_len=512,
                  num_gpu_blocks=256, enforce_eager=eager, seed=3,
                  speculative_config={"method": "mtp", "num_speculative_tokens": 3})
        runner = llm.engine.worker.model_runner
        assert runner.mtp is not None and runner.mtp_k == 3
        outs[eager] = [o.output_token_ids for o in llm.generate(prompts, sp)]
        assert all(len(t) == 20 for t in outs[eager])
        st = llm.engine.scheduler.spec_stats
        assert st["drafted"] >= 3 * llm.engine.stats["spec_decode_steps"] > 0
        assert llm.engine.scheduler.pool.num_free == 256
        ops.check_status()
        del llm
    assert outs[False] == outs[True]


def test_mixed_batches_give_the_tokens_of_separate_steps():
    """Decoding requests ride along in the prefill steps of later requests (their rows go through the
    decode attention kernel, the prompt rows through the prefill kernel, one GEMM over all rows).  A
    rider's row is multiplied inside a larger launch than in a decode step, so the logits agree to
    rounding, not bit for bit: every request starts with the same tokens and most tokens agree."""
    cfg = _small_cfg()
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (48, 200, 130, 64, 170, 33, 90, 120)]
    sps = [SamplingParams(max_tokens=m, ignore_eos=True) for m in (24, 6, 17, 12, 30, 9, 12, 24)]
    outs, steps = {}, {}
    for mixed in (False, True):
        llm = LLM(model=cfg, device="cuda", max_num_seqs=3, max_num_batched_tokens=256, max_model_len=512,
                  num_gpu_blocks=256, seed=3, enable_mixed_batches=mixed)
        outs[mixed] = [o.output_token_ids for o in llm.generate(prompts, sps)]
        steps[mixed] = llm.engine.stats["steps"]
        ops.check_status()
        assert llm.engine.scheduler.pool.num_free == 256
        del llm
    assert steps[True] < steps[False]
    same = total = 0
    for a, b in zip(outs[True], outs[False]):
        assert len(a) == len(b) and a[:2] == b[:2]
        same += sum(x == y for x, y in zip(a, b))
        total += len(a)
    assert same >= 0.6 * total
