"""Multi-process tests on CPU (gloo, world size 2): communicator semantics and a
tensor-parallel engine run compared with the plain PyTorch model."""
import json
import os
import tempfile

import pytest
import torch

import reference_llama as refm
from dist_utils import run_ranks
from omni_npu_b200.config import tiny_llama
from test_cpu_plumbing import _save


def test_communicator_semantics_two_ranks():
    with tempfile.TemporaryDirectory() as d:
        r0, r1 = run_ranks("comm", 2, d)
    assert r0["all_reduce"] == 3.0 and r1["all_reduce"] == 3.0
    assert r0["all_gather0"] == [0.0, 0.0, 1.0, 1.0]
    assert r0["all_gather_last_shape"] == [2, 6] and r0["all_gather_last_row"] == [0, 0, 0, 1, 1, 1]
    assert r0["reduce_scatter"] == [0.0, 2.0] and r1["reduce_scatter"] == [4.0, 6.0]
    assert r1["all_gatherv"] == [0.0, 1.0, 1.0]
    assert r0["reduce_scatterv_shape"] == [1, 2] and r1["reduce_scatterv_shape"] == [2, 2]
    assert r0["reduce_scatterv_val"] == 2.0
    assert r0["all_to_all"] == [0.0, 1.0, 100.0, 101.0] and r1["all_to_all"] == [2.0, 3.0, 102.0, 103.0]
    assert r0["gather"] == [0.0, 1.0] and r1["gather"] is None
    assert r1["recv"] == [7.0, 8.0]
    assert r0["swap"] == [11.0] * 3 and r1["swap"] == [10.0] * 3
    assert r1["bcast_obj"] == {"k": 0}
    assert r0["async"] == [3.0, [0.0, 0.0, 1.0, 1.0], [0.0, 2.0]] and r1["async"][2] == [4.0, 6.0]
    assert r0["layer_group"] == [2, 0] and r1["layer_group"] == [2, 1]


def test_tensor_parallel_engine_matches_plain_pytorch():
    cfg = tiny_llama()
    weights = refm.make_weights(cfg, seed=3)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (20, 33, 9)]
    with tempfile.TemporaryDirectory() as d:
        os.makedirs(os.path.join(d, "model"))
        _save(weights, cfg, os.path.join(d, "model"))
        json.dump(prompts, open(os.path.join(d, "prompts.json"), "w"))
        res = run_ranks("tp_engine", 2, d)
    for p, toks in zip(prompts, res[0]["tokens"]):
        assert toks == refm.greedy_generate(weights, cfg, p, 12)
    assert res[0]["tokens"] == res[1]["tokens"]


def test_sequence_parallel_residual_stream_matches_plain_pytorch():
    """Token-sharded residual stream (reduce-scatter / all-gather around every block); prompt
    lengths that do not divide by the group size exercise the padding."""
    cfg = tiny_llama()
    weights = refm.make_weights(cfg, seed=5)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (21, 34, 7)]
    with tempfile.TemporaryDirectory() as d:
        os.makedirs(os.path.join(d, "model"))
        _save(weights, cfg, os.path.join(d, "model"))
        json.dump(prompts, open(os.path.join(d, "prompts.json"), "w"))
        open(os.path.join(d, "sequence_parallel"), "w").close()
        res = run_ranks("tp_engine", 2, d)
    for p, toks in zip(prompts, res[0]["tokens"]):
        assert toks == refm.greedy_generate(weights, cfg, p, 12)
    assert res[0]["tokens"] == res[1]["tokens"]


@pytest.mark.parametrize("world,pcp,split", [(2, 2, False), (4, 2, False), (2, 2, True)])
def test_prefill_context_parallel_engine_matches_plain_pytorch(world, pcp, split):
    """Prefill steps split over two ranks by tokens (every layer gathers the step's keys and values,
    each rank attends with its own query rows, the owner of a prompt's last row samples); decode
    steps replicated.  Prompts are longer than the 64-token step budget, so later chunks attend
    to keys that earlier steps gathered into the cache; tokens equal the plain PyTorch model."""
    cfg = tiny_llama()
    weights = refm.make_weights(cfg, seed=7)
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (21, 70, 7, 50, 3)]
    with tempfile.TemporaryDirectory() as d:
        os.makedirs(os.path.join(d, "model"))
        _save(weights, cfg, os.path.join(d, "model"))
        json.dump(prompts, open(os.path.join(d, "prompts.json"), "w"))
        open(os.path.join(d, "prefill_context_parallel"), "w").write(str(pcp))
        if split:
            # decode steps: every sequence decoded by ONE rank of the group, tokens gathered
            open(os.path.join(d, "pcp_decode_split"), "w").close()
        res = run_ranks("tp_engine", world, d)             # world = pcp x tensor-parallel size
    for p, toks in zip(prompts, res[0]["tokens"]):
        assert toks == refm.greedy_generate(weights, cfg, p, 12)
    for r in res[1:]:
        assert r["tokens"] == res[0]["tokens"]
        assert res[0]["pcp_steps"] >= 3 and r["pcp_steps"] == res[0]["pcp_steps"]
    if split:
        rows = [r["pcp_decode_rows"] for r in res]
        assert sum(rows) == 5 * 11 and all(0 < x < 5 * 11 for x in rows)     # 5 requests x 11 decode steps, shared out
    else:
        assert all(r["pcp_decode_rows"] == 0 for r in res)


def test_api_server_loop_replicates_requests_to_the_other_tensor_parallel_rank():
    """Requests reach rank 0 only; its loop broadcasts them (and aborts) before each step and rank 1
    follows step for step: tokens equal the plain PyTorch model, rank 1 ends idle with all blocks free."""
    cfg = tiny_llama()
    weights = refm.make_weights(cfg, seed=11)
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (20, 33, 9)]
    with tempfile.TemporaryDirectory() as d:
        os.makedirs(os.path.join(d, "model"))
        _save(weights, cfg, os.path.join(d, "model"))
        json.dump(prompts, open(os.path.join(d, "prompts.json"), "w"))
        res = run_ranks("server_loop", 2, d)
    for p, toks in zip(prompts, res[0]["tokens"]):
        assert toks == refm.greedy_generate(weights, cfg, p, 12)
    assert res[1]["unfinished"] is False and res[1]["free_blocks"] == 64


def _pipeline_case(world: int, pp: int, seed: int, partition=None):
    cfg = tiny_llama()
    weights = refm.make_weights(cfg, seed=seed)
    g = torch.Generator().manual_seed(seed)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (20, 33, 9, 70)]
    with tempfile.TemporaryDirectory() as d:
        os.makedirs(os.path.join(d, "model"))
        _save(weights, cfg, os.path.join(d, "model"))
        json.dump(prompts, open(os.path.join(d, "prompts.json"), "w"))
        open(os.path.join(d, "pipeline_parallel"), "w").write(str(pp))
        old = os.environ.pop("OMNI_B200_PP_LAYER_PARTITION", None)
        if partition:
            os.environ["OMNI_B200_PP_LAYER_PARTITION"] = partition
        try:
            res = run_ranks("tp_engine", world, d)
        finally:
            os.environ.pop("OMNI_B200_PP_LAYER_PARTITION", None)
            if old is not None:
                os.environ["OMNI_B200_PP_LAYER_PARTITION"] = old
    for p, toks in zip(prompts, res[0]["tokens"]):
        assert toks == refm.greedy_generate(weights, cfg, p, 12)
    for r in res[1:]:
        assert r["tokens"] == res[0]["tokens"]


def test_pipeline_parallel_two_stages_matches_plain_pytorch():
    """Two pipeline stages (gloo): hidden state and residual cross the boundary, the last stage
    samples and every rank books the same tokens (the 70-token prompt is chunked at 64)."""
    _pipeline_case(world=2, pp=2, seed=7)


def test_pipeline_times_tensor_parallel_with_uneven_stages():
    """pp 2 x tp 2 with an uneven layer split: the un-reduced partial sums travel between equal
    tensor-parallel ranks of neighbouring stages."""
    cfg = tiny_llama()
    part = f"1,{cfg.num_layers - 1}"
    _pipeline_case(world=4, pp=2, seed=8, partition=part)


@pytest.mark.parametrize("sparse", [False, True])
def test_pipeline_parallel_deepseek_matches_single_process(sparse, monkeypatch):
    """MLA + routed experts (and the sparse-attention indexer with its third cache) over two
    pipeline stages whose boundary follows a dense layer, against the same model in one process."""
    from omni_npu_b200 import SamplingParams
    from omni_npu_b200.config import ModelConfig
    from omni_npu_b200.engine.llm import LLM
    model = dict(architecture="DeepseekV3ForCausalLM", model_type="deepseek_v3", hidden_size=128, num_layers=4,
                 num_heads=4, num_kv_heads=4, head_dim=48, intermediate_size=256, vocab_size=512,
                 rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512, rope_neox=False,
                 num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, num_shared_experts=1,
                 first_k_dense=2, use_mla=True, q_lora_rank=48, kv_lora_rank=512, qk_nope_head_dim=32,
                 qk_rope_head_dim=64, v_head_dim=32, scoring_func="sigmoid", norm_topk_prob=True)
    if sparse:
        model.update(architecture="DeepseekV32ForCausalLM", index_topk=12, index_n_heads=4, index_head_dim=128)
    engine = dict(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=16,
                  num_gpu_blocks=64, seed=5)
    g = torch.Generator().manual_seed(13)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (21, 34, 5)]
    monkeypatch.delenv("OMNI_B200_PP_LAYER_PARTITION", raising=False)
    monkeypatch.setenv("OMNI_B200_INIT_BY_NAME", "1")     # the one-process oracle draws by name like the stages
    with tempfile.TemporaryDirectory() as d:
        json.dump({"model": model, "engine": engine, "prompts": prompts, "max_tokens": 6},
                  open(os.path.join(d, "spec.json"), "w"))
        res = run_ranks("pp_deepseek", 2, d)
    llm = LLM(model=ModelConfig(dtype=torch.float32, **model), device="cpu", **engine)
    want = [o.output_token_ids for o in llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))]
    assert res[0]["tokens"] == want and res[1]["tokens"] == want
    assert res[0]["kv_layers"] == 2 and res[1]["kv_layers"] == 2


def test_decode_context_parallel_mla_two_ranks_gloo():
    with tempfile.TemporaryDirectory() as d:
        res = run_ranks("dcp_mla", 2, d)
    for r in res:
        assert r["max_err"] < 1e-4, r


def test_expert_parallel_moe_two_ranks_gloo():
    with tempfile.TemporaryDirectory() as d:
        res = run_ranks("ep_moe", 2, d)
    for r in res:
        assert max(r["max_err"].values()) < 1e-4, r


def test_prefill_context_parallel_ranks_share_the_experts_two_ranks_gloo():
    """The pcp dimension of the rank grid: two ranks hold different token shards, the expert-parallel
    group spans them, every rank gets the MoE output of its own shard."""
    with tempfile.TemporaryDirectory() as d:
        res = run_ranks("pcp_moe", 2, d)
    for r in res:
        assert max(r["max_err"].values()) < 1e-4, r


def test_rank_grid_with_a_prefill_context_parallel_dimension():
    """Group membership on the [dp, pp, pcp, tp] grid, without processes: the lists that
    init_model_parallel builds for 16 ranks as dp 2 x pp 2 x pcp 2 x tp 2."""
    import torch
    grid = torch.arange(16).view(2, 2, 2, 2)
    tp = grid.reshape(-1, 2).tolist()
    pcp = grid.permute(0, 1, 3, 2).reshape(-1, 2).tolist()
    ep = grid.permute(1, 0, 2, 3).reshape(2, 8).tolist()
    assert [0, 1] in tp and [2, 3] in tp
    assert [0, 2] in pcp and [1, 3] in pcp and [4, 6] in pcp
    assert ep[0] == [0, 1, 2, 3, 8, 9, 10, 11] and ep[1] == [4, 5, 6, 7, 12, 13, 14, 15]


def test_decode_context_parallel_engine_matches_plain_tensor_parallel(monkeypatch):
    """The latent KV cache sharded by tokens over the two tensor-parallel ranks (token p on rank
    p % 2): cache writes skip foreign tokens, prefill gathers the shards of the context (a 70-token
    prompt is chunked at 64, so the second chunk reads gathered context), decode merges the ranks'
    partial attentions by their log-sum-exp.  Tokens equal the same deployment with a replicated
    cache, and a block id covers twice the tokens."""
    model = dict(architecture="DeepseekV2ForCausalLM", model_type="deepseek_v2", hidden_size=128, num_layers=3,
                 num_heads=4, num_kv_heads=4, head_dim=48, intermediate_size=256, vocab_size=512,
                 rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512, rope_neox=False,
                 num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, num_shared_experts=1,
                 first_k_dense=1, use_mla=True, q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=32,
                 qk_rope_head_dim=64, v_head_dim=32)
    engine = dict(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=16,
                  num_gpu_blocks=64, seed=5)
    g = torch.Generator().manual_seed(17)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (21, 70, 5)]
    monkeypatch.setenv("OMNI_B200_INIT_BY_NAME", "1")
    res = {}
    for dcp in (0, 1):
        with tempfile.TemporaryDirectory() as d:
            json.dump({"model": model, "engine": engine, "prompts": prompts, "max_tokens": 8, "dcp": dcp},
                      open(os.path.join(d, "spec.json"), "w"))
            res[dcp] = run_ranks("dcp_engine", 2, d)
    assert res[1][0]["tokens"] == res[0][0]["tokens"]
    assert res[1][0]["tokens"] == res[1][1]["tokens"]
    assert all(len(t) == 8 for t in res[1][0]["tokens"])
    assert res[1][0]["max_blocks"] * 2 == res[0][0]["max_blocks"]
    assert res[1][0]["free_blocks"] == 64 and res[1][1]["free_blocks"] == 64


@pytest.mark.parametrize("sparse", [False, True])
def test_prefill_context_parallel_latent_attention_model_matches_one_process(monkeypatch, sparse):
    """A small latent-attention (MLA) + MoE model with its prefill steps split by tokens over two
    ranks: every layer gathers the step's compressed keys into the local cache, the prefill reads
    all keys from there.  Tokens equal the single-process engine on the same weights."""
    from omni_npu_b200 import SamplingParams
    from omni_npu_b200.config import ModelConfig
    from omni_npu_b200.engine.llm import LLM
    model = dict(architecture="DeepseekV2ForCausalLM", model_type="deepseek_v2", hidden_size=128, num_layers=3,
                 num_heads=4, num_kv_heads=4, head_dim=48, intermediate_size=256, vocab_size=512,
                 rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512, rope_neox=False,
                 num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, num_shared_experts=1,
                 first_k_dense=1, use_mla=True, q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=32,
                 qk_rope_head_dim=64, v_head_dim=32)
    if sparse:
        # keys restricted to the indexer's top 16: the index keys of the step are gathered as well
        model.update(architecture="DeepseekV32ForCausalLM", model_type="deepseek_v32", index_topk=16,
                     index_n_heads=4, index_head_dim=64)
    engine = dict(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=16,
                  num_gpu_blocks=64, seed=5)
    g = torch.Generator().manual_seed(19)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (21, 70, 5)]
    monkeypatch.setenv("OMNI_B200_INIT_BY_NAME", "1")
    with tempfile.TemporaryDirectory() as d:
        json.dump({"model": model, "engine": engine, "prompts": prompts, "max_tokens": 8, "dcp": 0, "pcp": 2},
                  open(os.path.join(d, "spec.json"), "w"))
        res = run_ranks("dcp_engine", 2, d)
    one = LLM(model=ModelConfig(dtype=torch.float32, **model), device="cpu", **engine)
    want = [o.output_token_ids for o in one.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))]
    assert res[0]["tokens"] == res[1]["tokens"]
    if sparse:
        # a 32-row and a 64-row product round a row's index key differently in the last bit, and a
        # top-16 selection over near-equal scores can then differ: the tokens agree up to such a flip
        for got, ref_toks in zip(res[0]["tokens"], want):
            assert got[:4] == ref_toks[:4] and sum(a == b for a, b in zip(got, ref_toks)) >= 6
    else:
        assert res[0]["tokens"] == want
    assert res[0]["pcp_steps"] >= 2 and res[0]["free_blocks"] == 64


def test_decode_split_over_the_prefill_context_parallel_ranks_with_sharded_experts(monkeypatch):
    """A small MLA + MoE model, experts sharded over the two pcp ranks: with every sequence decoded
    by one rank (a lone request leaves the other rank with dummy batches that keep the expert
    exchanges in step) the tokens are those of the same deployment decoding replicated."""
    model = dict(architecture="DeepseekV2ForCausalLM", model_type="deepseek_v2", hidden_size=128, num_layers=3,
                 num_heads=4, num_kv_heads=4, head_dim=48, intermediate_size=256, vocab_size=512,
                 rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512, rope_neox=False,
                 num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, num_shared_experts=1,
                 first_k_dense=1, use_mla=True, q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=32,
                 qk_rope_head_dim=64, v_head_dim=32)
    engine = dict(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=16,
                  num_gpu_blocks=64, seed=5)
    g = torch.Generator().manual_seed(23)
    monkeypatch.setenv("OMNI_B200_INIT_BY_NAME", "1")
    for lens in ((21, 70, 5), (33,)):
        prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in lens]
        res = {}
        for split in (False, True):
            with tempfile.TemporaryDirectory() as d:
                json.dump({"model": model, "engine": engine, "prompts": prompts, "max_tokens": 8, "dcp": 0, "pcp": 2,
                           "ep": True, "pcp_decode_split": split}, open(os.path.join(d, "spec.json"), "w"))
                res[split] = run_ranks("dcp_engine", 2, d)
        assert res[True][0]["tokens"] == res[False][0]["tokens"] == res[True][1]["tokens"]
        rows = [r["pcp_decode_rows"] for r in res[True]]
        assert sum(rows) == 7 * len(lens)                       # one owner per sequence and decode step
        if len(lens) == 1:
            assert sorted(rows) == [0, 7]                       # the other rank ran dummy batches only
