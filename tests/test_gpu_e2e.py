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


def test_engine_logits_match_cpu_reference_path():
    """Same weights through the CUDA kernels and through the fp32 CPU ops: the
    greedy continuation agrees for the first tokens (bf16 rounding can flip a
    near-tie later on, so only a prefix is compared) and decode is stable."""
    cfg = _small_cfg()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 2048, (40,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(max_tokens=4, ignore_eos=True)
    gpu = LLM(model=cfg, device="cuda", max_num_seqs=4, max_num_batched_tokens=128, max_model_len=256,
              num_gpu_blocks=64, seed=5)
    cpu = LLM(model=cfg, device="cpu", max_num_seqs=4, max_num_batched_tokens=128, max_model_len=256,
              num_gpu_blocks=64, seed=5)
    cpu.engine.worker.get_model().load_state_dict(
        {k: v.cpu() for k, v in gpu.engine.worker.get_model().state_dict().items()})
    a = [o.output_token_ids for o in gpu.generate(prompts, sp)]
    b = [o.output_token_ids for o in cpu.generate(prompts, sp)]
    agree = sum(x[0] == y[0] for x, y in zip(a, b))
    assert agree >= 2
