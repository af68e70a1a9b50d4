"""Latent attention with learned sink tokens and a sliding window: the two-partial latent-space
path (window through the sparse mode of the cache kernel, sinks as a small GEMM, merged by
log-sum-exp) against plain per-head attention computed from the same weights."""
import pytest
import torch

from omni_npu_b200 import SamplingParams
from omni_npu_b200.attention.metadata import AttentionMetadata, set_forward_context
from omni_npu_b200.attention.mla import MLABackend, StaticSinkMLAAttention
from omni_npu_b200.config import ModelConfig
from omni_npu_b200.engine.llm import LLM
from omni_npu_b200.models.utils import random_init_


def _cfg(**kw):
    base = dict(architecture="DeepseekV3ForCausalLM", model_type="deepseek_v3", hidden_size=128, num_layers=3,
                num_heads=4, num_kv_heads=4, head_dim=48, intermediate_size=256, vocab_size=512,
                rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512, rope_neox=False,
                num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, num_shared_experts=1,
                first_k_dense=1, use_mla=True, q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=32,
                qk_rope_head_dim=64, v_head_dim=32, dtype=torch.float32)
    base.update(kw)
    return ModelConfig(**base)


def _rope_interleaved(x, pos, cache):
    """x [T, H, D] rotated pairwise (x0,x1),(x2,x3)...; cache rows = [cos | sin] halves."""
    d = x.shape[-1]
    cs = cache[pos.long()].float()
    c, s = cs[:, None, : d // 2], cs[:, None, d // 2:]
    xe, xo = x[..., 0::2].float(), x[..., 1::2].float()
    out = torch.empty_like(x, dtype=torch.float32)
    out[..., 0::2] = xe * c - xo * s
    out[..., 1::2] = xo * c + xe * s
    return out


@pytest.mark.parametrize("sink_len,window", [(4, 8), (3, 0), (0, 6)])
def test_sink_window_latent_attention_matches_plain_attention(sink_len, window):
    torch.manual_seed(0)
    cfg = _cfg()
    att = StaticSinkMLAAttention(cfg, 0, torch.device("cpu"), "model.layers.0.self_attn",
                                 sink_len=sink_len, sliding_window=window)
    random_init_(att, seed=3, std=0.08)
    if sink_len:
        att.param_sink_kv.data.normal_(0, 0.5)
    att.process_weights_after_loading()
    bs, nblk = 16, 8
    cache = MLABackend.allocate_kv_cache(nblk, bs, 512, 64, torch.float32, torch.device("cpu"))
    lens = [21, 13]
    T = sum(lens)
    hidden = torch.randn(T, cfg.hidden_size)
    pos = torch.cat([torch.arange(n) for n in lens]).to(torch.int32)
    block_tables = torch.tensor([[1, 2, 0, 0], [3, 4, 0, 0]], dtype=torch.int32)
    slots = torch.cat([block_tables[b, torch.arange(n) // bs] * bs + torch.arange(n) % bs
                       for b, n in enumerate(lens)]).to(torch.int32)
    cu = torch.tensor([0, lens[0], T], dtype=torch.int32)
    md = AttentionMetadata(is_prefill=True, num_seqs=2, num_tokens=T, max_q_len=max(lens), max_seq_len=max(lens),
                           q_len=0, positions=pos, slot_mapping=slots, block_tables=block_tables,
                           seq_lens=torch.tensor(lens, dtype=torch.int32), cu_q=cu, num_actual_tokens=T,
                           num_actual_seqs=2)
    with set_forward_context(md, [cache]):
        got = att(hidden)

    # ---- plain attention from the same weights
    n, nope, rope, vd, L = att.num_heads, att.nope, att.rope_dim, att.v_dim, att.kv_lora_rank
    q = att.q_proj(hidden).view(T, n, nope + rope)
    q = torch.cat([q[..., :nope].float(), _rope_interleaved(q[..., nope:], pos, att.rotary.cos_sin_cache)], -1)
    kv_a = att.kv_a_proj_with_mqa(hidden)
    c_kv = att.kv_a_layernorm(kv_a[:, :L].contiguous())
    k_pe = _rope_interleaved(kv_a[:, None, L:], pos, att.rotary.cos_sin_cache)[:, 0]
    kv = att.kv_b_proj(c_kv).view(T, n, nope + vd).float()
    if sink_len:
        s_lat = att.sink_latent
        s_kv = att.kv_b_proj(s_lat[:, :L].contiguous()).view(sink_len, n, nope + vd).float()
        s_pe = s_lat[:, L:].float()
    outs = []
    start = 0
    for b, ln in enumerate(lens):
        for i in range(ln):
            lo = max(0, i - window + 1) if window else 0
            rows = torch.arange(start + lo, start + i + 1)
            k_n, v, pe = kv[rows, :, :nope], kv[rows, :, nope:], k_pe[rows]
            if sink_len:
                k_n, v, pe = torch.cat([s_kv[:, :, :nope], k_n]), torch.cat([s_kv[:, :, nope:], v]), torch.cat([s_pe, pe])
            qt = q[start + i]                                           # [n, nope + rope]
            sc = (torch.einsum("nd,knd->nk", qt[:, :nope], k_n) + qt[:, nope:] @ pe.t()) * att.scale
            outs.append(torch.einsum("nk,knd->nd", sc.softmax(-1), v).reshape(-1))
        start += ln
    want = att.o_proj(torch.stack(outs).to(hidden.dtype))
    torch.testing.assert_close(got, want, rtol=2e-4, atol=2e-5)


def test_sink_window_model_decode_continues_like_repeated_prefill():
    """Whole model (learned sinks + window from the HF config): cached decode steps must produce the
    tokens that re-running the growing sequence as a prefill produces."""
    cfg = _cfg(sliding_window=16, hf_config={"param_sink_number": 4})
    llm = LLM(model=cfg, device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128,
              block_size=16, num_gpu_blocks=64, seed=7)
    model = llm.engine.worker.get_model()
    sinks = [m for m in model.modules() if isinstance(m, StaticSinkMLAAttention)]
    assert len(sinks) == cfg.num_layers
    g = torch.Generator().manual_seed(2)
    for m in sinks:
        m.param_sink_kv.data.copy_(torch.randn(m.param_sink_kv.shape, generator=g) * 0.5)
        m.process_weights_after_loading()
    prompts = [torch.randint(0, 512, (k,), generator=g).tolist() for k in (23, 40)]
    fast = llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
    for p, o in zip(prompts, fast):
        toks = list(p)
        for _ in range(6):
            toks.append(llm.generate([toks], SamplingParams(max_tokens=1, ignore_eos=True))[0].output_token_ids[0])
        assert o.output_token_ids == toks[len(p):]
