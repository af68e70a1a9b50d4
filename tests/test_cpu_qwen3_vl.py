"""Qwen3-VL on CPU: vision tower against an independent plain-PyTorch restatement (Conv3d patch
embedding, explicit bilinear interpolation, per-frame attention), M-RoPE positions, embedding
merge, DeepStack injection, and the text path through the engine."""
import math

import pytest
import torch
import torch.nn.functional as F

from omni_npu_b200 import SamplingParams
from omni_npu_b200.attention.gqa import GQABackend
from omni_npu_b200.attention.metadata import AttentionMetadata, set_forward_context
from omni_npu_b200.config import EngineConfig, ModelConfig
from omni_npu_b200.engine.llm import LLM
from omni_npu_b200.models.qwen3_vl import (Qwen3VLForConditionalGeneration, VisionConfig, VisionTransformer,
                                           merge_multimodal_embeddings)
from omni_npu_b200.parallel import state

VC = dict(depth=3, hidden_size=32, intermediate_size=48, num_heads=2, in_channels=3, patch_size=4,
          temporal_patch_size=2, spatial_merge_size=2, out_hidden_size=64, num_position_embeddings=36,
          deepstack_visual_indexes=[0, 2], hidden_act="gelu_pytorch_tanh")


def _cfg():
    return ModelConfig(architecture="Qwen3VLForConditionalGeneration", model_type="qwen3_vl", hidden_size=64,
                       num_layers=3, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=96,
                       vocab_size=300, max_position_embeddings=512, qk_norm=True, dtype=torch.float32,
                       rope_scaling={"rope_type": "default", "mrope_section": [4, 2, 2], "mrope_interleaved": True},
                       hf_config={"vision_config": VC, "image_token_id": 290, "video_token_id": 291})


def _reference_vision(vt: VisionTransformer, pixels, grid_thw):
    c = vt.cfg
    # patch embedding as the strided Conv3d it stands for
    w = vt.patch_embed.weight.view(c.hidden_size, c.in_channels, c.temporal_patch_size, c.patch_size, c.patch_size)
    x = F.conv3d(pixels.view(-1, c.in_channels, c.temporal_patch_size, c.patch_size, c.patch_size), w,
                 vt.patch_embed.bias).view(-1, c.hidden_size)
    side = vt.grid_side
    m = c.spatial_merge_size
    pos, rows_all, cols_all, frames = [], [], [], []
    for t, h, wd in grid_thw:
        table = vt.pos_embed.weight.view(side, side, -1).permute(2, 0, 1).unsqueeze(0)
        emb = F.interpolate(table, size=(h, wd), mode="bilinear", align_corners=True)[0].permute(1, 2, 0)
        order = torch.arange(h * wd).view(h // m, m, wd // m, m).permute(0, 2, 1, 3).reshape(-1)
        pos.append(emb.reshape(h * wd, -1)[order].repeat(t, 1))
        rows_all.append((order // wd).repeat(t))
        cols_all.append((order % wd).repeat(t))
        frames += [h * wd] * t
    x = x + torch.cat(pos)
    rows, cols = torch.cat(rows_all), torch.cat(cols_all)
    d = c.hidden_size // c.num_heads
    inv = 1.0 / (10000.0 ** (torch.arange(0, d // 2, 2).float() / (d // 2)))
    freqs = torch.cat([torch.outer(rows.float(), inv), torch.outer(cols.float(), inv)], -1)
    emb = torch.cat([freqs, freqs], -1)
    cos, sin = emb.cos().unsqueeze(1), emb.sin().unsqueeze(1)

    def rot(v):
        return v * cos + torch.cat([-v[..., d // 2:], v[..., : d // 2]], -1) * sin

    deep = []
    for i, blk in enumerate(vt.blocks):
        qkv = blk.attn_qkv(blk.norm1(x)).view(-1, 3, c.num_heads, d)
        q, k, v = rot(qkv[:, 0]), rot(qkv[:, 1]), qkv[:, 2]
        out = torch.zeros_like(q)
        s = 0
        for n in frames:
            att = torch.softmax(torch.einsum("qhd,khd->hqk", q[s:s + n], k[s:s + n]) / math.sqrt(d), -1)
            out[s:s + n] = torch.einsum("hqk,khd->qhd", att, v[s:s + n])
            s += n
        x = x + blk.attn_proj(out.reshape(-1, c.hidden_size))
        x = x + blk.linear_fc2(F.gelu(blk.linear_fc1(blk.norm2(x)), approximate="tanh"))
        if i in c.deepstack_visual_indexes:
            mg = vt.deepstack_merger_list[c.deepstack_visual_indexes.index(i)]
            deep.append(mg.linear_fc2(F.gelu(mg.linear_fc1(mg.norm(x.view(-1, mg.merged))))))
    mg = vt.merger
    return mg.linear_fc2(F.gelu(mg.linear_fc1(mg.norm(x).view(-1, mg.merged)))), deep


def test_vision_tower_matches_plain_pytorch():
    torch.manual_seed(0)
    vt = VisionTransformer(VisionConfig.from_dict(VC), torch.float32, "cpu")
    for p in vt.parameters():
        p.data.normal_(0, 0.2)
    grid = [(1, 4, 6), (2, 2, 4)]
    n = sum(t * h * w for t, h, w in grid)
    pixels = torch.randn(n, 3 * 2 * 4 * 4)
    got, deep = vt(pixels, grid)
    want, wdeep = _reference_vision(vt, pixels, grid)
    assert got.shape == (n // 4, 64) and len(deep) == 2
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-4)
    for a, b in zip(deep, wdeep):
        assert torch.allclose(a, b, atol=2e-4, rtol=1e-4)


def test_mrope_positions_and_merge():
    state.ensure_initialized(torch.device("cpu"))
    model = Qwen3VLForConditionalGeneration(EngineConfig(model=_cfg(), device="cpu"), device="cpu")
    img = 290
    # 3 text tokens, one image of grid (1, 4, 4) -> 4 merged tokens, 2 text tokens
    toks = [5, 6, 7] + [img] * 4 + [8, 9]
    pos, delta = model.get_mrope_input_positions(toks, [(1, 4, 4)])
    assert pos.shape == (3, 9)
    assert pos[:, :3].tolist() == [[0, 1, 2]] * 3
    assert pos[0, 3:7].tolist() == [3, 3, 3, 3]                 # one temporal index
    assert pos[1, 3:7].tolist() == [3, 3, 4, 4] and pos[2, 3:7].tolist() == [3, 4, 3, 4]
    assert pos[:, 7:].tolist() == [[5, 6]] * 3                  # continues after max(t, h, w) = 2
    assert delta == 7 - 9
    e = torch.zeros(9, 4)
    merge_multimodal_embeddings(e, torch.ones(4, 4), torch.tensor(toks) == img)
    assert e.sum() == 16 and e[3:7].min() == 1
    with pytest.raises(ValueError):
        merge_multimodal_embeddings(e, torch.ones(3, 4), torch.tensor(toks) == img)


def _prefill_md(t, positions, block_size=16, num_blocks=8):
    i32 = torch.int32
    return AttentionMetadata(is_prefill=True, num_seqs=1, num_tokens=t, max_q_len=t, max_seq_len=t, q_len=0,
                             positions=positions, slot_mapping=torch.arange(t, dtype=i32),
                             block_tables=torch.arange(num_blocks, dtype=i32).view(1, -1),
                             seq_lens=torch.tensor([t], dtype=i32), cu_q=torch.tensor([0, t], dtype=i32),
                             num_actual_tokens=t, num_actual_seqs=1)


def test_multimodal_prefill_uses_vision_embeds_deepstack_and_three_axis_positions():
    state.ensure_initialized(torch.device("cpu"))
    torch.manual_seed(1)
    cfg = _cfg()
    model = Qwen3VLForConditionalGeneration(EngineConfig(model=cfg, device="cpu"), device="cpu")
    for p in model.parameters():
        p.data.normal_(0, 0.1)
    img = 290
    toks = torch.tensor([5, 6] + [img] * 4 + [8])
    grid = [(1, 4, 4)]
    pixels = torch.randn(16, 96)
    caches = [GQABackend.allocate_kv_cache(8, 16, 2, 16, torch.float32, torch.device("cpu")) for _ in range(3)]
    pos3, _ = model.get_mrope_input_positions(toks.tolist(), grid)

    def run(use_deep, positions):
        mm, deep = model.embed_multimodal(pixels, grid)
        emb = model.embed_input_ids(toks, mm, deep if use_deep else None)
        with set_forward_context(_prefill_md(7, positions), caches):
            return model.compute_logits(model(toks, positions, emb))

    full = run(True, pos3.to(torch.int32))
    assert full.shape == (7, 300) and torch.isfinite(full).all()
    # DeepStack features matter, and so do the image's (row, col) positions
    assert not torch.allclose(full, run(False, pos3.to(torch.int32)), atol=1e-4)
    flat = torch.arange(7, dtype=torch.int32)
    assert not torch.allclose(full, run(True, flat.unsqueeze(0).expand(3, -1).contiguous()), atol=1e-4)
    # 3-axis positions that coincide are the same as ordinary positions (text-only requests)
    a = run(True, flat.unsqueeze(0).expand(3, -1).contiguous())
    b = run(True, flat)
    assert torch.allclose(a, b, atol=1e-4)


def test_text_only_requests_run_through_the_engine():
    llm = LLM(model=_cfg(), device="cpu", max_num_seqs=2, max_num_batched_tokens=32, max_model_len=64,
              block_size=16, num_gpu_blocks=16, seed=2)
    out = llm.generate([[3, 4, 5, 6, 7]], SamplingParams(max_tokens=5, ignore_eos=True))[0]
    toks = [3, 4, 5, 6, 7]
    for _ in range(5):
        toks.append(llm.generate([toks], SamplingParams(max_tokens=1, ignore_eos=True))[0].output_token_ids[0])
    assert out.output_token_ids == toks[5:]


def test_checkpoint_names():
    state.ensure_initialized(torch.device("cpu"))
    model = Qwen3VLForConditionalGeneration(EngineConfig(model=_cfg(), device="cpu"), device="cpu")
    conv = torch.randn(32, 3, 2, 4, 4)
    loaded = model.load_weights([
        ("model.visual.patch_embed.proj.weight", conv),
        ("model.visual.blocks.1.attn.qkv.bias", torch.ones(96)),
        ("model.visual.blocks.1.mlp.linear_fc1.weight", torch.ones(48, 32)),
        ("model.visual.deepstack_merger_list.1.norm.weight", torch.full((128,), 2.0)),
        ("model.language_model.layers.0.self_attn.q_proj.weight", torch.ones(64, 64)),
        ("model.language_model.norm.weight", torch.full((64,), 3.0))])
    assert torch.equal(model.visual.patch_embed.weight.data, conv.reshape(32, -1))
    assert {"visual.blocks.1.attn_qkv.bias", "visual.blocks.1.linear_fc1.weight",
            "visual.deepstack_merger_list.1.norm.weight", "model.norm.weight",
            "model.layers.0.self_attn.qkv_proj.weight"} <= loaded
