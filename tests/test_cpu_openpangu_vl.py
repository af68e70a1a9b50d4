"""OpenPangu-VL on CPU: window partition, the windowed vision tower against a brute-force masked
attention restatement, checkpoint name mapping, and a multimodal prefill through the Pangu decoder."""
import math

import torch
import torch.nn.functional as F

from omni_npu_b200.attention.metadata import AttentionMetadata, set_forward_context
from omni_npu_b200.config import EngineConfig, ModelConfig
from omni_npu_b200.models.openpangu_vl import (OpenPanguVLForConditionalGeneration, OpenPanguVisionConfig,
                                               OpenPanguVisionTransformer, window_index)
from omni_npu_b200.models.registry import resolve_model_cls
from omni_npu_b200.parallel import state

VC = dict(depth=4, hidden_size=32, intermediate_size=40, num_heads=2, in_channels=3, patch_size=2, temporal_patch_size=2,
          spatial_merge_size=2, out_hidden_size=64, window_size=8, fullatt_block_indexes=[1, 3], hidden_act="silu",
          mm_unit_vision_select_layer=[-1, -3])


def test_window_index_is_a_permutation_with_contiguous_windows():
    grid = [(1, 12, 8), (2, 4, 4)]                       # merged grids 6 x 4 and 2 frames of 2 x 2; window side 2
    perm, lengths = window_index(grid, window_size=8, patch_size=2, merge=2)
    n = 6 * 4 + 2 * 2 * 2
    assert sorted(perm.tolist()) == list(range(n)) and sum(lengths) == n
    assert lengths == [4] * 6 + [4, 4]
    # tokens of the first window: rows 0-1, cols 0-1 of the 6 x 4 grid
    assert perm[:4].tolist() == [0, 1, 4, 5]
    # ragged edge: a 3 x 3 merged grid with side 2 gives windows of 4, 2, 2, 1 tokens
    _, ragged = window_index([(1, 6, 6)], window_size=8, patch_size=2, merge=2)
    assert ragged == [4, 2, 2, 1]


def _brute_force(vt, pixels, grid):
    c = vt.cfg
    m, unit = c.spatial_merge_size, c.spatial_merge_size ** 2
    d = c.hidden_size // c.num_heads
    x = pixels @ vt.patch_embed.weight.t()
    rows, cols, frame_id, win_id = [], [], [], []
    side = c.window_size // m // c.patch_size
    f = 0
    for t, h, w in grid:
        order = torch.arange(h * w).view(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
        r, cl = order // w, order % w
        for ti in range(t):
            rows.append(r)
            cols.append(cl)
            frame_id.append(torch.full_like(r, f))
            win_id.append(f * 10000 + (r // m // side) * 100 + (cl // m // side))
            f += 1
    rows, cols, frame_id, win_id = (torch.cat(v) for v in (rows, cols, frame_id, win_id))
    inv = 1.0 / (10000.0 ** (torch.arange(0, d // 2, 2).float() / (d // 2)))
    freqs = torch.cat([torch.outer(rows.float(), inv), torch.outer(cols.float(), inv)], -1)
    emb = torch.cat([freqs, freqs], -1)
    cos, sin = emb.cos().unsqueeze(1), emb.sin().unsqueeze(1)

    def rot(v):
        return v * cos + torch.cat([-v[..., d // 2:], v[..., : d // 2]], -1) * sin

    def rms(v, wt):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + c.rms_norm_eps) * wt

    taken = {}
    for i, blk in enumerate(vt.blocks):
        qkv = blk.attn_qkv(rms(x, blk.norm1.weight)).view(-1, 3, c.num_heads, d)
        q, k, v = rot(qkv[:, 0]), rot(qkv[:, 1]), qkv[:, 2]
        group = frame_id if i in c.fullatt_block_indexes else win_id
        mask = group.unsqueeze(0) == group.unsqueeze(1)
        att = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(d)
        att = att.masked_fill(~mask.unsqueeze(0), float("-inf")).softmax(-1)
        x = x + blk.attn_proj(torch.einsum("hqk,khd->qhd", att, v).reshape(-1, c.hidden_size))
        gu = blk.gate_up_proj(rms(x, blk.norm2.weight))
        x = x + blk.down_proj(F.silu(gu[:, : c.intermediate_size]) * gu[:, c.intermediate_size:])
        if i in vt.take:
            taken[i] = rms(x, vt.final_layernorm.weight)
    out = 0
    for j, layer in enumerate(vt.take):
        mg = vt.merger[j]
        out = out + mg.fc2(F.gelu(mg.fc1(rms(taken[layer], mg.ln_q.weight).view(-1, mg.merged))))
    return out


def test_windowed_vision_tower_matches_masked_attention():
    torch.manual_seed(0)
    vt = OpenPanguVisionTransformer(OpenPanguVisionConfig.from_dict(VC), torch.float32, "cpu")
    for p in vt.parameters():
        p.data.normal_(0, 0.2)
    grid = [(1, 12, 8), (2, 4, 4), (1, 6, 6)]
    n = sum(t * h * w for t, h, w in grid)
    pixels = torch.randn(n, 3 * 2 * 2 * 2)
    got = vt(pixels, grid)
    assert got.shape == (n // 4, 64)
    assert torch.allclose(got, _brute_force(vt, pixels, grid), atol=2e-4)
    assert vt.take == [3, 1] and len(vt.merger) == 2


def _cfg():
    return ModelConfig(architecture="OpenPanguVLForConditionalGeneration", model_type="openpangu_vl", hidden_size=64,
                       num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32, intermediate_size=128, vocab_size=300,
                       rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=512, rope_neox=False,
                       num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32, num_shared_experts=1,
                       first_k_dense=1, dtype=torch.float32, norm_topk_prob=True,
                       rope_scaling={"rope_type": "default", "mrope_section": [4, 2, 2]},
                       hf_config={"param_sink_number": 8, "param_sink_with_value": True, "v_channels": 24,
                                  "qk_rope_dim": 16, "vision_config": VC, "image_token_id": 290, "video_token_id": 291})


def test_model_is_registered_and_positions_follow_the_image_grid():
    state.ensure_initialized(torch.device("cpu"))
    assert resolve_model_cls("OpenPanguVLForConditionalGeneration") is OpenPanguVLForConditionalGeneration
    model = OpenPanguVLForConditionalGeneration(EngineConfig(model=_cfg(), device="cpu"), device="cpu")
    toks = [5, 6] + [290] * 6 + [8, 9]                      # one image of 1 x 4 x 6 patches -> 2 x 3 merged tokens
    pos, delta = model.get_mrope_input_positions(toks, [(1, 4, 6)])
    assert pos.shape == (3, 10)
    assert pos[:, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 2:8].tolist() == [2] * 6                   # one frame: temporal index constant
    assert pos[1, 2:8].tolist() == [2, 2, 2, 3, 3, 3] and pos[2, 2:8].tolist() == [2, 3, 4, 2, 3, 4]
    assert pos[:, 8].tolist() == [5, 5, 5] and delta == 7 - 10
    emb = model.embed_input_ids(torch.tensor(toks), model.embed_multimodal(torch.randn(24, 24), [(1, 4, 6)]))
    assert emb.shape == (10, 64)


def test_checkpoint_names_of_the_vision_tower():
    state.ensure_initialized(torch.device("cpu"))
    model = OpenPanguVLForConditionalGeneration(EngineConfig(model=_cfg(), device="cpu"), device="cpu")
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g)              # noqa: E731
    w = {"visual.patch_embed.proj.weight": r(32, 3, 2, 2, 2),
         "visual.blocks.0.attn.q.weight": r(32, 32), "visual.blocks.0.attn.k.weight": r(32, 32),
         "visual.blocks.0.attn.v.weight": r(32, 32), "visual.blocks.0.attn.proj.bias": r(32),
         "visual.blocks.0.mlp.gate_proj.weight": r(40, 32), "visual.blocks.0.mlp.up_proj.weight": r(40, 32),
         "visual.blocks.0.mlp.down_proj.weight": r(32, 40), "visual.blocks.1.norm1.weight": r(32),
         "visual.merger.1.mlp.0.weight": r(128, 128), "visual.merger.1.mlp.2.bias": r(64),
         "visual.merger.0.ln_q.weight": r(32), "visual.final_layernorm.weight": r(32)}
    loaded = model.load_weights(w.items())
    v = model.visual
    assert torch.equal(v.patch_embed.weight, w["visual.patch_embed.proj.weight"].reshape(32, -1))
    assert torch.equal(v.blocks[0].attn_qkv.weight[32:64], w["visual.blocks.0.attn.k.weight"])
    assert torch.equal(v.blocks[0].gate_up_proj.weight[40:], w["visual.blocks.0.mlp.up_proj.weight"])
    assert torch.equal(v.blocks[0].down_proj.weight, w["visual.blocks.0.mlp.down_proj.weight"])
    assert torch.equal(v.merger[1].fc1.weight, w["visual.merger.1.mlp.0.weight"])
    assert torch.equal(v.merger[1].fc2.bias, w["visual.merger.1.mlp.2.bias"])
    assert "visual.blocks.0.attn_qkv.weight" in loaded and "visual.final_layernorm.weight" in loaded


def test_multimodal_prefill_through_the_pangu_decoder():
    state.ensure_initialized(torch.device("cpu"))
    torch.manual_seed(2)
    model = OpenPanguVLForConditionalGeneration(EngineConfig(model=_cfg(), device="cpu"), device="cpu")
    for p in model.parameters():
        p.data.normal_(0, 0.1)
    toks = torch.tensor([5, 6] + [290] * 6 + [8])
    grid = [(1, 4, 6)]
    pixels = torch.randn(24, 24)
    caches = model.allocate_kv_cache(16, 8, torch.device("cpu"))
    pos3, _ = model.get_mrope_input_positions(toks.tolist(), grid)
    reserved = getattr(model, "num_reserved_kv_blocks", 0)

    def md(positions):
        t = toks.numel()
        blocks = torch.arange(reserved, reserved + 4, dtype=torch.int32).unsqueeze(0)
        slots = (blocks[0, torch.arange(t) // 8] * 8 + torch.arange(t) % 8).to(torch.int32)
        return AttentionMetadata(is_prefill=True, num_seqs=1, num_tokens=t, max_q_len=t, max_seq_len=t, q_len=0,
                                 positions=positions, slot_mapping=slots, block_tables=blocks,
                                 seq_lens=torch.tensor([t], dtype=torch.int32),
                                 cu_q=torch.tensor([0, t], dtype=torch.int32), num_actual_tokens=t, num_actual_seqs=1)

    def run(positions, with_image=True):
        emb = model.embed_input_ids(toks, model.embed_multimodal(pixels, grid) if with_image else None)
        with set_forward_context(md(positions), caches):
            return model.compute_logits(model(toks, positions, emb))

    full = run(pos3.to(torch.int32))
    assert full.shape == (9, 300) and torch.isfinite(full).all()
    assert not torch.allclose(full, run(pos3.to(torch.int32), with_image=False), atol=1e-4)     # image features matter
    flat = torch.arange(9, dtype=torch.int32)
    assert not torch.allclose(full, run(flat), atol=1e-4)                                       # and so do 2-D positions
