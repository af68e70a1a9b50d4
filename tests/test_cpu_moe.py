"""Mixture-of-experts on CPU: router reference properties, layer against a dense
per-token computation, and expert parallelism over gloo."""
import torch

from omni_npu_b200 import ops
from omni_npu_b200.layers.moe import FusedMoE, select_experts
from omni_npu_b200.ops import ref


def test_router_softmax_and_renorm():
    torch.manual_seed(0)
    logits = torch.randn(17, 64)
    ids, w = ref.moe_topk(logits, None, 6, renorm=False)
    probs = logits.softmax(-1)
    want = probs.topk(6).values
    torch.testing.assert_close(w, want)
    assert (ids.long() == probs.topk(6).indices).all()
    _, w2 = ref.moe_topk(logits, None, 6, renorm=True, scale=2.5)
    torch.testing.assert_close(w2.sum(-1), torch.full((17,), 2.5))


def test_router_grouped_sigmoid_with_bias_only_picks_from_best_groups():
    torch.manual_seed(1)
    t, e, g, kg, k = 11, 256, 8, 4, 8
    logits = torch.randn(t, e)
    bias = torch.randn(e) * 0.1
    ids, w = ref.moe_topk(logits, bias, k, sigmoid=True, n_group=g, topk_group=kg, renorm=True, scale=2.5)
    scores = torch.sigmoid(logits) + bias
    gscore = scores.view(t, g, e // g).topk(2, -1).values.sum(-1)
    best = gscore.topk(kg, -1).indices
    for i in range(t):
        groups = set((ids[i] // (e // g)).tolist())
        assert groups <= set(best[i].tolist())
    # weights are the unbiased sigmoid scores, renormalised
    raw = torch.sigmoid(logits).gather(1, ids.long())
    torch.testing.assert_close(w, raw / raw.sum(-1, keepdim=True) * 2.5)


def _dense_reference(layer: FusedMoE, x):
    logits = ref.gemm(x, layer.gate.weight, out_dtype=torch.float32)
    w, ids = select_experts(logits, layer.top_k, layer.scoring_func, layer.e_score_correction_bias,
                            layer.n_group, layer.topk_group, layer.renormalize, layer.routed_scaling_factor)
    out = ref.moe_experts(x, layer.w13, layer.w2, ids, w)
    if layer.shared_experts is not None:
        out = out + layer.shared_experts(x)
    return out


def test_fused_moe_layer_matches_dense_reference():
    torch.manual_seed(2)
    layer = FusedMoE(8, 2, 64, 32, dtype=torch.float32, num_shared_experts=1, renormalize=True)
    for p in layer.parameters():
        p.data.normal_(0, 0.1)
    x = torch.randn(13, 64)
    torch.testing.assert_close(layer(x), _dense_reference(layer, x), atol=1e-5, rtol=1e-5)


def test_expert_weight_loader_interleaves_gate_and_up():
    layer = FusedMoE(4, 2, 32, 16, dtype=torch.float32)
    gate, up, down = torch.randn(16, 32), torch.randn(16, 32), torch.randn(32, 16)
    assert layer.weight_loader(layer.w13, gate, 2, "gate")
    assert layer.weight_loader(layer.w13, up, 2, "up")
    assert layer.weight_loader(layer.w2, down, 2, "down")
    torch.testing.assert_close(layer.w13[2], ref.interleave_gate_up(gate, up))
    torch.testing.assert_close(layer.w2[2], down)
