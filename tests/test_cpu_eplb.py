"""Expert-parallel load balancing: planner, remap, MoE layer with redundant experts, weight moves."""
import torch

from omni_npu_b200.parallel import state
from omni_npu_b200.parallel.eplb import (EplbState, initial_physical_to_logical, logical_to_physical, plan_placement,
                                          rearrange_expert_weights)


def test_initial_map_and_tables():
    assert initial_physical_to_logical(4, 3) == [0, 1, 2, 3, 0, 1, 2]
    table, counts = logical_to_physical([0, 1, 2, 3, 0, 1, 2], 4)
    assert counts.tolist() == [2, 2, 2, 1]
    assert table[0].tolist() == [0, 4] and table[3].tolist() == [3, 3]


def test_planner_replicates_hot_experts_and_balances_ranks():
    load = [100, 10, 10, 10, 10, 10, 10, 10]
    phy2log = plan_placement(load, 12, 4)
    assert len(phy2log) == 12 and set(phy2log) == set(range(8))
    assert phy2log.count(0) == 5                      # the four spare slots all go to the hot expert
    # its replicas sit on different ranks as far as possible
    per_rank = [phy2log[r * 3:(r + 1) * 3] for r in range(4)]
    assert all(0 in slots for slots in per_rank)
    rank_load = [sum(load[e] / phy2log.count(e) for e in slots) for slots in per_rank]
    assert max(rank_load) / (sum(rank_load) / 4) < 1.2
    # without redundancy the same load is badly skewed
    flat = plan_placement(load, 8, 4)
    flat_load = [sum(load[e] for e in flat[r * 2:(r + 1) * 2]) for r in range(4)]
    assert max(flat_load) / (sum(flat_load) / 4) > 2.0


def test_state_record_remap_and_replan():
    st = EplbState(4, 2, 2)
    ids = torch.tensor([[0, 1], [0, 2], [0, 3], [0, -1]], dtype=torch.int32)
    st.record(ids)
    assert st.load.tolist() == [4.0, 1.0, 1.0, 1.0]
    phys = st.remap(ids)
    assert (phys[ids < 0] == -1).all()
    p2l = st.placement()
    assert all(p2l[int(p)] == int(l) for p, l in zip(phys.flatten(), ids.flatten()) if l >= 0)
    # expert 0 has two replicas from the start (slots 0 and 4): consecutive tokens alternate
    assert phys[:, 0].tolist() == [0, 4, 0, 4]
    before = st.imbalance()
    old, new = st.replan()
    st.set_placement(new)
    st.record(ids)
    assert new.count(0) == 3 and st.imbalance() < 1.2 and before < 1.2
    assert st.remap(ids)[:, 0].unique().numel() == 3


def test_moe_layer_with_redundant_experts_matches_plain_layer():
    from omni_npu_b200.layers.moe import FusedMoE
    state.ensure_initialized(torch.device("cpu"))
    torch.manual_seed(0)
    e, k, h, inter = 4, 2, 32, 16
    plain = FusedMoE(e, k, h, inter, dtype=torch.float32, enable_expert_parallel=False)
    red = FusedMoE(e, k, h, inter, dtype=torch.float32, enable_expert_parallel=False, num_redundant_experts=2)
    gate_w = torch.randn(e, h) * 0.5
    plain.gate.weight.data.copy_(gate_w)
    red.gate.weight.data.copy_(gate_w)
    for i in range(e):
        g, u, d = torch.randn(inter, h) * 0.2, torch.randn(inter, h) * 0.2, torch.randn(h, inter) * 0.2
        for layer in (plain, red):
            assert layer.weight_loader(layer.w13, g, i, "gate")
            layer.weight_loader(layer.w13, u, i, "up")
            layer.weight_loader(layer.w2, d, i, "down")
    assert red.w13.shape[0] == 6 and torch.equal(red.w13[4], red.w13[0])
    x = torch.randn(9, h)
    want = plain(x)
    assert torch.allclose(red(x), want, atol=1e-5)
    assert red.eplb.load.sum() == 9 * k
    # re-plan from the recorded load, move the weights, results unchanged
    red.eplb.load.copy_(torch.tensor([50.0, 1.0, 1.0, 1.0]))
    moved = red.rebalance()
    assert red.eplb.placement().count(0) == 3 and moved >= 1
    assert torch.allclose(red(x), want, atol=1e-5)


def test_rearrange_single_rank_moves_within_rank():
    w = torch.arange(4, dtype=torch.float32).view(4, 1).clone()       # slot i holds expert value i (3 = copy of 0)
    w[3] = 0.0
    old, new = [0, 1, 2, 0], [0, 1, 2, 2]
    assert rearrange_expert_weights([w], old, new, None) == 1
    assert w.flatten().tolist() == [0.0, 1.0, 2.0, 2.0]


def test_fp8_block_scaled_experts_expand_to_the_same_layer():
    """An MoE layer loaded from block-scaled e4m3 expert tensors computes what the layer with the
    de-quantised weights computes (gate/up rows are interleaved, their scale blocks are not)."""
    from omni_npu_b200.layers.moe import FusedMoE
    from omni_npu_b200.layers.quant_fp8 import quantize_weight_block
    from omni_npu_b200.ops import ref
    state.ensure_initialized(torch.device("cpu"))
    torch.manual_seed(1)
    e, k, h, inter = 2, 1, 256, 256
    q = FusedMoE(e, k, h, inter, dtype=torch.float32, enable_expert_parallel=False, quant="fp8")
    plain = FusedMoE(e, k, h, inter, dtype=torch.float32, enable_expert_parallel=False)
    gate_w = torch.randn(e, h)
    q.gate.weight.data.copy_(gate_w)
    plain.gate.weight.data.copy_(gate_w)
    for i in range(e):
        for shard, shape, param, sparam in (("gate", (inter, h), "w13", "w13_scale"), ("up", (inter, h), "w13", "w13_scale"),
                                            ("down", (h, inter), "w2", "w2_scale")):
            w = torch.randn(*shape) * torch.logspace(-1, 1, shape[0]).unsqueeze(1)     # block scales differ a lot
            wq, ws = quantize_weight_block(w)
            q.weight_loader(getattr(q, param), wq, i, shard)
            q.weight_loader(getattr(q, sparam), ws, i, shard)
            plain.weight_loader(getattr(plain, param), ref.dequant_fp8_block(wq, ws), i, shard)
    q.process_weights_after_loading()
    assert q.w13.dtype == torch.float32 and q.quant == "fp8-expanded"
    x = torch.randn(5, h)
    assert torch.allclose(q(x), plain(x), rtol=1e-4, atol=1e-4)
