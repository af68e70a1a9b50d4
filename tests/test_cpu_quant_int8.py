"""compressed-tensors int8 W8A8: config parsing, scheme selection, numerics of the linear method."""
import pytest
import torch

from omni_npu_b200.layers.linear import ColumnParallelLinear
from omni_npu_b200.layers.quant_int8 import (CompressedTensorsConfig, QUANT_NAME, W8A8Int8LinearMethod,
                                             int8_linear, quantize_weight_per_channel)
from omni_npu_b200 import ops
from omni_npu_b200.ops import ref
from omni_npu_b200.parallel import state

HF = {"quant_method": "compressed-tensors", "format": "int-quantized", "ignore": ["lm_head", "re:.*\\.mlp\\.gate$"],
      "kv_cache_scheme": None,
      "config_groups": {"group_0": {
          "targets": ["Linear"],
          "weights": {"num_bits": 8, "type": "int", "symmetric": True, "strategy": "channel", "dynamic": False},
          "input_activations": {"num_bits": 8, "type": "int", "symmetric": True, "strategy": "token", "dynamic": True}}}}


def test_config_parsing_and_scheme_selection():
    assert CompressedTensorsConfig.override_quantization_method(HF, None) == QUANT_NAME
    assert CompressedTensorsConfig.override_quantization_method({"quant_method": "fp8"}, None) is None
    cfg = CompressedTensorsConfig.from_config(HF)
    assert isinstance(cfg.get_quant_method("model.layers.0.self_attn.o_proj"), W8A8Int8LinearMethod)
    assert cfg.get_quant_method("lm_head") is None
    assert cfg.get_quant_method("model.layers.3.mlp.gate") is None          # regex ignore
    w4 = {**HF, "config_groups": {"g": {**HF["config_groups"]["group_0"],
                                        "weights": {"num_bits": 4, "type": "int", "strategy": "group"}}}}
    with pytest.raises(NotImplementedError):
        CompressedTensorsConfig.from_config(w4).get_quant_method("model.layers.0.mlp.down_proj")
    static_act = {**HF, "config_groups": {"g": {**HF["config_groups"]["group_0"],
                                                "input_activations": {"num_bits": 8, "type": "int", "dynamic": False,
                                                                      "strategy": "tensor"}}}}
    with pytest.raises(NotImplementedError):
        CompressedTensorsConfig.from_config(static_act).get_quant_method("model.layers.0.mlp.down_proj")


def test_int8_linear_numerics_cpu():
    torch.manual_seed(0)
    x = torch.randn(7, 96)
    w = torch.randn(40, 96) * 0.1
    wq, ws = quantize_weight_per_channel(w)
    assert wq.dtype == torch.int8 and ws.shape == (40,)
    y = int8_linear(x, wq, ws, out_dtype=torch.float32)
    want = x @ w.t()
    assert (y - want).abs().max() < 0.06 * want.abs().max()
    # the integer product itself is exact
    xq, xs = ref.quant_int8_per_token(x)
    acc = (xq.long() @ wq.long().t()).float() * xs[:, None] * ws[None, :]
    assert torch.allclose(ref.gemm_scaled(xq, wq, xs, ws, out_dtype=torch.float32), acc, atol=1e-5)


def test_linear_layer_with_int8_method():
    state.ensure_initialized(torch.device("cpu"))
    torch.manual_seed(1)
    lin = ColumnParallelLinear(64, 48, bias=True, dtype=torch.float32, device="cpu",
                               quant_method=W8A8Int8LinearMethod(), prefix="model.layers.0.mlp.up_proj")
    assert lin.weight.dtype == torch.int8 and lin.weight_scale.shape == (48, 1)
    w = torch.randn(48, 64) * 0.2
    wq, ws = quantize_weight_per_channel(w)
    lin.weight.data.copy_(wq)
    lin.weight_scale.data.copy_(ws.view(-1, 1))
    lin.bias.data.copy_(torch.randn(48))
    lin.process_weights_after_loading()
    x = torch.randn(5, 64)
    y = lin(x).float()
    want = x @ w.t() + lin.bias
    assert (y - want).abs().max() < 0.05 * want.abs().max()


def test_norm_quant_pair_feeds_int8_linear():
    """RMSNorm fused with activation quantisation hands (q, scale) straight to the W8A8 product;
    the result equals norm -> quantise -> product done separately."""
    from omni_npu_b200.layers.norm import RMSNorm
    from omni_npu_b200.layers.quant_int8 import int8_linear, quantize_weight_per_channel
    torch.manual_seed(0)
    x, res = torch.randn(6, 64), torch.randn(6, 64)
    norm = RMSNorm(64, 1e-6, torch.float32)
    norm.weight.data = torch.rand(64) + 0.5
    wq, ws = quantize_weight_per_channel(torch.randn(32, 64))
    res2 = res.clone()
    pair, r_out, y = norm.forward_quant(x, res, "int8", want_bf16=True)
    y_ref, r_ref = norm(x, res2)
    assert torch.allclose(r_out, r_ref) and torch.allclose(y, y_ref, atol=1e-6)
    assert torch.allclose(int8_linear(pair, wq, ws, out_dtype=torch.float32),
                          int8_linear(y_ref, wq, ws, out_dtype=torch.float32), atol=1e-5)
    q, s = ops.silu_and_mul_quant(torch.randn(4, 32), "int8")
    assert q.dtype == torch.int8 and q.shape == (4, 16) and s.shape == (4,)
