"""Deployment-plan lookup: fingerprints, quant type, PD scheme, file choice, overrides.
Modelled on the reference's loader tests (tests/unit_tests/v1/models/config_loader)."""
import json

import pytest

from omni_npu_b200.models import config_loader as cl

DS_V3 = {"model_type": "deepseek_v3", "hidden_size": 7168, "num_attention_heads": 128, "vocab_size": 129280,
         "intermediate_size": 18432, "n_routed_experts": 256, "n_shared_experts": 1, "moe_intermediate_size": 2048,
         "max_position_embeddings": 163840}


def test_fingerprint_and_quant_type():
    assert cl.parse_hf_config(DS_V3) == ("deepseek_v3", "bf16")
    assert cl.parse_hf_config(dict(DS_V3, quantization_config={"quant_method": "fp8"})) == ("deepseek_v3", "fp8")
    q = {"format": "int-quantized", "kv_cache_scheme": None,
         "config_groups": {"group_0": {"weights": {"num_bits": 8}, "input_activations": {"num_bits": 8}}}}
    assert cl.parse_hf_config(dict(DS_V3, quantization_config=q))[1] == "w8a8c16"
    q["kv_cache_scheme"] = {"num_bits": 8}
    assert cl.quant_type_of({"quantization_config": q}) == "w8a8c8"
    q["kv_cache_scheme"] = "Opti-C8"
    q["config_groups"]["group_0"]["weights"]["num_bits"] = {"a": 4, "b": 8}
    assert cl.quant_type_of({"quantization_config": q}) == "w4a8_fa_c8"
    # no fingerprint matches: the model type is the name
    assert cl.parse_hf_config({"model_type": "mystery", "hidden_size": 3})[0] == "mystery"
    # an object with attributes works like a dict
    class Cfg:
        pass
    c = Cfg()
    c.__dict__.update(model_type="llama", hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                      intermediate_size=14336, vocab_size=128256)
    assert cl.parse_hf_config(c)[0] == "llama3_8b"


def test_ambiguous_fingerprint(tmp_path):
    (tmp_path / "fingerprints.json").write_text(json.dumps({"a": {"hidden_size": 8}, "b": {"hidden_size": 8},
                                                            "m": {"hidden_size": 8}}))
    with pytest.raises(RuntimeError):
        cl.parse_hf_config({"model_type": "zzz", "hidden_size": 8}, tmp_path)
    assert cl.parse_hf_config({"model_type": "m", "hidden_size": 8}, tmp_path)[0] == "m"


def test_plan_files_by_role_and_scheme():
    t = cl.TaskProfile(model_name="deepseek_v3", quant_type="fp8", is_pd_disaggregation=True, is_prefill_node=True)
    assert cl.pd_scheme_of(t) == "1P1D"
    assert cl.find_plan_file(t).name == "ds_v3_fp8_b200_1p1d_p.json"
    t.is_prefill_node = False
    assert cl.find_plan_file(t).name == "ds_v3_fp8_b200_1p1d_d.json"
    t.is_pd_disaggregation = False
    assert cl.find_plan_file(t).name == "ds_v3_fp8_b200_hybrid.json"
    t.is_pd_disaggregation, t.prefill_node_num = True, 7
    assert cl.find_plan_file(t) is None                    # 7P1D has no plan: defaults
    t.enable_pd_elastic_scaling = True
    assert cl.pd_scheme_of(t) == "pd_elastic_scaling"
    assert cl.find_plan_file(cl.TaskProfile(model_name="nope")) is None


def test_every_indexed_plan_exists_and_loads():
    for mode in ("throughput", "latency"):
        for entry in json.load(open(cl.CONFIG_ROOT / mode / "index.json")):
            for scheme, files in entry["configs"].items():
                for rel in files.values():
                    data = json.load(open(cl.CONFIG_ROOT / mode / rel))
                    cl.ParallelPlan(**cl._keep_known(cl.ParallelPlan, data["parallel"]))
                    cl.KernelPlan(**cl._keep_known(cl.KernelPlan, data["kernels"]))
                    assert not set(data["kernels"]) - {f.name for f in cl.fields(cl.KernelPlan)}, rel


def test_load_decode_plan_and_overrides(monkeypatch):
    env = {"ROLE": "decode", "PREFILL_POD_NUM": "1", "DECODE_POD_NUM": "1"}
    cfg = cl.load_model_extra_config(dict(DS_V3, quantization_config={"quant_method": "fp8"}), env=env)
    assert cfg is cl.model_extra_config and cfg.source.endswith("ds_v3_fp8_b200_1p1d_d.json")
    assert cfg.task.is_pd_disaggregation and not cfg.task.is_prefill_node
    assert cfg.parallel.dense_mlp_tp_size == 4
    assert cfg.parallel.layer_parallel_config["mlp.down_proj"]["y_transform"]["type"] == "AllReduce"
    assert cfg.kernels.decode_moe_dispatch_combine and cfg.kernels.expert_gate_up_prefetch == 24
    assert cfg.operator_opt_config is cfg.kernels and cfg.parall_config is cfg.parallel
    assert cl.is_mlp_weight_prefetch_on()
    # eager mode switches prefetch and stream tuning off
    cfg = cl.load_model_extra_config(dict(DS_V3, quantization_config={"quant_method": "fp8"}), env=env,
                                     enforce_eager=True)
    assert cfg.task.graph_mode == "eager_mode"
    assert not cfg.kernels.enable_prefetch and cfg.kernels.attn_prefetch == 0 and not cfg.kernels.moe_multi_stream_tune
    assert not cl.is_mlp_weight_prefetch_on()
    # unknown model: defaults, no source
    cfg = cl.load_model_extra_config({"model_type": "mystery"}, env={})
    assert cfg.source is None and cfg.kernels == cl.KernelPlan() and cfg.task.model_name == "mystery"
    json.loads(cfg.to_json())


def test_kernel_plan_validation(monkeypatch):
    with pytest.raises(ValueError):
        cl.KernelPlan(enable_pipeline_comm=True, enable_round_pipeline_comm=True)
    with pytest.raises(ValueError):
        cl.KernelPlan(expert_gate_up_prefetch=80, expert_down_prefetch=40)
    k = cl.KernelPlan(enable_prefetch=False, attn_prefetch=50)
    assert k.attn_prefetch == 0 and k.lm_head_prefetch == 0
    monkeypatch.setenv("ENABLE_OMNI_CACHE", "1")
    assert cl.KernelPlan().use_host_kv_pool


def test_layer_parallel_plan_applies_to_linear_layers():
    import torch
    from omni_npu_b200.layers.linear import RowParallelLinear
    from omni_npu_b200.parallel import state
    state.ensure_initialized(torch.device("cpu"))
    try:
        made = state.apply_layer_parallel_config({
            "mlp.down_proj": {"tp_size_or_ranks": 1, "x_transform": {"type": "None"},
                              "y_transform": {"type": "ReduceScatter"}},
            "self_attn.qkv_proj": {"x_transform": {"type": "AllGather"}}})
        assert set(made) == {"mlp.down_proj"}
        assert state.get_layer_transforms("mlp.down_proj") == (None, "ReduceScatter")
        assert state.get_layer_transforms("self_attn.qkv_proj") == ("AllGather", None)
        lin = RowParallelLinear(16, 8, dtype=torch.float32, device="cpu", prefix="model.layers.0.mlp.down_proj")
        assert lin.group is made["mlp.down_proj"] and lin.y_transform == "ReduceScatter"
        with pytest.raises(ValueError):
            state.apply_layer_parallel_config({"x.y": {"y_transform": {"type": "Shuffle"}}})
    finally:
        state.destroy_model_parallel()
