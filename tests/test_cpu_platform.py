"""Plugin entry point and platform class: activation rules, config defaults, backend selection."""
import importlib
import types

import pytest
import torch

from omni_npu_b200 import plugin as plugin_mod
from omni_npu_b200.platform import ATTN_BACKENDS, B200Platform, COMMUNICATOR_CLS, WORKER_CLS


def test_plugin_stays_dormant_without_a_blackwell_gpu(monkeypatch):
    monkeypatch.setenv("OMNI_B200_PLUGIN", "0")
    assert plugin_mod.plugin() is None
    monkeypatch.setenv("OMNI_B200_PLUGIN", "1")
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    assert plugin_mod.plugin() is None


def test_plugin_activates_on_compute_capability_10_only(monkeypatch):
    from omni_npu_b200 import ops
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "device_count", lambda: 1)
    monkeypatch.setattr(ops, "load_extension", lambda required=False: True)
    monkeypatch.setattr(torch.cuda, "get_device_capability", lambda i=0: (9, 0))
    monkeypatch.setenv("OMNI_B200_PLUGIN", "1")
    assert plugin_mod.plugin() is None                        # Hopper: leave vLLM's own CUDA platform in charge
    monkeypatch.setenv("OMNI_B200_PLUGIN", "force")
    assert plugin_mod.plugin() == plugin_mod.PLATFORM_CLS
    monkeypatch.setenv("OMNI_B200_PLUGIN", "1")
    monkeypatch.setattr(torch.cuda, "get_device_capability", lambda i=0: (10, 0))
    assert plugin_mod.plugin() == plugin_mod.PLATFORM_CLS
    monkeypatch.setattr(ops, "load_extension", lambda required=False: False)
    assert plugin_mod.plugin() is None                        # no native extension: never a silent fallback
    mod, _, cls = plugin_mod.PLATFORM_CLS.rpartition(".")
    assert getattr(importlib.import_module(mod), cls) is B200Platform


def test_every_class_path_the_platform_hands_out_resolves():
    paths = [WORKER_CLS, COMMUNICATOR_CLS, B200Platform.get_static_graph_wrapper_cls(),
             B200Platform.get_compile_backend(), *ATTN_BACKENDS.values()]
    for path in paths:
        mod, _, name = path.rpartition(".")
        assert hasattr(importlib.import_module(mod), name), path


def test_attention_backend_selection():
    sel = types.SimpleNamespace
    assert B200Platform.get_attn_backend_cls(None, sel(use_mla=False, use_sparse=False), 32) == ATTN_BACKENDS["gqa"]
    assert B200Platform.get_attn_backend_cls(None, sel(use_mla=True, use_sparse=False), 128) == ATTN_BACKENDS["mla"]
    assert B200Platform.get_attn_backend_cls(None, sel(use_mla=True, use_sparse=True), 128) == ATTN_BACKENDS["dsa"]
    assert B200Platform.get_attn_backend_cls(use_mla=True) == ATTN_BACKENDS["mla"]      # keyword form of older vLLM


def test_check_and_update_config_fills_worker_block_size_and_options():
    cfg = types.SimpleNamespace(
        parallel_config=types.SimpleNamespace(worker_cls="auto"),
        cache_config=types.SimpleNamespace(block_size=None),
        compilation_config=types.SimpleNamespace(pass_config=types.SimpleNamespace(enable_fusion=True, enable_noop=True)),
        additional_config={"enable_kv_rmsnorm_rope_cache": True})
    B200Platform.check_and_update_config(cfg)
    assert cfg.parallel_config.worker_cls == WORKER_CLS
    assert cfg.cache_config.block_size and cfg.cache_config.block_size % 16 == 0
    assert cfg.compilation_config.pass_config.enable_fusion is False
    assert cfg.b200_options == {"enable_kv_rmsnorm_rope_cache": True}
    keep = types.SimpleNamespace(parallel_config=types.SimpleNamespace(worker_cls="my.Worker"),
                                 cache_config=types.SimpleNamespace(block_size=64), compilation_config=None,
                                 additional_config=None)
    B200Platform.check_and_update_config(keep)
    assert keep.parallel_config.worker_cls == "my.Worker" and keep.cache_config.block_size == 64


def test_platform_capabilities_and_quantisation_check():
    assert B200Platform.support_static_graph_mode() and B200Platform.use_custom_allreduce()
    assert B200Platform.supports_fp8() and not B200Platform.support_hybrid_kv_cache()
    for q in B200Platform.supported_quantization:
        B200Platform.verify_quantization(q)
    with pytest.raises(ValueError):
        B200Platform.verify_quantization("awq-int3")
    import argparse
    p = argparse.ArgumentParser()
    B200Platform.pre_register_and_update(p)
    ns = p.parse_args(["--reasoning-config", '{"think_start_str": "<think>"}'])
    assert ns.reasoning_config == {"think_start_str": "<think>"} and ns.enable_kv_rmsnorm_rope_cache is True
