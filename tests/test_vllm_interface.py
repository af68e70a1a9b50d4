"""Snapshot of the vLLM surface this package plugs into.  When vLLM is importable the
adapter classes must subclass the installed interfaces and implement the methods vLLM
calls; when the installed vLLM drifts, this file is where it shows.  Without vLLM the
adapters must still import (they fall back to plain base classes)."""
import importlib
import inspect

import pytest

from omni_npu_b200 import compat

needs_vllm = pytest.mark.skipif(not compat.vllm_available(), reason="vLLM is not installed")


def test_adapters_import_without_side_effects():
    for mod in ("omni_npu_b200.parallel.vllm_communicator", "omni_npu_b200.attention.vllm_backends",
                "omni_npu_b200.kv_transfer.vllm_connector", "omni_npu_b200.worker.vllm_worker",
                "omni_npu_b200.layers.vllm_custom_ops", "omni_npu_b200.models.vllm_adapters",
                "omni_npu_b200.compilation.eager_backend"):
        importlib.import_module(mod)


def test_platform_class_paths_resolve():
    from omni_npu_b200 import platform as P
    paths = [P.WORKER_CLS, P.COMMUNICATOR_CLS, P.GRAPH_WRAPPER_CLS, P.COMPILE_BACKEND_CLS] + list(P.ATTN_BACKENDS.values()) \
        if hasattr(P, "ATTN_BACKENDS") else [P.WORKER_CLS, P.COMMUNICATOR_CLS, P.GRAPH_WRAPPER_CLS, P.COMPILE_BACKEND_CLS]
    for path in paths:
        mod, _, name = path.rpartition(".")
        assert hasattr(importlib.import_module(mod), name), path


@needs_vllm
def test_communicator_matches_vllm_base():
    from vllm.distributed.device_communicators.base_device_communicator import DeviceCommunicatorBase
    from omni_npu_b200.parallel.vllm_communicator import B200VllmCommunicator
    assert issubclass(B200VllmCommunicator, DeviceCommunicatorBase)
    for name in ("all_reduce", "all_gather", "reduce_scatter", "all_gatherv", "reduce_scatterv", "gather", "send",
                 "recv", "broadcast", "dispatch", "combine", "prepare_communication_buffer_for_model", "destroy"):
        assert hasattr(DeviceCommunicatorBase, name), f"vLLM dropped DeviceCommunicatorBase.{name}"
        assert name in B200VllmCommunicator.__dict__, name
    assert list(inspect.signature(DeviceCommunicatorBase.__init__).parameters)[:5] == \
        ["self", "cpu_group", "device", "device_group", "unique_name"]


@needs_vllm
def test_attention_backends_match_vllm_interface():
    from vllm.v1.attention.backend import AttentionBackend, AttentionImpl, AttentionMetadataBuilder
    from omni_npu_b200.attention import vllm_backends as B
    for cls, name in ((B.B200AttentionBackend, "B200_ATTN"), (B.B200MLABackend, "B200_MLA"), (B.B200DSABackend, "B200_DSA")):
        assert issubclass(cls, AttentionBackend) and cls.get_name() == name
    assert issubclass(B.B200AttentionImpl, AttentionImpl) and issubclass(B.B200AttentionMetadataBuilder, AttentionMetadataBuilder)
    assert list(inspect.signature(AttentionImpl.forward).parameters)[:8] == \
        ["self", "layer", "query", "key", "value", "kv_cache", "attn_metadata", "output"]
    assert list(inspect.signature(AttentionMetadataBuilder.build).parameters)[:3] == \
        ["self", "common_prefix_len", "common_attn_metadata"]
    from vllm.v1.attention.backend import CommonAttentionMetadata
    for f in ("query_start_loc", "seq_lens", "num_reqs", "num_actual_tokens", "max_query_len", "max_seq_len",
              "block_table_tensor", "slot_mapping"):
        assert f in CommonAttentionMetadata.__dataclass_fields__, f"vLLM dropped CommonAttentionMetadata.{f}"
    assert B.B200AttentionBackend.get_kv_cache_shape(4, 16, 8, 128) == (2, 4, 8, 16, 128)
    assert B.B200MLABackend.is_mla() and B.B200DSABackend.is_sparse()


@needs_vllm
def test_connector_and_custom_ops_match_vllm_interface():
    from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorBase_V1
    from omni_npu_b200.kv_transfer.vllm_connector import B200KVConnector
    assert issubclass(B200KVConnector, KVConnectorBase_V1)
    for name in ("get_num_new_matched_tokens", "update_state_after_alloc", "build_connector_meta", "request_finished",
                 "register_kv_caches", "start_load_kv", "wait_for_layer_load", "save_kv_layer", "wait_for_save",
                 "get_finished"):
        assert hasattr(KVConnectorBase_V1, name), f"vLLM dropped KVConnectorBase_V1.{name}"
        assert name in B200KVConnector.__dict__, name
    from omni_npu_b200.kv_transfer import register
    assert register.CONNECTOR_NAMES[:2] == ("P2PKVConnector", "LLMDataDistConnector")
    assert "HostPoolKVConnector" in register.CONNECTOR_NAMES
    from omni_npu_b200.layers import vllm_custom_ops
    assert {"SiluAndMul", "RMSNorm"} <= set(vllm_custom_ops.REGISTERED)
    from vllm.model_executor.custom_op import CustomOp
    assert hasattr(CustomOp, "register_oot") and hasattr(CustomOp, "forward_oot")


@needs_vllm
def test_worker_and_model_adapters():
    from omni_npu_b200.worker.vllm_worker import B200Worker
    for name in ("init_device", "load_model", "execute_model", "sleep", "wake_up", "initialize_from_config"):
        assert callable(getattr(B200Worker, name))
    from omni_npu_b200.models.vllm_adapters import ADAPTERS, StandaloneModelAdapter
    assert set(ADAPTERS) == {"PanguUltraMoEForCausalLM", "PanguProMoEV2ForCausalLM", "OpenPanguMTPModel", "MockModel"}
    for path in ADAPTERS.values():
        mod, _, name = path.partition(":")
        assert issubclass(getattr(importlib.import_module(mod), name), StandaloneModelAdapter)
    sig = inspect.signature(StandaloneModelAdapter.__init__)
    assert "vllm_config" in sig.parameters and sig.parameters["vllm_config"].kind is inspect.Parameter.KEYWORD_ONLY


def test_thinking_budget_processor_follows_vllm_batch_updates():
    """Rows added / moved / removed through vLLM's BatchUpdate keep their budget state; a row past its
    budget is forced to the end marker."""
    import torch
    from vllm import SamplingParams
    from vllm.v1.sample.logits_processor import BatchUpdate, LogitsProcessor, MoveDirectionality
    from omni_npu_b200.sample.vllm_logits_processor import ThinkingBudgetLogitsProcessor
    from omni_npu_b200.serving.reasoning_config import ReasoningConfig
    assert issubclass(ThinkingBudgetLogitsProcessor, LogitsProcessor)
    cfg = ReasoningConfig(think_start_token_ids=[5], think_end_token_ids=[6])
    proc = ThinkingBudgetLogitsProcessor(None, torch.device("cpu"), False, reasoning_config=cfg)
    out0, out1 = [], []
    sp = SamplingParams(max_tokens=8, extra_args={"thinking_token_budget": 2})
    ThinkingBudgetLogitsProcessor.validate_params(sp)
    proc.update_state(BatchUpdate(batch_size=2, removed=[], moved=[],
                                  added=[(0, sp, [1, 5], out0), (1, SamplingParams(max_tokens=8), [1, 5], out1)]))
    logits = torch.zeros(2, 10)
    assert torch.isfinite(proc.apply(logits.clone())).all()           # budget not used up yet
    out0.extend([7, 8])                                               # two thinking tokens generated
    got = proc.apply(logits.clone())
    assert got[0].argmax() == 6 and torch.isinf(got[0, 7]) and torch.isfinite(got[1]).all()
    # the budgeted row moves to slot 1 (swap), then is removed
    proc.update_state(BatchUpdate(batch_size=2, removed=[], added=[], moved=[(0, 1, MoveDirectionality.SWAP)]))
    got = proc.apply(logits.clone())
    assert got[1].argmax() == 6 and torch.isfinite(got[0]).all()
    proc.update_state(BatchUpdate(batch_size=1, removed=[1], added=[], moved=[]))
    assert torch.isfinite(proc.apply(logits.clone())).all() and not proc.inner.state


def test_padded_metadata_patch_applies_and_reverts():
    """``unpadded`` keeps the padded metadata while the patch is applied and trims again after revert."""
    pytest.importorskip("vllm")
    from vllm.v1.attention.backends.utils import CommonAttentionMetadata
    from omni_npu_b200.patches.common import backends_utils as bu
    patch = bu.PaddedAttentionMetadataPatch
    original = CommonAttentionMetadata.__dict__["unpadded"]
    patch.apply()
    try:
        sentinel = object.__new__(CommonAttentionMetadata)
        assert CommonAttentionMetadata.unpadded(sentinel, 3, 2) is sentinel
    finally:
        patch.revert()
    assert CommonAttentionMetadata.__dict__["unpadded"] is original
