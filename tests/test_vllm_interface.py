"""Snapshot of the vLLM surface this package plugs into.  When vLLM is importable the
adapter classes must subclass the installed interfaces and implement the methods vLLM
calls; when the installed vLLM drifts, this file is where it shows.  Without vLLM the
adapters must still import (they fall back to plain base classes)."""
import importlib
import inspect

import pytest
import torch

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


def test_vllm_attention_impl_prefill_then_decode_matches_dense_attention():
    """The backend's ``forward`` (cache write + paged attention through this package's ops, CPU
    reference path here) against plain causal attention, with vLLM-shaped metadata: a two-sequence
    prefill, then one decode step that reads the cache the prefill filled."""
    pytest.importorskip("vllm")
    import types

    from omni_npu_b200.attention.vllm_backends import (B200AttentionBackend, B200AttentionImpl,
                                                       B200AttentionMetadataBuilder)
    torch.manual_seed(0)
    H, HK, D, BS, NB = 4, 2, 64, 16, 8
    impl = B200AttentionImpl(H, D, D ** -0.5, HK)
    kv_cache = torch.zeros(B200AttentionBackend.get_kv_cache_shape(NB, BS, HK, D))
    lens = [19, 7]
    T = sum(lens)
    q, k, v = torch.randn(T, H, D), torch.randn(T, HK, D), torch.randn(T, HK, D)
    bt = torch.tensor([[2, 5], [3, 0]], dtype=torch.int32)
    slots = torch.cat([bt[b, torch.arange(n) // BS] * BS + torch.arange(n) % BS for b, n in enumerate(lens)])
    builder = B200AttentionMetadataBuilder(None, ["model.layers.0.self_attn.attn"], None, torch.device("cpu"))

    def common(n_tok, qsl, seq_lens, max_q, slot):
        return types.SimpleNamespace(num_actual_tokens=n_tok, num_reqs=2, max_query_len=max_q,
                                     max_seq_len=int(max(seq_lens)), query_start_loc=torch.tensor(qsl),
                                     seq_lens=torch.tensor(seq_lens), block_table_tensor=bt, slot_mapping=slot,
                                     causal=True)

    md = builder.build(0, common(T, [0, lens[0], T], lens, max(lens), slots))
    assert not md.is_decode
    out = torch.zeros(T + 3, H * D)                      # vLLM hands over a padded output buffer
    impl.forward(None, q, k, v, kv_cache, md, output=out)

    def dense(qs, ks, vs):                               # qs [n,H,D] are the LAST n positions of ks/vs
        n, L = qs.shape[0], ks.shape[0]
        kk, vv = ks.repeat_interleave(H // HK, 1), vs.repeat_interleave(H // HK, 1)
        s = torch.einsum("qhd,khd->hqk", qs, kk) * D ** -0.5
        mask = torch.arange(L)[None, :] <= (torch.arange(n)[:, None] + L - n)
        s = s.masked_fill(~mask, float("-inf"))
        return torch.einsum("hqk,khd->qhd", s.softmax(-1), vv).reshape(n, H * D)

    want = torch.cat([dense(q[:19], k[:19], v[:19]), dense(q[19:], k[19:], v[19:])])
    torch.testing.assert_close(out[:T], want, rtol=1e-4, atol=1e-5)
    assert float(out[T:].abs().sum()) == 0               # padding rows stay untouched

    # decode: one new token per sequence
    q2, k2, v2 = torch.randn(2, H, D), torch.randn(2, HK, D), torch.randn(2, HK, D)
    new_slots = torch.tensor([bt[0, 19 // BS] * BS + 19 % BS, bt[1, 0] * BS + 7])
    md2 = builder.build(0, common(2, [0, 1, 2], [20, 8], 1, new_slots))
    assert md2.is_decode
    got = impl.forward(None, q2, k2, v2, kv_cache, md2)
    want2 = torch.cat([dense(q2[:1], torch.cat([k[:19], k2[:1]]), torch.cat([v[:19], v2[:1]])),
                       dense(q2[1:], torch.cat([k[19:], k2[1:]]), torch.cat([v[19:], v2[1:]]))])
    torch.testing.assert_close(got.reshape(2, H * D), want2, rtol=1e-4, atol=1e-5)
    # a profiling run without metadata returns zeros of the query's shape
    assert float(impl.forward(None, q2, k2, v2, kv_cache, None).abs().sum()) == 0


def test_no_adapter_class_is_left_abstract():
    """A class that leaves an abstract method of its vLLM base undefined imports fine and only fails
    when vLLM instantiates it."""
    pytest.importorskip("vllm")
    import importlib
    import inspect
    mods = ["omni_npu_b200.attention.vllm_backends", "omni_npu_b200.worker.vllm_worker",
            "omni_npu_b200.kv_transfer.vllm_connector", "omni_npu_b200.parallel.vllm_communicator",
            "omni_npu_b200.layers.vllm_custom_ops", "omni_npu_b200.models.vllm_adapters",
            "omni_npu_b200.sample.vllm_logits_processor", "omni_npu_b200.serving.parsers.vllm_adapters",
            "omni_npu_b200.platform"]
    abstract = []
    for mn in mods:
        m = importlib.import_module(mn)
        abstract += [f"{mn}.{n}: {sorted(c.__abstractmethods__)}" for n, c in vars(m).items()
                     if inspect.isclass(c) and c.__module__ == mn and inspect.isabstract(c)]
    assert abstract == []


def test_vllm_connector_wrapper_with_vllm_request_status(monkeypatch):
    """The wrapper builds from a vLLM-shaped config and hands out transfer parameters for a request
    that carries vLLM's own ``RequestStatus`` enum (not this package's)."""
    pytest.importorskip("vllm")
    import types

    from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorRole
    from vllm.v1.request import RequestStatus as VllmStatus

    from omni_npu_b200.kv_transfer.vllm_connector import B200ConnectorMetadata, B200KVConnector
    kt = types.SimpleNamespace(kv_connector="P2PKVConnector", kv_role="kv_producer", kv_rank=0, kv_parallel_size=1,
                               kv_ip="127.0.0.1", kv_port=25101, kv_connector_extra_config={"kv_port": 25101},
                               is_kv_producer=True, is_kv_consumer=False, engine_id="e0")
    vc = types.SimpleNamespace(kv_transfer_config=kt, cache_config=types.SimpleNamespace(block_size=16),
                               parallel_config=types.SimpleNamespace(tensor_parallel_size=1), additional_config={})
    c = B200KVConnector(vc, KVConnectorRole.SCHEDULER)
    try:
        assert c.role == KVConnectorRole.SCHEDULER
        req = types.SimpleNamespace(request_id="r", status=VllmStatus.FINISHED_LENGTH_CAPPED, spec_token_ids=[],
                                    num_prompt_tokens=20, kv_transfer_params=None)
        keep, params = c.request_finished(req, [4, 5])
        assert keep is True and params["remote_block_ids"] == [4, 5]
        stopped = types.SimpleNamespace(request_id="s", status=VllmStatus.FINISHED_STOPPED, spec_token_ids=[])
        assert c.request_finished(stopped, [6]) == (False, None)
        assert isinstance(c.build_connector_meta(None), B200ConnectorMetadata)
        assert c.get_num_new_matched_tokens(req, 0) == (0, False)
    finally:
        c.shutdown()


def test_model_adapter_translates_vllm_metadata_and_matches_the_inner_model(monkeypatch):
    """A standalone model behind the vLLM-facing adapter: config taken from a vLLM-shaped object,
    a profiling call without metadata, then a prefill whose metadata arrives through vLLM's forward
    context; hidden states must equal the inner model run under this package's own context."""
    pytest.importorskip("vllm")
    import types

    import vllm.forward_context as vfc

    from omni_npu_b200.attention.gqa import GQABackend
    from omni_npu_b200.attention.metadata import set_forward_context
    from omni_npu_b200.attention.vllm_backends import B200AttentionMetadata
    from omni_npu_b200.models.utils import random_init_
    from omni_npu_b200.models.vllm_adapters import StandaloneModelAdapter, metadata_from_vllm
    hf = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 64, "num_hidden_layers": 2,
          "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128,
          "vocab_size": 97, "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 256,
          "torch_dtype": "float32"}
    vc = types.SimpleNamespace(
        model_config=types.SimpleNamespace(hf_config=types.SimpleNamespace(**hf), dtype="float32", max_model_len=128),
        cache_config=types.SimpleNamespace(block_size=16), parallel_config=types.SimpleNamespace(tensor_parallel_size=1),
        scheduler_config=types.SimpleNamespace(max_num_seqs=4, max_num_batched_tokens=64), additional_config={})
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.float32)
    try:
        model = StandaloneModelAdapter(vllm_config=vc)
    finally:
        torch.set_default_dtype(prev)
    assert model.engine_config.model.num_layers == 2 and model.engine_config.scheduler.max_model_len == 128
    random_init_(model.inner, seed=2, std=0.1)
    caches = [GQABackend.allocate_kv_cache(8, 16, 2, 16, torch.float32, torch.device("cpu")) for _ in range(2)]
    model.bind_kv_caches(caches)
    lens = [9, 5]
    T = sum(lens)
    ids = torch.randint(0, 97, (T,))
    pos = torch.cat([torch.arange(n) for n in lens])
    bt = torch.tensor([[1, 0], [2, 0]], dtype=torch.int32)
    slots = torch.cat([bt[b, 0] * 16 + torch.arange(n) for b, n in enumerate(lens)]).to(torch.int32)
    md = B200AttentionMetadata(num_actual_tokens=T, num_reqs=2, max_query_len=9, max_seq_len=9,
                               query_start_loc=torch.tensor([0, 9, 14], dtype=torch.int32),
                               seq_lens=torch.tensor(lens, dtype=torch.int32), block_table=bt, slot_mapping=slots,
                               is_decode=False)
    ctx = types.SimpleNamespace(attn_metadata=None)
    monkeypatch.setattr(vfc, "get_forward_context", lambda: ctx)
    assert float(model(ids, pos).abs().sum()) == 0            # profiling run: zeros of the hidden size
    ctx.attn_metadata = {"model.layers.0.self_attn.attn": md}
    got = model(ids, pos)
    for k, v in caches:
        k.zero_(), v.zero_()
    with set_forward_context(metadata_from_vllm(md, pos), caches, model.engine_config):
        want = model.inner(ids, pos.to(torch.int32))
    torch.testing.assert_close(got, want)
    assert model.compute_logits(got).shape == (T, 97)


def test_worker_describes_sink_models_with_the_sink_spec():
    """Static attention sinks under vLLM: the worker names the sink length so that vLLM's sink manager
    takes the blocks after the null block out of circulation, and K / V head sizes may differ."""
    pytest.importorskip("vllm")
    import types

    import torch
    from vllm.v1.kv_cache_interface import FullAttentionSpec, SinkFullAttentionSpec

    from omni_npu_b200.worker.model_runner import KVCacheSpec
    from omni_npu_b200.worker.vllm_worker import B200Worker
    bs, hk, dk, dv, layers = 16, 2, 192, 128, 3
    per_layer = bs * hk * (dk + dv) * 2
    w = B200Worker.__new__(B200Worker)
    w.engine_config = types.SimpleNamespace(model=types.SimpleNamespace(dtype=torch.bfloat16, num_kv_heads=hk, head_dim=dk))
    w.model_runner = types.SimpleNamespace(get_kv_cache_spec=lambda: KVCacheSpec(
        "gqa", layers, bs, per_layer * layers, {"k": (hk, bs, dk), "v": (hk, bs, dv)}))
    for reserved, cls, sink in ((1 + 128 // bs, SinkFullAttentionSpec, 128), (0, FullAttentionSpec, None)):
        w.inner = types.SimpleNamespace(get_model=lambda r=reserved: types.SimpleNamespace(num_reserved_kv_blocks=r))
        specs = w.get_kv_cache_spec()
        assert len(specs) == layers
        s = specs["model.layers.0.self_attn.attn"]
        assert type(s) is cls and s.head_size == dk and s.head_size_v == dv and s.page_size_bytes == per_layer
        assert getattr(s, "sink_len", None) == sink


def test_grammar_bitmask_masks_the_rows_of_structured_requests_only():
    """The worker's bitmask application: one row of int32 words per structured request (bit set =
    token allowed), in vLLM's order of structured request ids, applied to the logits rows of the
    step in the step's own order."""
    import numpy as np
    import torch
    from omni_npu_b200.worker.vllm_worker import grammar_mask_fn
    vocab = 70                                            # three words, the last one partly used
    logits = torch.arange(3 * vocab, dtype=torch.float32).view(3, vocab)
    words = np.zeros((2, 3), dtype=np.uint32)
    words[0, 0] = (1 << 5) | (1 << 31)                    # request "c": tokens 5 and 31 (the sign bit of the int32 word)
    words[0, 2] = 1 << 3                                  # ... and token 67
    words[1, 1] = 1 << 1                                  # request "a": token 33
    words = words.view(np.int32)
    fn = grammar_mask_fn(["a", "b", "c"], ["c", "a", "gone"], np.vstack([words, np.full((1, 3), -1, dtype=np.int32)]))
    out = fn(logits.clone())
    assert torch.equal(out[1], logits[1])                                 # "b" is not structured
    assert torch.isfinite(out[0]).nonzero().flatten().tolist() == [33]    # "a" takes the second bitmask row
    assert torch.isfinite(out[2]).nonzero().flatten().tolist() == [5, 31, 67]
    assert out[2, 67] == logits[2, 67]


def test_runner_applies_a_step_logits_adjustment_before_sampling():
    """``ModelRunner.extra_logits_fn`` (what the vLLM worker installs for a structured-output step)
    is applied to the step's logits rows: with every token but one masked, that token is sampled,
    and the step runs eagerly."""
    import torch
    from omni_npu_b200 import SamplingParams
    from omni_npu_b200.config import ModelConfig
    from omni_npu_b200.engine.llm import LLM
    cfg = ModelConfig(hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128,
                      vocab_size=97, rope_theta=10000.0, max_position_embeddings=512, dtype=torch.float32)
    llm = LLM(model=cfg, device="cpu", max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, block_size=4,
              num_gpu_blocks=64, seed=3, additional_config={"async_scheduling": False})
    runner = llm.engine.worker.model_runner

    def only_token_42(logits):
        masked = torch.full_like(logits, float("-inf"))
        masked[:, 42] = logits[:, 42]
        return masked
    runner.extra_logits_fn = only_token_42
    try:
        outs = llm.generate([[1, 2, 3, 4, 5], [9, 8, 7]], SamplingParams(max_tokens=4, ignore_eos=True))
    finally:
        runner.extra_logits_fn = None
    assert all(o.output_token_ids == [42] * 4 for o in outs)
    free = llm.generate([[1, 2, 3, 4, 5]], SamplingParams(max_tokens=4, ignore_eos=True))
    assert free[0].output_token_ids != [42] * 4
