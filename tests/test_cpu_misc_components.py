"""Small components: group-scoped comm helpers, graph-mode config / decorators, tracing."""
import pytest
import torch

from omni_npu_b200.attention.metadata import AttentionMetadata, set_forward_context
from omni_npu_b200.compilation.config import B200CompilationConfig
from omni_npu_b200.compilation.decorators import step_is_capturable, support_graph_replay
from omni_npu_b200.parallel import comm_ops, state
from omni_npu_b200.utils import trace


def test_comm_ops_are_identity_on_one_rank():
    state.ensure_initialized(torch.device("cpu"))
    x = torch.arange(12.0).view(4, 3)
    for fn in (comm_ops.all_reduce, comm_ops.all_reduce_two_stage):
        assert fn(x) is x
    assert comm_ops.all_gather(x, 0) is x and comm_ops.reduce_scatter(x, 0) is x
    assert comm_ops.all_gather_pipeline(x) is x and comm_ops.all_gather_local(x) is x
    assert comm_ops.all_to_all(x) is x and comm_ops.sequence_parallel_chunk(x) is x
    assert comm_ops.get_world_size() == 1 and comm_ops.get_rank("mlp.down_proj") == 0


def test_compilation_config_gears():
    cfg = B200CompilationConfig.from_additional_config({"decode_gear_list": [8, 2, 32]}, max_num_seqs=48)
    assert cfg.decode_gear_list == [2, 8, 32, 48]            # the largest gear covers a full batch
    gears = cfg.gears(48)
    assert cfg.pad_to_gear(1, gears) == 2 and cfg.pad_to_gear(9, gears) == 32 and cfg.pad_to_gear(49, gears) is None
    auto = B200CompilationConfig().gears(128)
    assert auto[:5] == [1, 2, 4, 8, 16] and auto[-1] == 128
    assert B200CompilationConfig(cudagraph_mode="NONE").gears(128) == []
    with pytest.raises(ValueError):
        B200CompilationConfig.from_additional_config({"cudagraph_mode": "PIECEWISE"})
    with pytest.raises(ValueError):
        B200CompilationConfig.from_additional_config({"decode_gear_list": list(range(1, 80))})


def _md(prefill):
    z = torch.zeros(1, dtype=torch.int32)
    return AttentionMetadata(prefill, 1, 1, 1, 1, 1, z, z, z.view(1, 1), z, torch.zeros(2, dtype=torch.int32), 1, 1)


def test_prefill_bypasses_the_graph_path():
    calls = []

    @support_graph_replay
    class M:
        device = torch.device("cpu")
        cudagraph_mode = "NONE"

        def forward(self, x):
            calls.append("forward")
            return x + 1

        def __call__(self, x):
            calls.append("call")
            return self.forward(x)

    m = M()
    assert M._graph_bypass_installed
    with set_forward_context(_md(True), []):
        assert m(torch.ones(1)).item() == 2
    with set_forward_context(_md(False), []):
        assert m(torch.ones(1)).item() == 2                  # mode NONE: eager as well
    assert calls == ["forward", "forward"]
    assert not step_is_capturable(_md(True), "FULL_DECODE_ONLY") and step_is_capturable(_md(False), "FULL_DECODE_ONLY")


def test_trace_timers_and_request_lines():
    trace.enable(True)
    try:
        @trace.timer("unit.work")
        def work(n):
            return sum(range(n))

        work(10), work(20)
        rep = trace.timer_report(reset=True)
        assert rep["unit.work"]["calls"] == 2 and rep["unit.work"]["total_s"] >= 0
        lines = []
        t = trace.RequestTracer(role="prefill", sink=lines.append)
        line = t.trace("first_token", "req-1", ttft_ms=12.5)
        assert lines == [line] and "event=first_token" in line and "role=prefill" in line and "ttft_ms=12.5" in line
        with trace.nvtx_range("block"):
            pass
    finally:
        trace.enable(False)
    assert trace.RequestTracer(sink=lambda l: (_ for _ in ()).throw(AssertionError)).trace("x", "r")


def test_sharded_rows_fall_back_to_gather_without_peer_memory():
    """A column-parallel projection handed token shards either fuses the gather into its GEMM
    (peer memory, GPU) or asks the stream for the gathered rows; on CPU it must be the latter."""
    import torch
    from omni_npu_b200.layers.flashcomm import SequenceParallelStream, ShardedRows
    from omni_npu_b200.layers.linear import ColumnParallelLinear, MergedColumnParallelLinear
    from omni_npu_b200.parallel import state
    state.ensure_initialized(torch.device("cpu"))
    sp = SequenceParallelStream(state.get_tp_group())
    x = torch.randn(6, 16)
    shard = sp.scatter(x)
    lin = ColumnParallelLinear(16, 8, dtype=torch.float32)
    lin.weight.data.normal_()
    rows = ShardedRows(shard, sp)
    assert rows.shape == (6, 16)
    assert torch.allclose(lin(rows), x @ lin.weight.t(), atol=1e-5)
    merged = MergedColumnParallelLinear(16, [8, 8], dtype=torch.float32)
    merged.weight.data.normal_()
    assert torch.allclose(merged(ShardedRows(shard, sp)), x @ merged.weight.t(), atol=1e-5)


def test_stop_buffer_is_not_applied_inside_the_reasoning_span():
    from omni_npu_b200.patches.common.think_stream import hold_back, reasoning_finished
    assert not reasoning_finished([1, 2, 3])
    assert not reasoning_finished([5, 151668])                   # end marker just emitted, no newline yet
    assert reasoning_finished([5, 151668, 271, 9])               # Qwen3: </think> then a blank line
    assert reasoning_finished([128799, 201])                     # DeepSeek-R1
    assert not reasoning_finished([151668, 7])
    assert reasoning_finished([9, 8, 7], {8: (7,)})              # ids from a reasoning config
    assert hold_back(5, finished=False, done_reasoning=False, new_text="abc") == 0
    assert hold_back(5, finished=False, done_reasoning=True, new_text="x</think>\n") == 0
    assert hold_back(5, finished=False, done_reasoning=True, new_text="answer") == 5
    assert hold_back(5, finished=True, done_reasoning=True, new_text="answer") == 0


def test_trace_namelist_wraps_functions_by_name(tmp_path):
    from omni_npu_b200.engine.block_manager import BlockPool
    from omni_npu_b200.utils import trace
    spec = tmp_path / "names.yaml"
    spec.write_text("type: timer\ntargets:\n  - module: omni_npu_b200.engine.block_manager:BlockPool\n"
                    "    function_name: [allocate, free]\n")
    original = BlockPool.allocate
    try:
        assert trace.apply_namelist(str(spec)) == 2
        assert trace.apply_namelist(str(spec)) == 0              # already wrapped: not wrapped twice
        trace.enable(True)
        trace.timer_report(reset=True)
        pool = BlockPool(8, 4)
        pool.free(pool.allocate(3))
        rep = trace.timer_report()
        key = "omni_npu_b200.engine.block_manager:BlockPool.allocate"
        assert rep[key]["calls"] == 1 and pool.num_free == 8
    finally:
        trace.enable(False)
        BlockPool.allocate = original
        BlockPool.free = BlockPool.free.__wrapped__


def test_status_word_created_under_inference_mode_can_be_cleared_outside(monkeypatch):
    """The first kernel of a process usually runs under inference_mode; the status word it creates
    must still be clearable by a caller outside that mode (``check_status`` after a timeout)."""
    import torch
    from omni_npu_b200 import ops
    monkeypatch.setattr(ops, "_states", {})
    with torch.inference_mode():
        st = ops._DeviceState(torch.device("cpu"))
    assert not st.status.is_inference()
    st.status.fill_(5)
    ops._states[0] = st
    import pytest
    with pytest.raises(RuntimeError, match="status 5"):
        ops.check_status()
    ops.check_status()


def test_pp_layer_range_splits_evenly_and_honours_override(monkeypatch):
    from omni_npu_b200.models.utils import PPMissingLayer, pp_layer_range
    monkeypatch.delenv("OMNI_B200_PP_LAYER_PARTITION", raising=False)
    assert [pp_layer_range(8, r, 2) for r in range(2)] == [(0, 4), (4, 8)]
    spans = [pp_layer_range(10, r, 4) for r in range(4)]
    assert spans[0][0] == 0 and spans[-1][1] == 10
    assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    sizes = [e - s for s, e in spans]
    assert sorted(sizes) == [2, 2, 3, 3] and sizes[1] == 3 and sizes[2] == 3   # middle stages take the remainder
    monkeypatch.setenv("OMNI_B200_PP_LAYER_PARTITION", "1,5,2")
    assert [pp_layer_range(8, r, 3) for r in range(3)] == [(0, 1), (1, 6), (6, 8)]
    monkeypatch.setenv("OMNI_B200_PP_LAYER_PARTITION", "4,5")
    import pytest as _pt
    with _pt.raises(ValueError):
        pp_layer_range(8, 0, 2)
    x = torch.ones(2)
    assert PPMissingLayer()(x) is x and not list(PPMissingLayer().parameters())


def test_public_ops_dispatch_through_the_ops_module_not_the_reference():
    """Every op that has a CUDA kernel must be defined in ``ops`` itself (device dispatch), never
    be a bare alias of its CPU reference: an alias would silently run tensor ops on the GPU."""
    from omni_npu_b200 import ops
    from omni_npu_b200.ops import ref
    import types
    aliased = [name for name in dir(ops)
               if isinstance(getattr(ops, name), types.FunctionType) and getattr(ref, name, None) is getattr(ops, name)]
    assert aliased == []


def test_every_name_imported_inside_the_package_exists():
    """``from .module import Name`` statements that sit inside functions or behind
    ``contextlib.suppress`` only fail when (or never visibly where) they run; resolve all of them here."""
    import ast
    import importlib
    import pathlib
    root = pathlib.Path(__file__).resolve().parent.parent / "omni_npu_b200"
    missing = []
    for f in sorted(root.rglob("*.py")):
        parts = list(f.relative_to(root.parent).with_suffix("").parts)
        is_pkg = parts[-1] == "__init__"
        if is_pkg:
            parts = parts[:-1]
        for node in ast.walk(ast.parse(f.read_text())):
            if not isinstance(node, ast.ImportFrom) or node.level == 0:
                continue
            base = parts if is_pkg else parts[:-1]
            base = base[: len(base) - (node.level - 1)]
            target = ".".join(base + ([node.module] if node.module else []))
            try:
                mod = importlib.import_module(target)
            except ImportError as e:
                missing.append(f"{f.name}: cannot import {target}: {e}")
                continue
            for alias in node.names:
                if alias.name == "*" or hasattr(mod, alias.name):
                    continue
                try:
                    importlib.import_module(f"{target}.{alias.name}")
                except ImportError:
                    missing.append(f"{f.name}: {target} has no {alias.name}")
    assert missing == []
