"""Per-descriptor capture / replay cache with the CUDA runtime replaced by a recording fake:
capture happens once per descriptor, later calls replay, prefill-like calls (no descriptor or
mode NONE) run eagerly, the debug mode notices inputs that moved, and outputs are held weakly."""
import contextlib
import gc

import pytest
import torch

from omni_npu_b200 import ops
from omni_npu_b200.compilation import cuda_graph as cg


class _FakeStream:
    def wait_stream(self, other):
        pass


class _FakeGraph:
    instances = []

    def __init__(self):
        self.replays = 0
        _FakeGraph.instances.append(self)

    def replay(self):
        self.replays += 1

    def pool(self):
        return ("pool", id(self))


@pytest.fixture
def fake_cuda(monkeypatch):
    _FakeGraph.instances = []
    pools = []

    @contextlib.contextmanager
    def graph(g, pool=None):
        pools.append(pool)
        yield

    @contextlib.contextmanager
    def stream(s):
        yield

    monkeypatch.setattr(torch.cuda, "Stream", lambda device=None: _FakeStream())
    monkeypatch.setattr(torch.cuda, "current_stream", lambda device=None: _FakeStream())
    monkeypatch.setattr(torch.cuda, "stream", stream)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda device=None: None)
    monkeypatch.setattr(torch.cuda, "CUDAGraph", _FakeGraph)
    monkeypatch.setattr(torch.cuda, "graph", graph)
    return pools


def test_capture_once_then_replay_per_descriptor(fake_cuda):
    calls = []

    def model(x):
        calls.append(x.shape[0])
        return x + 1

    w = cg.CUDAGraphWrapper(model, torch.device("cuda", 0), debug=True)
    x4, x8 = torch.zeros(4), torch.zeros(8)
    d4, d8 = cg.BatchDescriptor(4), cg.BatchDescriptor(8)
    out = w(d4, x4)
    assert calls == [4, 4]                          # one warm-up run + the captured run
    assert torch.equal(out, torch.ones(4))
    before = ops.launch_count()
    assert w(d4, x4) is out and calls == [4, 4]     # replay: the callable does not run again
    assert _FakeGraph.instances[0].replays == 1
    assert ops.launch_count() == before + w.entries[d4].runner.num_kernels
    w(d8, x8)
    assert len(_FakeGraph.instances) == 2 and calls == [4, 4, 8, 8]
    assert fake_cuda == [None, _FakeGraph.instances[0].pool()]     # later captures share the first pool
    assert set(w.entries) == {d4, d8}


def test_eager_paths_and_moved_inputs(fake_cuda):
    calls = []

    def model(x):
        calls.append("run")
        return x * 2

    w = cg.CUDAGraphWrapper(model, torch.device("cuda", 0), debug=True)
    x = torch.ones(3)
    assert torch.equal(w(None, x), x * 2) and not w.entries                 # prefill: no descriptor
    assert torch.equal(w(cg.BatchDescriptor(3), x, mode="NONE"), x * 2) and not w.entries
    cpu = cg.CUDAGraphWrapper(model, torch.device("cpu"))
    assert torch.equal(cpu(cg.BatchDescriptor(3), x), x * 2) and not cpu.entries
    d = cg.BatchDescriptor(3)
    w(d, x)
    with pytest.raises(RuntimeError, match="inputs moved"):
        w(d, torch.ones(3))                                                 # another buffer: refused in debug mode
    relaxed = cg.CUDAGraphWrapper(model, torch.device("cuda", 0), debug=False)
    relaxed(d, x)
    relaxed(d, torch.ones(3))                                               # not checked outside debug mode


def test_outputs_are_held_weakly_and_attributes_pass_through(fake_cuda):
    class Out:
        pass

    class Model:
        hidden_size = 64

        def __call__(self, x):
            return Out()

    m = Model()
    w = cg.CUDAGraphWrapper(m, torch.device("cuda", 0))
    d = cg.BatchDescriptor(2)
    out = w(d, torch.zeros(2))
    assert w.entries[d].output_ref() is out
    assert w.hidden_size == 64                      # unknown attributes resolve on the wrapped callable
    # the runner keeps the captured output alive (it is what a replay returns); the cache entry does not add a
    # second strong reference
    runner = w.entries[d].runner
    runner.output = None
    del out
    gc.collect()
    assert w.entries[d].output_ref() is None


def test_vllm_compile_decorator_patch_bypasses_prefill_and_non_full_modes():
    import types

    from omni_npu_b200.compilation import decorators as dec

    log = []

    def fake_support(cls):                 # stands in for vLLM's class preparation
        def compiled_call(self, x):
            log.append("compiled")
            return ([x + 100],)
        cls.__call__ = compiled_call
        return cls

    mod = types.SimpleNamespace(_support_torch_compile=fake_support)
    ctx = types.SimpleNamespace(attn_metadata=None, cudagraph_runtime_mode="FULL")
    assert dec.patch_compile_decorators(mod, lambda: ctx, "FULL")
    assert dec.patch_compile_decorators(mod, lambda: ctx, "FULL")          # idempotent
    assert mod._support_torch_compile._omni_original is fake_support

    class Model:
        def forward(self, x):
            log.append("eager")
            return x + 1

    Model = mod._support_torch_compile(Model)
    m = Model()
    one = torch.tensor(1)
    assert m(one) == 2 and log == ["eager"]                                # profile run: no metadata
    ctx.attn_metadata = {"layer.0": types.SimpleNamespace(num_prefills=2)}
    assert m(one) == 2 and log == ["eager", "eager"]                       # a prefill in the batch
    ctx.attn_metadata = {"layer.0": types.SimpleNamespace(num_prefills=0)}
    out = m(one)
    assert torch.is_tensor(out) and out == 101 and log[-1] == "compiled"   # pure decode, FULL: graph path, unwrapped
    ctx.cudagraph_runtime_mode = "PIECEWISE"
    assert m(one) == 2 and log[-1] == "eager"
    dec.unpatch_compile_decorators(mod)
    assert mod._support_torch_compile is fake_support


def test_vllm_compile_decorator_patch_installs_on_the_real_module():
    pytest.importorskip("vllm")
    import vllm.compilation.decorators as vdec

    from omni_npu_b200.compilation import decorators as dec
    before = vdec._support_torch_compile
    try:
        assert dec.patch_compile_decorators()
        assert vdec._support_torch_compile._omni_original is before
    finally:
        dec.unpatch_compile_decorators()
    assert vdec._support_torch_compile is before
