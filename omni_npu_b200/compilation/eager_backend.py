"""Compile backend handed to vLLM when it insists on one: run the captured FX graph as is.

On B200 the decode step is replayed from a CUDA graph and the kernels are hand written, so
no tracing compiler sits on the hot path; vLLM's compilation level is forced to "no
compilation" by the platform, and where a ``backend`` object is still requested this one
returns the graph module's own ``forward``.  (The reference offers ``NpuGraphExAdaptor`` /
torchair GE compilation here: omni_npu/compilation/npugraph_ex.py, ge_wrapper.py:100-199.)
"""
from __future__ import annotations

from typing import Any, Callable, List


class EagerGraphBackend:
    def __init__(self, *args: Any, **kwargs: Any) -> None:
        self.compiled_graphs = 0

    def __call__(self, graph_module, example_inputs: List[Any]) -> Callable:
        self.compiled_graphs += 1
        return graph_module.forward

    def compute_hash(self, *args: Any, **kwargs: Any) -> str:
        return "b200-eager"
