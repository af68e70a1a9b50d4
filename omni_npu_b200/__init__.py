"""omni_npu_b200: a Blackwell (B200, sm_100a) native LLM serving framework with the
capabilities of the omni-npu vLLM platform plugin.

Public API:
    LLM, SamplingParams, EngineConfig, ModelConfig      offline / embedded serving
    omni_npu_b200.plugin:plugin                         vLLM platform-plugin entry point
    omni_npu_b200.ops                                   device kernels
"""
__version__ = "0.1.0"

from .config import EngineConfig, ModelConfig  # noqa: F401
from .engine.request import RequestOutput, SamplingParams  # noqa: F401


def __getattr__(name):
    if name in ("LLM", "LLMEngine", "build_engine_config"):
        from .engine import llm as _llm
        return getattr(_llm, name)
    raise AttributeError(name)
