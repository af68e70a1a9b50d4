"""Response parsers: reasoning extraction and tool-call extraction for Pangu models.

``register_lazy_parsers`` makes them available to vLLM's OpenAI server as
``--reasoning-parser pangu`` / ``--tool-call-parser pangu`` when vLLM is
importable (omni_npu/v1/parsers/__init__.py:16-35); without vLLM they are used
by this package's own server."""
from __future__ import annotations

from .pangu_reasoning_parser import PanguReasoningParser  # noqa: F401
from .pangu_tool_parser import PanguToolParser  # noqa: F401

PARSER_NAME = "pangu"


def register_lazy_parsers() -> bool:
    from ... import compat
    if not compat.vllm_available():
        return False
    ok = False
    try:
        mgr = compat.reasoning_parser_manager()
        if hasattr(mgr, "register_lazy_module"):
            mgr.register_lazy_module(PARSER_NAME, "omni_npu_b200.serving.parsers.vllm_adapters",
                                     "VllmPanguReasoningParser")
        else:
            from .vllm_adapters import VllmPanguReasoningParser
            mgr.register_module(PARSER_NAME, module=VllmPanguReasoningParser, force=True)
        ok = True
    except Exception:
        pass
    try:
        mgr = compat.tool_parser_manager()
        if hasattr(mgr, "register_lazy_module"):
            mgr.register_lazy_module(PARSER_NAME, "omni_npu_b200.serving.parsers.vllm_adapters",
                                     "VllmPanguToolParser")
        else:
            from .vllm_adapters import VllmPanguToolParser
            mgr.register_module(PARSER_NAME, module=VllmPanguToolParser, force=True)
        ok = True
    except Exception:
        pass
    return ok
