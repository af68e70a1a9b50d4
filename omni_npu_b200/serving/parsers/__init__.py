"""Response parsers: reasoning extraction and tool-call extraction for Pangu models.

``register_lazy_parsers`` makes them available to vLLM's OpenAI server as
``--reasoning-parser pangu`` / ``--tool-call-parser pangu`` when vLLM is
importable (omni_npu/v1/parsers/__init__.py:16-35); without vLLM they are used
by this package's own server."""
from __future__ import annotations

from .pangu_reasoning_parser import PanguReasoningParser  # noqa: F401
from .pangu_tool_parser import PanguToolParser  # noqa: F401

PARSER_NAME = "pangu"

_REASONING = {PARSER_NAME: PanguReasoningParser}
_TOOLS = {PARSER_NAME: PanguToolParser}


def get_reasoning_parser(name: str):
    """Parser class for ``--reasoning-parser <name>`` of this package's own server."""
    try:
        return _REASONING[name]
    except KeyError:
        raise ValueError(f"unknown reasoning parser {name!r}; known: {sorted(_REASONING)}") from None


def get_tool_parser(name: str):
    try:
        return _TOOLS[name]
    except KeyError:
        raise ValueError(f"unknown tool-call parser {name!r}; known: {sorted(_TOOLS)}") from None


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
