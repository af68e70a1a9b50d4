"""Thin shims over the installed vLLM version.

Everything that touches vLLM imports through this module so that version drift
shows up in one place (and in tests/test_vllm_interface.py, which snapshots the
signatures this package relies on).  The reference is written against vLLM
0.12; the container ships a newer release in which several modules moved
(``vllm.attention.*`` -> ``vllm.v1.attention.*`` and friends).
"""
from __future__ import annotations

import importlib
from typing import Any, Optional

_vllm = None
_checked = False


def vllm_available() -> bool:
    global _vllm, _checked
    if not _checked:
        _checked = True
        try:
            _vllm = importlib.import_module("vllm")
        except Exception:
            _vllm = None
    return _vllm is not None


def vllm_version() -> Optional[str]:
    return getattr(_vllm, "__version__", None) if vllm_available() else None


def try_import(*candidates: str) -> Any:
    """Import the first module / attribute path that exists.  A candidate is
    ``"pkg.module"`` or ``"pkg.module:attr"``."""
    last: Optional[Exception] = None
    for cand in candidates:
        mod, _, attr = cand.partition(":")
        try:
            m = importlib.import_module(mod)
            return getattr(m, attr) if attr else m
        except Exception as e:  # pragma: no cover - depends on vLLM version
            last = e
    raise ImportError(f"none of {candidates} could be imported: {last}")


def platform_base():
    return try_import("vllm.platforms.interface:Platform")


def platform_enum():
    return try_import("vllm.platforms.interface:PlatformEnum")


def worker_base():
    return try_import("vllm.v1.worker.worker_base:WorkerBase")


def kv_connector_base():
    return try_import("vllm.distributed.kv_transfer.kv_connector.v1.base:KVConnectorBase_V1")


def kv_connector_factory():
    return try_import("vllm.distributed.kv_transfer.kv_connector.factory:KVConnectorFactory")


def model_registry():
    return try_import("vllm:ModelRegistry")


def reasoning_parser_manager():
    return try_import("vllm.reasoning:ReasoningParserManager")


def tool_parser_manager():
    return try_import("vllm.tool_parsers:ToolParserManager",
                      "vllm.entrypoints.openai.tool_parsers:ToolParserManager")


def custom_op_base():
    return try_import("vllm.model_executor.custom_op:CustomOp")
