"""Smallest possible patches, as a how-to (counterpart of
omni_npu/vllm_patches/patches/examples/llm_engine_hello_world.py:12-34).

    OMNI_B200_VLLM_PATCHES=HelloWorldRequest python ...
"""
from __future__ import annotations

from ...engine import request as _request
from ..core import Patch, register_patch


@register_patch("HelloWorldRequest", _request.Request)
class HelloWorldRequest(Patch):
    attributes = ["hello"]

    def hello(self) -> str:
        return f"hello from request {self.request_id}"
