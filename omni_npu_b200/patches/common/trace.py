"""Name-list driven tracing for vLLM processes.

With ``PROFILING_NAMELIST=<yaml>`` set, importing this module (the patch entry point imports
every module under ``patches/common``) wraps the functions the list names with timers / NVTX
ranges (``utils.trace.apply_namelist``), in the API-server process and in every worker, before
the engine starts.  Without the variable nothing is touched.  The standalone engine does the
same from ``Worker.init_device`` and writes the request life-cycle lines itself
(``utils.trace.request_event``).
(reference: omni_npu/vllm_patches/patches/common/patch_trace.py:60-227)
"""
from __future__ import annotations

import os

from ...logger import logger

wrapped = 0
if os.environ.get("PROFILING_NAMELIST"):
    try:
        from ...utils.trace import apply_namelist
        wrapped = apply_namelist()
        logger.info("tracing: wrapped %d functions named by %s", wrapped, os.environ["PROFILING_NAMELIST"])
    except Exception as e:  # a broken name list must not keep the server from starting
        logger.warning("tracing disabled: %s", e)
