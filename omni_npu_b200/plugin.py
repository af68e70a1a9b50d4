"""vLLM platform-plugin entry point.

``plugin()`` is registered under the ``vllm.platform_plugins`` entry-point
group.  It returns the dotted path of the platform class when a Blackwell
(compute capability 10.x) CUDA device is visible and the native extension is
available, otherwise ``None`` so vLLM falls back to its built-in platforms.
An activated out-of-tree platform takes precedence over the built-in CUDA
platform.  (Counterpart of omni_npu/vllm_plugin.py:1-23, which probes for
``torch_npu`` instead.)

Set ``OMNI_B200_PLUGIN=0`` to keep the plugin dormant, ``=force`` to activate
it on any CUDA device.
"""
from __future__ import annotations

import os
from typing import Optional

PLATFORM_CLS = "omni_npu_b200.platform.B200Platform"


def plugin() -> Optional[str]:
    mode = os.environ.get("OMNI_B200_PLUGIN", "1").lower()
    if mode in ("0", "off", "false"):
        return None
    try:
        import torch
    except Exception:
        return None
    try:
        if not torch.cuda.is_available() or torch.cuda.device_count() == 0:
            return None
        major, _ = torch.cuda.get_device_capability(0)
    except Exception:
        return None
    if major != 10 and mode != "force":
        return None
    from . import ops
    if not ops.load_extension(required=False):
        return None
    return PLATFORM_CLS
