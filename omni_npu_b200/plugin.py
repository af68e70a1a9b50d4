"""vLLM platform-plugin entry point.

``plugin()`` is registered under the ``vllm.platform_plugins`` entry-point
group.  It returns the dotted path of the platform class when a Blackwell
(compute capability 10.x) CUDA device is visible and the native extension is
available, otherwise ``None`` so vLLM falls back to its built-in platforms.
An activated out-of-tree platform takes precedence over the built-in CUDA
platform.  (Counterpart of omni_npu/vllm_plugin.py:1-23, which probes for
``torch_npu`` instead.)

Set ``OMNI_B200_PLUGIN=0`` to keep the plugin dormant, ``=force`` to activate
it on any CUDA device, ``=cpu`` to activate the CPU / gloo variant of the
platform (plumbing tests of the worker and model runner without a GPU).

vLLM finds entry points through installed package metadata (``pip install -e .``).
``write_entry_point_metadata`` writes that metadata into a directory of the
caller's choice instead, for running from a source tree that is not installed:
put the directory on ``PYTHONPATH``.
"""
from __future__ import annotations

import os
from typing import Optional

PLATFORM_CLS = "omni_npu_b200.platform.B200Platform"
CPU_PLATFORM_CLS = "omni_npu_b200.platform.B200CpuPlatform"


def plugin() -> Optional[str]:
    mode = os.environ.get("OMNI_B200_PLUGIN", "1").lower()
    if mode in ("0", "off", "false"):
        return None
    if mode == "cpu":
        return CPU_PLATFORM_CLS
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


def write_entry_point_metadata(directory: str) -> str:
    """Write ``omni_npu_b200-<version>.dist-info`` (METADATA + entry_points.txt) into
    ``directory`` and return its path.  With ``directory`` on ``sys.path`` / ``PYTHONPATH`` the
    platform, patch and model plugins are discovered exactly as after ``pip install``."""
    info = os.path.join(directory, "omni_npu_b200-0.1.0.dist-info")
    os.makedirs(info, exist_ok=True)
    with open(os.path.join(info, "METADATA"), "w") as f:
        f.write("Metadata-Version: 2.1\nName: omni-npu-b200\nVersion: 0.1.0\n")
    with open(os.path.join(info, "entry_points.txt"), "w") as f:
        f.write("[vllm.platform_plugins]\nomni-npu-b200 = omni_npu_b200.plugin:plugin\n\n"
                "[vllm.general_plugins]\nomni_b200_patches = omni_npu_b200.patches:apply_patches\n"
                "omni_b200_models = omni_npu_b200.models.registry:register_models\n")
    return info
