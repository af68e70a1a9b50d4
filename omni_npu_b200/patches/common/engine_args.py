"""CLI / engine-argument additions.

* ``--enable-kv-rmsnorm-rope-cache``  use the fused KV RMSNorm + RoPE + cache-write
  kernel (default on; the flag exists so that launch scripts written for the
  reference keep working, omni_npu/vllm_patches/patches/common/patch_engine_args.py:17-115);
* ``--reasoning-config '<json>'``      thinking-token budget configuration
  (omni_npu/vllm_patches/patches/common/patch_think_limit.py:57-66);
* ``--device``                         accepted and checked: the platform is chosen
  by the plugin, ``cuda`` / ``auto`` are the only valid values.

When vLLM is importable the patches below extend its ``EngineArgs``; without
vLLM ``add_cli_args`` still works on a plain ``argparse`` parser (used by this
package's own server).
"""
from __future__ import annotations

import argparse
import json
from typing import Any, Dict

from ... import compat
from ..core import Patch, register_patch


def add_cli_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    existing = {a for act in parser._actions for a in act.option_strings}
    if "--enable-kv-rmsnorm-rope-cache" not in existing:
        parser.add_argument("--enable-kv-rmsnorm-rope-cache", action="store_true", default=True,
                            help="fuse KV RMSNorm, RoPE and the paged-cache write into one kernel")
    if "--reasoning-config" not in existing:
        parser.add_argument("--reasoning-config", type=json.loads, default=None,
                            help='JSON, e.g. {"think_start_str": "<think>", "think_end_str": "</think>"}')
    if "--device" not in existing:
        parser.add_argument("--device", default="auto", choices=["auto", "cuda", "cpu"],
                            help="device type; the B200 platform plugin serves 'cuda'")
    return parser


def additional_config_from_args(ns: argparse.Namespace) -> Dict[str, Any]:
    out: Dict[str, Any] = {}
    if getattr(ns, "enable_kv_rmsnorm_rope_cache", None) is not None:
        out["enable_kv_rmsnorm_rope_cache"] = bool(ns.enable_kv_rmsnorm_rope_cache)
    if getattr(ns, "reasoning_config", None):
        out["reasoning_config"] = ns.reasoning_config
    return out


if compat.vllm_available():
    try:
        from vllm.engine.arg_utils import EngineArgs as _EngineArgs

        _orig_add_cli_args = _EngineArgs.__dict__["add_cli_args"]

        @register_patch("EngineArgsPatch", _EngineArgs)
        class EngineArgsPatch(Patch):
            attributes = ["add_cli_args"]

            @staticmethod
            def add_cli_args(parser, *a, **kw):
                fn = _orig_add_cli_args.__func__ if hasattr(_orig_add_cli_args, "__func__") else _orig_add_cli_args
                parser = fn(parser, *a, **kw)
                grp = parser
                try:
                    add_cli_args(grp)
                except argparse.ArgumentError:
                    pass
                return parser
    except Exception:  # pragma: no cover - depends on the vLLM version
        pass
