"""Entry point ``apply_patches`` (a ``vllm.general_plugins`` plugin): imports the
patch modules so that they register themselves, then applies the ones selected
through the environment.

Import order follows the reference (omni_npu/vllm_patches/__init__.py:85-181):
``common/*`` first, then the directory under ``models/`` named after the
``model_type`` of the model being served (taken from the ``--model`` /
positional argument's ``config.json``, or ``OMNI_B200_PATCHES_DIR`` /
``OMNI_NPU_PATCHES_DIR``).
"""
from __future__ import annotations

import importlib
import json
import os
import pkgutil
import sys
from pathlib import Path
from typing import List, Optional

from ..logger import logger
from .core import Patch, PatchRegistry, register_patch  # noqa: F401

_manager: Optional[PatchRegistry] = None


def _model_path_from_argv(argv: List[str]) -> Optional[str]:
    for i, a in enumerate(argv):
        if a in ("--model",) and i + 1 < len(argv):
            return argv[i + 1]
        if a.startswith("--model="):
            return a.split("=", 1)[1]
    if len(argv) > 2 and argv[1] == "serve" and not argv[2].startswith("-"):
        return argv[2]
    return None


def detect_model_type(argv: Optional[List[str]] = None) -> Optional[str]:
    path = _model_path_from_argv(argv if argv is not None else sys.argv)
    if not path:
        return None
    cfg = os.path.join(path, "config.json")
    try:
        with open(cfg) as f:
            return json.load(f).get("model_type")
    except Exception:
        return None


def _import_package_modules(pkg_name: str) -> List[str]:
    done = []
    try:
        pkg = importlib.import_module(pkg_name)
    except Exception as e:
        logger.debug("patch package %s not importable: %s", pkg_name, e)
        return done
    for info in pkgutil.iter_modules(pkg.__path__):
        if info.name.startswith("_"):
            continue
        try:
            importlib.import_module(f"{pkg_name}.{info.name}")
            done.append(info.name)
        except Exception as e:
            logger.warning("patch module %s.%s failed to import: %s", pkg_name, info.name, e)
    return done


def auto_import_patches(argv: Optional[List[str]] = None) -> List[str]:
    imported = _import_package_modules(f"{__name__}.common")
    model_dir = os.environ.get("OMNI_B200_PATCHES_DIR", os.environ.get("OMNI_NPU_PATCHES_DIR"))
    if not model_dir:
        mt = detect_model_type(argv)
        if mt:
            model_dir = mt.replace("-", "_")
    if model_dir and (Path(__file__).parent / "models" / model_dir).is_dir():
        imported += _import_package_modules(f"{__name__}.models.{model_dir}")
    return imported


def apply_patches() -> PatchRegistry:
    global _manager
    if _manager is None:
        _manager = PatchRegistry()
    auto_import_patches()
    try:
        from ..models.registry import register_models
        register_models()
    except Exception as e:
        logger.debug("model registration skipped: %s", e)
    _manager.apply_from_env()
    if _manager.applied:
        logger.info("applied patches: %s", _manager.applied)
    return _manager
