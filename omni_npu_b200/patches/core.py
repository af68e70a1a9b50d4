"""Patch framework: named, reversible attribute overrides of third-party classes
and modules (vLLM in practice).

A patch is a class deriving from :class:`Patch`, decorated with
``@register_patch(name, target)``, that lists in ``attributes`` the names it
wants to install on ``target``.  ``PatchRegistry`` applies patches selected by
the ``OMNI_B200_VLLM_PATCHES`` environment variable (``ALL`` or a comma list;
``OMNI_NPU_VLLM_PATCHES`` is honoured as an alias).  Two patches may not
override the same attribute of the same target, and every applied patch can be
reverted, which the tests rely on.

Same contract as the reference's ``VLLMPatch`` / ``PatchManager``
(omni_npu/vllm_patches/core.py:15-73, patch_manager.py:12-73), plus ``revert``.
"""
from __future__ import annotations

import os
from types import MethodType, ModuleType
from typing import Any, Dict, List, Optional, Tuple, Type, Union

from ..logger import logger

_MISSING = object()
_OWNER_ATTR = "_omni_b200_patched_by"


class Patch:
    """Base class.  Subclasses set ``attributes`` (names defined on the subclass)."""
    attributes: List[str] = []
    target: Union[Type, ModuleType, None] = None
    name: str = ""
    _saved: Dict[str, Any]

    @classmethod
    def apply(cls) -> None:
        if cls is Patch:
            raise TypeError("the Patch base class cannot be applied")
        target = cls.target
        if target is None:
            raise TypeError(f"{cls.__name__} has no target (use @register_patch)")
        owners: Dict[str, str] = target.__dict__.get(_OWNER_ATTR) if isinstance(target, type) else \
            getattr(target, _OWNER_ATTR, None)
        if owners is None:
            owners = {}
            setattr(target, _OWNER_ATTR, owners)
        # validate everything first so that a failing patch leaves no half-applied state
        for attr in cls.attributes:
            if attr in ("apply", "revert", "target", "attributes", "name"):
                raise ValueError(f"{cls.__name__}: {attr!r} is reserved")
            if attr not in cls.__dict__:
                raise ValueError(f"{cls.__name__} lists {attr!r} but does not define it")
            if attr in owners:
                raise ValueError(f"{_tname(target)}.{attr} is already patched by {owners[attr]}")
        cls._saved = {}
        for attr in cls.attributes:
            value = cls.__dict__[attr]
            if isinstance(value, classmethod) and isinstance(target, type):
                value = classmethod(value.__func__)
            elif isinstance(value, (staticmethod, classmethod)) and isinstance(target, ModuleType):
                value = value.__func__
            cls._saved[attr] = target.__dict__.get(attr, _MISSING)
            setattr(target, attr, value)
            owners[attr] = cls.__name__
            logger.debug("patch %s: %s.%s", cls.__name__, _tname(target), attr)

    @classmethod
    def revert(cls) -> None:
        target = cls.target
        owners = getattr(target, _OWNER_ATTR, {})
        for attr, old in getattr(cls, "_saved", {}).items():
            if owners.get(attr) != cls.__name__:
                continue
            if old is _MISSING:
                delattr(target, attr)
            else:
                setattr(target, attr, old)
            del owners[attr]
        cls._saved = {}


def _tname(t) -> str:
    return getattr(t, "__name__", repr(t))


class PatchRegistry:
    registered: Dict[str, Type[Patch]] = {}

    def __init__(self) -> None:
        self.applied: List[str] = []
        self.failed: Dict[str, str] = {}

    @classmethod
    def register(cls, name: str, patch: Type[Patch]) -> None:
        cls.registered[name] = patch

    def apply_patch(self, name: str) -> bool:
        patch = self.registered.get(name)
        if patch is None:
            logger.error("patch %s is not registered", name)
            self.failed[name] = "not registered"
            return False
        if name in self.applied:
            return True
        try:
            patch.apply()
        except Exception as e:
            logger.error("applying patch %s failed: %s", name, e)
            self.failed[name] = str(e)
            return False
        self.applied.append(name)
        return True

    def apply_all(self) -> None:
        for name in list(self.registered):
            self.apply_patch(name)

    def apply_from_env(self) -> None:
        spec = os.environ.get("OMNI_B200_VLLM_PATCHES", os.environ.get("OMNI_NPU_VLLM_PATCHES", "")).strip()
        if not spec:
            return
        if spec == "ALL":
            self.apply_all()
            return
        for name in (p.strip() for p in spec.split(",")):
            if name:
                self.apply_patch(name)

    def revert_all(self) -> None:
        for name in reversed(self.applied):
            self.registered[name].revert()
        self.applied = []


def register_patch(name: str, target: Union[Type, ModuleType]):
    if not isinstance(target, (type, ModuleType)):
        raise TypeError(f"only classes and modules can be patched, got {type(target).__name__}")

    def deco(cls: Type[Patch]) -> Type[Patch]:
        cls.target = target
        cls.name = name
        PatchRegistry.register(name, cls)
        return cls

    return deco
