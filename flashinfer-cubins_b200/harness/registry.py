"""Name -> workload class registry with an architecture filter.

Same entry points as ``harness/registry.py`` of the reference (lines 14-61):
``@register(name=..., supported_arches=...)`` for a hand-written class,
``register_variant`` for a generated subclass, ``get_workload(name)`` to look one up.
"""

from __future__ import annotations

import re
from collections.abc import Callable, Iterable
from typing import Any, TypeVar

from .workload import Workload, normalize_arch

W = TypeVar("W", bound=type[Workload])

REGISTRY: dict[str, type[Workload]] = {}


def register(*, name: str, supported_arches: Iterable[str]) -> Callable[[W], W]:
    """Register a Workload subclass under a unique name; sets ``cls.name`` and
    ``cls.supported_arches`` (normalized, duplicates dropped, order kept)."""
    arches: list[str] = []
    for arch in supported_arches:
        arch = normalize_arch(arch)
        if arch not in arches:
            arches.append(arch)
    if not arches:
        raise ValueError(f"{name}: supported_arches must be nonempty")

    def decorate(cls: W) -> W:
        if not (isinstance(cls, type) and issubclass(cls, Workload)):
            raise TypeError("@register applies to Workload subclasses")
        existing = REGISTRY.get(name)
        if existing is not None and existing is not cls:
            raise ValueError(f"workload {name!r} is already registered")
        cls.name = name
        cls.supported_arches = tuple(arches)
        REGISTRY[name] = cls
        return cls

    return decorate


def register_variant(
    base: type[Workload], *, name: str, supported_arches: Iterable[str], **attributes: Any
) -> type[Workload]:
    """Register a generated subclass of ``base`` that carries ``attributes`` as class
    attributes; the class is placed in ``base``'s module."""
    qualname = "".join(part.title() for part in re.split(r"[^0-9A-Za-z]+", name))
    body = {"__module__": base.__module__, "__qualname__": qualname, **attributes}
    return register(name=name, supported_arches=supported_arches)(type(qualname, (base,), body))


def get_workload(name: str) -> type[Workload]:
    from . import workloads  # noqa: F401  (importing registers the built-in workloads)

    return REGISTRY[name]
