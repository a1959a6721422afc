"""B200-native NVFP4 block-scaled GEMM family behind the operator API of
Aalanli/flashinfer-cubins (``harness/__init__.py:7-28`` there)."""

from .registry import REGISTRY, get_workload, register, register_variant
from .workload import CaseSpec, Workload, normalize_arch


def enumerate_workloads(arch: str | None = None) -> list[type[Workload]]:
    """Registered workload classes sorted by name; only those supporting ``arch`` if
    one is given."""
    from . import workloads  # noqa: F401  (importing registers the built-in workloads)

    wanted = None if arch is None else normalize_arch(arch)
    return [
        REGISTRY[name]
        for name in sorted(REGISTRY)
        if wanted is None or wanted in REGISTRY[name].supported_arches
    ]


__all__ = [
    "CaseSpec",
    "REGISTRY",
    "Workload",
    "enumerate_workloads",
    "get_workload",
    "normalize_arch",
    "register",
    "register_variant",
]
