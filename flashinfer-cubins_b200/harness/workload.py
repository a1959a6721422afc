"""Workloads: one operator, one native entry point, launched from Python.

This is the operator API of Aalanli/flashinfer-cubins (``harness/workload.py`` there,
lines 40-46 and 258-571) with its cubin plumbing replaced: where the reference loads
a one-kernel cubin through libcuda and rebuilds a CUTLASS ``Params`` struct in Python,
a workload here binds the C-ABI library ``lib/libnvfp4_b200.so`` (``harness.native``)
and hands it device pointers and shapes. Names, argument meaning and error behaviour
of the public methods are the reference's, so its tests read the same:

* ``cls(None, device=...)`` is a reference-only workload (works on CPU);
  ``cls.from_arch(arch, device=...)`` binds the native library;
* ``get_cases / get_inputs / get_reference / run / prepare / validate`` are the
  contract (``harness/workload.py:484-507``); ``get_inputs`` and ``get_reference`` run
  with TF32 off;
* ``run`` allocates outputs and launches once, asynchronously, on the caller's current
  PyTorch stream; ``prepare`` returns a callable that launches without allocating and
  returns the same outputs object every time;
* bad operands raise ``ValueError`` before any native call, an unsupported device
  raises ``RuntimeError`` and nothing is launched.

The "image" of a workload (``get_image`` / ``patch_image``) is a short byte string
naming the bound library; patching it re-binds the library and drops every cached
plan, which is what the reference's module reload exercises.
"""

from __future__ import annotations

import contextlib
import functools
import os
import re
import threading
from abc import ABC, abstractmethod
from collections.abc import Callable, Iterator
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, ClassVar

import torch

from . import native

# Where data files of the reference project are looked up (its ``resources/`` tree: the
# NVIDIA task definitions and the trace inventories, which are not part of this package).
# ``REFERENCE_ROOT`` names a checkout of the reference; without it the paths simply do not
# exist and everything that needs only this package's own case tables still works.
ROOT = Path(os.environ.get("REFERENCE_ROOT") or Path(__file__).resolve().parents[1])
IMPLS = ROOT / "impls"
MANIFEST = "kernels.json"
IMAGE_PREFIX = b"nvfp4-b200-cabi:"


@dataclass(frozen=True)
class CaseSpec:
    name: str
    params: dict[str, Any] = field(default_factory=dict)
    seed: int = 0
    suite: str = "smoke"
    source: dict[str, Any] = field(default_factory=dict)


def normalize_arch(arch: str | int) -> str:
    """``sm_100a`` for ``sm_100a``, ``100a``, ``compute_100a`` or ``-arch=sm_100a``."""
    text = str(arch)
    for prefix in ("-arch=", "sm_", "compute_"):
        if text.startswith(prefix):
            text = text[len(prefix):]
    if re.fullmatch(r"[0-9]{2,3}[af]?", text) is None:
        raise ValueError(f"Invalid CUDA architecture: {arch!r}")
    return "sm_" + text


def arch_capability(arch: str) -> tuple[int, int]:
    digits = int(normalize_arch(arch)[3:].rstrip("af"))
    return divmod(digits, 10)


def arch_compatible(binary_arch: str, arch: str) -> bool:
    """Whether code built for ``binary_arch`` runs on GPUs of ``arch``: same major;
    an ``a`` build only on its own minor; plain and ``f`` builds on equal or later
    minors."""
    binary_arch, arch = normalize_arch(binary_arch), normalize_arch(arch)
    (major, minor), (want_major, want_minor) = arch_capability(binary_arch), arch_capability(arch)
    if major != want_major:
        return False
    if binary_arch.endswith("a"):
        return minor == want_minor and not arch.endswith("f")
    return minor <= want_minor


def device_capability(device: torch.device | str | None = None) -> tuple[int, int] | None:
    if not torch.cuda.is_available():
        return None
    device = torch.device(device or "cuda")
    if device.type != "cuda":
        return None
    return torch.cuda.get_device_capability(device)


def device_matches(arch: str, device: torch.device | str | None = None) -> bool:
    """Exact compute-capability match: sm_100a code never runs on another GPU."""
    capability = device_capability(device)
    return capability is not None and capability == arch_capability(arch)


def device_runs(binary_arch: str, device: torch.device | str | None = None) -> bool:
    capability = device_capability(device)
    if capability is None:
        return False
    major, minor = capability
    return arch_compatible(binary_arch, f"sm_{major}{minor}{'a' if major >= 9 else ''}")


@contextlib.contextmanager
def exact_fp32() -> Iterator[None]:
    """FP32 matmuls and convolutions without TF32 inside the block, whatever the
    process enables; the previous flags come back afterwards."""
    matmul, cudnn = torch.backends.cuda.matmul, torch.backends.cudnn
    previous = (matmul.allow_tf32, cudnn.allow_tf32)
    matmul.allow_tf32 = False
    cudnn.allow_tf32 = False
    try:
        yield
    finally:
        matmul.allow_tf32, cudnn.allow_tf32 = previous


def _without_tf32(method: Callable[..., Any]) -> Callable[..., Any]:
    @functools.wraps(method)
    def wrapper(*args: Any, **kwargs: Any) -> Any:
        with exact_fp32():
            return method(*args, **kwargs)

    return wrapper


def library_image() -> bytes:
    """The byte string that stands for the native library as a workload's image."""
    return IMAGE_PREFIX + str(native.LIBRARY_PATH).encode()


class Workload(ABC):
    """One operator backed by one entry point of the native library.

    ``name`` and ``supported_arches`` are set by ``@register``. ``entry_point`` names
    the C function the workload launches (what ``image_name`` reports).
    """

    name: ClassVar[str]
    supported_arches: ClassVar[tuple[str, ...]] = ()
    package: ClassVar[str | None] = None
    entry_point: ClassVar[str] = ""

    def __init_subclass__(cls, **kwargs: Any) -> None:
        super().__init_subclass__(**kwargs)
        for attr in ("get_inputs", "get_reference"):
            method = cls.__dict__.get(attr)
            if method is not None and not getattr(method, "__isabstractmethod__", False):
                setattr(cls, attr, _without_tf32(method))

    def __init__(self, cubin: bytes | None, *, device: str | torch.device | None = None):
        """``cubin=None`` selects reference-only use (no native launches); otherwise
        it is the image returned by ``library_image()``."""
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.arch: str | None = None
        self.cubin_arch: str | None = None
        self._image: bytes | None = None
        self._closed = False
        self._lock = threading.RLock()
        self._plans: dict[Any, Any] = {}
        if cubin is not None:
            self._accept_image(cubin)

    # -- construction -------------------------------------------------------------------

    @classmethod
    def manifest_path(cls) -> Path:
        """Where the reference keeps the cubin manifest of this workload's package
        (``impls/<package>/kernels.json``, ``harness/workload.py:312-314`` there). Nothing
        is read from it here; its parent's name is how callers group workloads by
        package."""
        package = cls.package or cls.__module__.rsplit(".", 1)[-1]
        return IMPLS / package / MANIFEST

    @classmethod
    def default_arch(cls, device: str | torch.device | None = None) -> str | None:
        """The supported arch matching ``device``, if any."""
        for arch in cls.supported_arches:
            if device_matches(arch, device):
                return arch
        return None

    @classmethod
    def from_arch(cls, arch: str | None = None, *, device: str | torch.device | None = None):
        """Bind the native library for ``arch`` (default: the device's arch)."""
        arch = arch or cls.default_arch(device)
        if arch is None:
            raise RuntimeError(f"{cls.name} supports {cls.supported_arches}, not the current device")
        arch = normalize_arch(arch)
        if arch not in cls.supported_arches:
            raise ValueError(f"{cls.name} does not support {arch}")
        if not native.LIBRARY_PATH.is_file():
            raise FileNotFoundError(f"{native.LIBRARY_PATH} is missing; build the library first")
        workload = cls(library_image(), device=device)
        workload.arch = arch
        return workload

    # -- the image ------------------------------------------------------------------------

    def _accept_image(self, image: bytes) -> None:
        if not isinstance(image, bytes):
            raise TypeError("image must be bytes")
        if not image.startswith(IMAGE_PREFIX):
            raise ValueError("expected the native library's image")
        self._image = image
        self.cubin_arch = "sm_100a"
        self.arch = self.arch or self.cubin_arch

    def image_name(self) -> str:
        """The C entry point this workload launches."""
        if self._image is None:
            raise RuntimeError("reference-only workload has no image")
        return self.entry_point

    def get_image(self) -> bytes:
        with self._lock:
            self._check_open()
            if self._image is None:
                raise RuntimeError("reference-only workload has no image")
            return self._image

    def patch_image(self, image: bytes) -> None:
        """Re-bind the library: wait for the device, drop every plan, load again."""
        with self._lock:
            self._check_open()
            if self._image is None:
                raise RuntimeError("reference-only workload has no image")
            self._accept_image(image)
            self._drop_plans()
            native.unload()

    @property
    def kernel_params(self) -> list:
        """The reference lists a cubin's kernel parameters here; a C entry point has
        a prototype instead (``include/nvfp4_b200.h``)."""
        return []

    # -- native launch ----------------------------------------------------------------------

    def is_supported(self) -> bool:
        return (
            self._image is not None
            and not self._closed
            and device_runs("sm_100a", self.device)
            and (self.arch is None or device_matches(self.arch, self.device))
        )

    def _check_supported(self) -> None:
        # Fail before any native work.
        if not self.is_supported():
            raise RuntimeError(f"{self.arch} code cannot run on {self.device}")

    def device_index(self) -> int:
        index = self.device.index
        return torch.cuda.current_device() if index is None else index

    def stream_handle(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def plan_for(self, key: Any, create: Callable[[], native.Plan]):
        """(plan, workspace tensor) cached under ``key`` and the current stream. The
        workspace is a torch allocation owned by the workload, zeroed on that stream
        when the entry is made: launches on another stream get a plan and a workspace
        of their own, so a workspace is never shared by launches that could overlap and
        never used before its initialisation has run. A launch callable returned by
        ``prepare`` belongs to the stream that was current when it was prepared."""
        with self._lock:
            stream = self.stream_handle()
            entry = self._plans.get((key, stream))
            if entry is None:
                plan = create()
                size = max(plan.workspace_bytes(), 256)
                with torch.cuda.device(self.device):
                    workspace = torch.empty(size, dtype=torch.uint8, device=self.device)
                    plan.init_workspace(workspace.data_ptr(), stream)
                entry = (plan, workspace)
                self._plans[(key, stream)] = entry
            return entry

    def check_status(self) -> None:
        """Synchronise and raise ``native.NativeError`` if a kernel of any cached plan
        abandoned a bounded wait."""
        with self._lock:
            for (_, stream), (plan, workspace) in self._plans.items():
                plan.status(workspace.data_ptr(), stream)

    def _drop_plans(self) -> None:
        if self._plans:
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            for plan, _ in self._plans.values():
                plan.destroy()
            self._plans.clear()

    def prepare(self, inputs: tuple) -> tuple[Callable[[], tuple], tuple | None]:
        """(launch callable, outputs) for timing. Override to keep allocation and
        argument checks out of the timed callable."""
        return (lambda: self.run(inputs)), None

    # -- workload contract --------------------------------------------------------------------

    @abstractmethod
    def get_cases(self) -> list[CaseSpec]: ...

    @abstractmethod
    def get_inputs(self, case: CaseSpec) -> tuple: ...

    @abstractmethod
    def get_reference(self, inputs: tuple) -> tuple:
        """PyTorch reference on CPU or CUDA; must not mutate inputs."""

    @abstractmethod
    def run(self, inputs: tuple) -> tuple:
        """Allocate outputs and launch once (asynchronously)."""

    @abstractmethod
    def validate(self, ref: tuple, impl: tuple) -> None:
        """Raise AssertionError unless ``impl`` matches ``ref``."""

    # -- helpers ------------------------------------------------------------------------------

    @staticmethod
    def assert_close(ref: tuple, impl: tuple, rtol: float = 1e-2, atol: float = 1e-2) -> None:
        if not (isinstance(ref, tuple) and isinstance(impl, tuple) and len(ref) == len(impl)):
            raise AssertionError("outputs must be tuples of equal length")
        for expected, actual in zip(ref, impl):
            if not (isinstance(expected, torch.Tensor) and isinstance(actual, torch.Tensor)):
                raise AssertionError("every output must be a torch tensor")
            torch.testing.assert_close(
                actual, expected, rtol=rtol, atol=atol, equal_nan=False,
                check_device=True, check_dtype=True,
            )

    def generator(self, case: CaseSpec) -> torch.Generator:
        return torch.Generator(device=self.device).manual_seed(case.seed)

    def randn(self, shape, generator, dtype=torch.bfloat16, scale=1.0):
        return (torch.randn(shape, device=self.device, generator=generator) * scale).to(dtype)

    def scalar(self, value, dtype=torch.float32):
        return torch.tensor(value, dtype=dtype)

    # -- lifecycle ----------------------------------------------------------------------------

    def _check_open(self) -> None:
        if self._closed:
            raise RuntimeError("workload is closed")

    def close(self) -> None:
        with self._lock:
            self._drop_plans()
            self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
