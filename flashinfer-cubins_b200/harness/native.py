"""ctypes binding of the C-ABI library ``lib/libnvfp4_b200.so`` (``include/nvfp4_b200.h``).

The library is the only native code of this package: hand-written sm_100a kernels
behind plain C entry points. This module replaces the reference's libcuda binding
(``harness/cuda_driver.py`` there): instead of loading a cubin and marshalling a
CUTLASS ``Params`` struct, the workloads hand device pointers and shapes to the
library. There is no fallback: if the library is missing, ``load()`` raises.

Status codes map to exceptions the way the reference's host code behaves
(``harness/workloads/nvfp4_gemm.py:226-231,440-443``): invalid operands raise
``ValueError`` before anything is launched, an unsupported device or a CUDA error
raises ``RuntimeError``.
"""

from __future__ import annotations

import ctypes
import threading
from pathlib import Path

PACKAGE_ROOT = Path(__file__).resolve().parents[1]
LIBRARY_PATH = PACKAGE_ROOT / "lib" / "libnvfp4_b200.so"

E_INVALID_ARGUMENT = -1
E_UNSUPPORTED_SHAPE = -2
E_MISALIGNED = -3
E_UNSUPPORTED_DEVICE = -4
E_DEVICE_TIMEOUT = -5
E_NOT_BOUND = -6
E_SCRATCH_TOO_LARGE = -7

OUT_F16 = 0
OUT_F32 = 1
OUT_FP4 = 2
OUT_BF16 = 3

SCHEDULE_NAMES = {1: "data_parallel", 2: "stream_k", 3: "cluster_split_k"}


class NativeError(RuntimeError):
    """A CUDA error or a device-side timeout reported by the library."""

    def __init__(self, status: int, message: str):
        super().__init__(f"nvfp4 library error {status}: {message}")
        self.status = status


class Config(ctypes.Structure):
    _fields_ = [("tile_n", ctypes.c_int), ("schedule", ctypes.c_int), ("ctas", ctypes.c_int),
                ("pair", ctypes.c_int)]


class PlanInfo(ctypes.Structure):
    _fields_ = [
        ("tile_m", ctypes.c_int),
        ("tile_n", ctypes.c_int),
        ("tile_k", ctypes.c_int),
        ("stages", ctypes.c_int),
        ("schedule", ctypes.c_int),
        ("ctas", ctypes.c_int),
        ("threads", ctypes.c_int),
        ("smem_bytes", ctypes.c_int),
        ("tiles", ctypes.c_int64),
        ("units", ctypes.c_int64),
        ("sm_count", ctypes.c_int),
    ]


_P = ctypes.c_void_p
_PROTOTYPES = {
    "nvfp4_version": (ctypes.c_int, []),
    "nvfp4_last_error": (ctypes.c_char_p, []),
    "nvfp4_device_supported": (ctypes.c_int, [ctypes.c_int]),
    "nvfp4_gemm_plan_create": (
        ctypes.c_int,
        [ctypes.POINTER(_P), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
         ctypes.c_int, ctypes.c_int, ctypes.POINTER(Config)],
    ),
    "nvfp4_gemm_plan_create_shuffled": (
        ctypes.c_int,
        [ctypes.POINTER(_P), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
         ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(Config)],
    ),
    "nvfp4_dual_gemm_plan_create": (
        ctypes.c_int,
        [ctypes.POINTER(_P), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
         ctypes.c_int, ctypes.POINTER(Config)],
    ),
    "nvfp4_dual_gemm_plan_create_fp4": (
        ctypes.c_int,
        [ctypes.POINTER(_P), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
         ctypes.c_int, ctypes.POINTER(Config)],
    ),
    "nvfp4_dual_gemm_launch_fp4": (ctypes.c_int, [_P] * 12),
    "nvfp4_group_gemm_plan_create": (
        ctypes.c_int,
        [ctypes.POINTER(_P), ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int),
         ctypes.POINTER(Config)],
    ),
    "nvfp4_plan_destroy": (None, [_P]),
    "nvfp4_plan_workspace_bytes": (ctypes.c_size_t, [_P]),
    "nvfp4_plan_init_workspace": (ctypes.c_int, [_P, _P, _P]),
    "nvfp4_plan_info_get": (ctypes.c_int, [_P, ctypes.POINTER(PlanInfo)]),
    "nvfp4_gemm_launch": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "nvfp4_selftest_abandoned_wait": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "nvfp4_gemm_launch_fp4": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "nvfp4_gemm_launch_static": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P]),
    "nvfp4_static_scratch_bytes": (ctypes.c_size_t, []),
    "nvfp4_static_status": (ctypes.c_int, [ctypes.c_int, _P, ctypes.POINTER(ctypes.c_int)]),
    "nvfp4_dual_gemm_launch": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "nvfp4_group_gemm_bind": (
        ctypes.c_int,
        [_P, ctypes.POINTER(_P), ctypes.POINTER(_P), ctypes.POINTER(_P), ctypes.POINTER(_P),
         ctypes.POINTER(_P), _P, _P],
    ),
    "nvfp4_group_dual_gemm_plan_create_fp4": (
        ctypes.c_int,
        [ctypes.POINTER(_P), ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int),
         ctypes.POINTER(Config)],
    ),
    "nvfp4_group_dual_gemm_bind_fp4": (
        ctypes.c_int,
        [_P] + [ctypes.POINTER(_P)] * 8 + [_P, _P],
    ),
    "nvfp4_group_gemm_launch": (ctypes.c_int, [_P, _P, _P]),
    "nvfp4_plan_status": (ctypes.c_int, [_P, _P, _P, ctypes.POINTER(ctypes.c_int)]),
    "nvfp4_pack_scales": (
        ctypes.c_int, [_P, _P, ctypes.c_int, ctypes.c_int, ctypes.c_int, _P],
    ),
    "nvfp4_quantize": (
        ctypes.c_int, [_P, ctypes.c_int, _P, _P, ctypes.c_int, ctypes.c_int, ctypes.c_int, _P],
    ),
    "nvfp4_quantize_blocks": (
        ctypes.c_int, [_P, ctypes.c_int, _P, _P, ctypes.c_int, ctypes.c_int, _P, _P],
    ),
    "nvfp4_quantize_gather": (
        ctypes.c_int, [_P, ctypes.c_int, _P, _P, ctypes.c_int, ctypes.c_int, _P, _P],
    ),
    "nvfp4_moe_count": (
        ctypes.c_int, [_P, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, _P, _P],
    ),
    "nvfp4_moe_place": (
        ctypes.c_int, [_P, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, _P,
                       ctypes.c_int, _P, _P, _P, _P],
    ),
    "nvfp4_moe_plan_create": (
        ctypes.c_int, [ctypes.POINTER(_P), ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                       ctypes.c_int, ctypes.c_int, ctypes.POINTER(Config)],
    ),
    "nvfp4_moe_bind": (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "nvfp4_moe_layout": (ctypes.c_int, [_P, _P, _P, _P]),
    "nvfp4_moe_place_routed": (
        ctypes.c_int, [_P, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, _P, _P, _P, _P, _P, _P],
    ),
    "nvfp4_moe_combine": (
        ctypes.c_int, [_P, _P, _P, _P, ctypes.c_int, ctypes.c_int, ctypes.c_int, _P],
    ),
    "nvfp4_silu_product": (ctypes.c_int, [_P, _P, _P, ctypes.c_int64, _P]),
    "nvfp4_measure_mma_peak": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_double)]),
}

_lock = threading.Lock()
_library: ctypes.CDLL | None = None


def exported_symbols() -> tuple[str, ...]:
    """Names this binding expects the library to export."""
    return tuple(_PROTOTYPES)


def load() -> ctypes.CDLL:
    """The loaded library; raises ``FileNotFoundError`` if it has not been built
    (``python __graft_entry__.py`` or ``harness.build.build()`` builds it)."""
    global _library
    with _lock:
        if _library is None:
            if not LIBRARY_PATH.is_file():
                raise FileNotFoundError(
                    f"{LIBRARY_PATH} is missing; build it with harness.build.build()"
                )
            library = ctypes.CDLL(str(LIBRARY_PATH))
            for name, (restype, argtypes) in _PROTOTYPES.items():
                function = getattr(library, name)
                function.restype = restype
                function.argtypes = argtypes
            _library = library
        return _library


def unload() -> None:
    """Forget the loaded library; the next ``load()`` binds it again."""
    global _library
    with _lock:
        _library = None


def check(status: int) -> None:
    """Raise for a non-zero library status."""
    if status == 0:
        return
    message = (load().nvfp4_last_error() or b"").decode(errors="replace")
    if status in (E_UNSUPPORTED_DEVICE,):
        raise RuntimeError(message)
    if status in (E_DEVICE_TIMEOUT,):
        raise NativeError(status, message)
    if status < 0:
        raise ValueError(message)
    raise NativeError(status, message)


def device_supported(index: int) -> bool:
    status = load().nvfp4_device_supported(index)
    if status in (0, 1):
        return bool(status)
    check(status)
    return False


class Plan:
    """Owner of one ``nvfp4_plan`` handle."""

    def __init__(self, handle: int):
        self._handle = ctypes.c_void_p(handle)

    @staticmethod
    def _config(tile_n: int = 0, schedule: int = 0, ctas: int = 0, pair: int = 0):
        if not (tile_n or schedule or ctas or pair):
            return None
        return ctypes.byref(Config(tile_n, schedule, ctas, pair))

    @classmethod
    def dense(cls, device: int, out_kind: int, m: int, n: int, k: int, l: int, **config):  # noqa: E741
        handle = _P()
        check(load().nvfp4_gemm_plan_create(
            ctypes.byref(handle), device, out_kind, m, n, k, l, cls._config(**config)))
        return cls(handle.value)

    @classmethod
    def dense_shuffled(cls, device: int, out_kind: int, m: int, n: int, k: int, l: int,  # noqa: E741
                       shuffle_block: int, **config):
        """Dense GEMM on a B whose rows are in FlashInfer's epilogue-shuffled order."""
        handle = _P()
        check(load().nvfp4_gemm_plan_create_shuffled(
            ctypes.byref(handle), device, out_kind, m, n, k, l, shuffle_block,
            cls._config(**config)))
        return cls(handle.value)

    @classmethod
    def dual(cls, device: int, m: int, n: int, k: int, l: int, **config):  # noqa: E741
        handle = _P()
        check(load().nvfp4_dual_gemm_plan_create(
            ctypes.byref(handle), device, m, n, k, l, cls._config(**config)))
        return cls(handle.value)

    @classmethod
    def dual_fp4(cls, device: int, m: int, n: int, k: int, l: int, **config):  # noqa: E741
        """Fused dual GEMM whose gated output is quantised to NVFP4 in the epilogue."""
        handle = _P()
        check(load().nvfp4_dual_gemm_plan_create_fp4(
            ctypes.byref(handle), device, m, n, k, l, cls._config(**config)))
        return cls(handle.value)

    @classmethod
    def grouped(cls, device: int, problems, **config):
        flat = [int(v) for problem in problems for v in problem]
        array = (ctypes.c_int * len(flat))(*flat)
        handle = _P()
        check(load().nvfp4_group_gemm_plan_create(
            ctypes.byref(handle), device, len(flat) // 3, array, cls._config(**config)))
        return cls(handle.value)

    @classmethod
    def grouped_dual_fp4(cls, device: int, problems, **config):
        """Grouped fused dual GEMM (gate/up projection) with NVFP4 output."""
        flat = [int(v) for problem in problems for v in problem]
        array = (ctypes.c_int * len(flat))(*flat)
        handle = _P()
        check(load().nvfp4_group_dual_gemm_plan_create_fp4(
            ctypes.byref(handle), device, len(flat) // 3, array, cls._config(**config)))
        return cls(handle.value)

    @classmethod
    def routed(cls, device: int, out_kind: int, experts: int, n: int, k: int, max_rows: int,
               **config):
        """Grouped GEMM over ``experts`` groups whose row counts are decided on the device:
        ``OUT_FP4`` = gate/up dual GEMM with NVFP4 output, ``OUT_F16`` = GEMM with FP16 output;
        all groups share buffers of ``max_rows`` rows."""
        handle = _P()
        check(load().nvfp4_moe_plan_create(ctypes.byref(handle), device, experts, n, k, max_rows,
                                           out_kind, cls._config(**config)))
        return cls(handle.value)

    @property
    def handle(self) -> ctypes.c_void_p:
        if self._handle is None:
            raise RuntimeError("plan is destroyed")
        return self._handle

    def workspace_bytes(self) -> int:
        return int(load().nvfp4_plan_workspace_bytes(self.handle))

    def init_workspace(self, workspace: int, stream: int) -> None:
        check(load().nvfp4_plan_init_workspace(self.handle, workspace, stream))

    def info(self) -> dict:
        info = PlanInfo()
        check(load().nvfp4_plan_info_get(self.handle, ctypes.byref(info)))
        result = {name: getattr(info, name) for name, _ in PlanInfo._fields_}
        result["schedule"] = SCHEDULE_NAMES.get(result["schedule"], str(result["schedule"]))
        return result

    def launch_dense(self, a, b, sfa, sfb, alpha, d, workspace, stream) -> None:
        check(load().nvfp4_gemm_launch(self.handle, a, b, sfa, sfb, alpha, d, workspace, stream))

    def selftest_abandoned_wait(self, a, b, sfa, sfb, alpha, d, workspace, stream) -> None:
        """The failure-detection self-test: the same launch with a producer that issues
        nothing and waits that give up after milliseconds (``status`` then raises)."""
        check(load().nvfp4_selftest_abandoned_wait(
            self.handle, a, b, sfa, sfb, alpha, d, workspace, stream))

    def launch_dense_fp4(self, a, b, sfa, sfb, alpha, d_packed, d_scales, workspace, stream) -> None:
        """Dense launch of a plan made with ``OUT_FP4``: D quantised to NVFP4 in the epilogue."""
        check(load().nvfp4_gemm_launch_fp4(
            self.handle, a, b, sfa, sfb, alpha, d_packed, d_scales, workspace, stream))

    def launch_dense_static(self, a, b, sfa, sfb, alpha, d, stream) -> None:
        """Dense launch on the library's built-in scratch array: for callers that may
        not allocate a workspace. Raises ``ValueError`` if the plan needs more scratch
        than the array holds."""
        check(load().nvfp4_gemm_launch_static(self.handle, a, b, sfa, sfb, alpha, d, stream))

    def launch_dual(self, a, b1, b2, sfa, sfb1, sfb2, alpha, d, workspace, stream) -> None:
        check(load().nvfp4_dual_gemm_launch(
            self.handle, a, b1, b2, sfa, sfb1, sfb2, alpha, d, workspace, stream))

    def launch_dual_fp4(self, a, b1, b2, sfa, sfb1, sfb2, alpha, d_packed, d_scales, workspace,
                        stream) -> None:
        check(load().nvfp4_dual_gemm_launch_fp4(
            self.handle, a, b1, b2, sfa, sfb1, sfb2, alpha, d_packed, d_scales, workspace, stream))

    def bind_groups(self, a, b, sfa, sfb, d, workspace, stream) -> None:
        def array(values):
            return (_P * len(values))(*values)

        check(load().nvfp4_group_gemm_bind(
            self.handle, array(a), array(b), array(sfa), array(sfb), array(d), workspace, stream))

    def bind_dual_groups_fp4(self, a, b1, b2, sfa, sfb1, sfb2, d_packed, d_scales, workspace,
                             stream) -> None:
        def array(values):
            return (_P * len(values))(*values)

        check(load().nvfp4_group_dual_gemm_bind_fp4(
            self.handle, array(a), array(b1), array(b2), array(sfa), array(sfb1), array(sfb2),
            array(d_packed), array(d_scales), workspace, stream))

    def bind_routed(self, a, sfa, b, sfb, d, workspace, stream, b2=None, sfb2=None,
                    d_scales=0) -> None:
        """The shared buffers (``a``, ``sfa``, ``d``, ``d_scales``: addresses) and every
        expert's weights and scales (lists of addresses) of a routed plan, once."""
        def array(values):
            return (_P * len(values))(*values) if values is not None else None

        check(load().nvfp4_moe_bind(self.handle, a, sfa, array(b), array(sfb), array(b2),
                                    array(sfb2), d, d_scales, workspace, stream))

    def layout_routed(self, counts: int, workspace, stream) -> None:
        """Lay the groups out for the row counts in ``counts`` (device int32 array)."""
        check(load().nvfp4_moe_layout(self.handle, counts, workspace, stream))

    def place_routed(self, ids: int, ids_are_64bit: bool, pairs: int, choices: int, workspace,
                     cursors: int, row_of_pair: int, token_of_row: int, stream) -> None:
        """``moe_place`` with the first rows that ``layout_routed`` left in ``workspace``."""
        check(load().nvfp4_moe_place_routed(ids, int(ids_are_64bit), pairs, choices, self.handle,
                                            workspace, cursors, row_of_pair, token_of_row, stream))

    def launch_groups(self, workspace, stream) -> None:
        check(load().nvfp4_group_gemm_launch(self.handle, workspace, stream))

    def status(self, workspace, stream) -> int:
        """Synchronise ``stream`` and return the device status word (0 = ok);
        raises ``NativeError`` if a kernel abandoned a bounded wait."""
        value = ctypes.c_int(0)
        check(load().nvfp4_plan_status(self.handle, workspace, stream, ctypes.byref(value)))
        return value.value

    def destroy(self) -> None:
        if self._handle is not None:
            load().nvfp4_plan_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def static_status(device: int, stream: int) -> int:
    """Synchronise ``stream`` and return the status word shared by the launches on the
    built-in scratch array of ``device`` (0 = ok); raises ``NativeError`` if one of them
    abandoned a bounded wait."""
    value = ctypes.c_int(0)
    check(load().nvfp4_static_status(device, stream, ctypes.byref(value)))
    return value.value


def pack_scales(scales: int, packed: int, rows: int, cols: int, batches: int, stream: int) -> None:
    check(load().nvfp4_pack_scales(scales, packed, rows, cols, batches, stream))


IN_F32 = 0
IN_BF16 = 1


def quantize(x: int, x_kind: int, packed: int, scales: int, rows: int, k: int, batches: int,
             stream: int) -> None:
    check(load().nvfp4_quantize(x, x_kind, packed, scales, rows, k, batches, stream))


def quantize_blocks(x: int, x_kind: int, packed: int, scales: int, rows: int, k: int,
                    block_rows: int, stream: int) -> None:
    """``quantize`` of rows in 128-row blocks whose leading ``block_rows[b]`` rows hold data
    (a device array of int32); the other rows are left untouched in both outputs."""
    check(load().nvfp4_quantize_blocks(x, x_kind, packed, scales, rows, k, block_rows, stream))


def quantize_gather(x: int, x_kind: int, packed: int, scales: int, rows: int, k: int,
                    source_rows: int, stream: int) -> None:
    """Output row r = quantised row ``source_rows[r]`` of x (device int32 array; negative:
    the output row is left untouched)."""
    check(load().nvfp4_quantize_gather(x, x_kind, packed, scales, rows, k, source_rows, stream))


def moe_count(ids: int, ids_are_64bit: bool, pairs: int, experts: int, counts: int,
              stream: int) -> None:
    """``counts[e]`` (device int32) = number of ``ids`` equal to e."""
    check(load().nvfp4_moe_count(ids, int(ids_are_64bit), pairs, experts, counts, stream))


def moe_place(ids: int, ids_are_64bit: bool, pairs: int, choices: int, first_rows: list[int],
              rows: int, cursors: int, row_of_pair: int, token_of_row: int, stream: int) -> None:
    """Give every pair a row of its expert's block (``first_rows``: host list, one per expert)."""
    starts = (ctypes.c_int * len(first_rows))(*first_rows)
    check(load().nvfp4_moe_place(ids, int(ids_are_64bit), pairs, choices, len(first_rows), starts,
                                 rows, cursors, row_of_pair, token_of_row, stream))


def moe_combine(y: int, row_of_pair: int, weights: int, out: int, tokens: int, choices: int,
                hidden: int, stream: int) -> None:
    """``out[t] = sum_j weights[t, j] * y[row_of_pair[t * choices + j]]`` (FP16 rows, FP32 out)."""
    check(load().nvfp4_moe_combine(y, row_of_pair, weights, out, tokens, choices, hidden, stream))


def measure_mma_peak(device: int, iters: int = 4096) -> float:
    """TFLOP/s at which ``device`` issues block-scaled FP4 MMAs with nothing else running."""
    value = ctypes.c_double(0.0)
    check(load().nvfp4_measure_mma_peak(device, iters, ctypes.byref(value)))
    return value.value


def silu_product(h1: int, h2: int, out: int, size: int, stream: int) -> None:
    check(load().nvfp4_silu_product(h1, h2, out, size, stream))
