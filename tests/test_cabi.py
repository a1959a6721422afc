"""The C-ABI library without a GPU: it loads, exports every function that
include/nvfp4_b200.h declares, and rejects invalid arguments with negative codes before
touching CUDA."""

import ctypes
import re
from pathlib import Path

import pytest

from harness import native

HEADER = Path(__file__).resolve().parents[1] / "include" / "nvfp4_b200.h"


@pytest.fixture(scope="module")
def library():
    if not native.LIBRARY_PATH.is_file():
        from harness import build
        build.build()
    return native.load()


def declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(nvfp4_\w+)\s*\(", text)))


def test_every_declared_function_is_exported_and_bound(library):
    declared = declared_functions()
    assert len(declared) >= 17
    for name in declared:
        assert hasattr(library, name), name
    assert sorted(native.exported_symbols()) == declared
    assert library.nvfp4_version() >= 1000


def test_invalid_arguments_are_rejected_without_cuda(library):
    plan = ctypes.c_void_p()
    # Shape checks come before any device query.
    for m, n, k, l in ((0, 8, 32, 1), (8, 8, 48, 1), (8, 12, 32, 1), (8, 8, 32, 0)):  # noqa: E741
        rc = library.nvfp4_gemm_plan_create(ctypes.byref(plan), 0, native.OUT_F16, m, n, k, l, None)
        assert rc == native.E_UNSUPPORTED_SHAPE, (m, n, k, l)
        assert b"unsupported problem" in library.nvfp4_last_error()
    assert library.nvfp4_gemm_plan_create(ctypes.byref(plan), 0, 7, 8, 8, 32, 1, None) == \
        native.E_INVALID_ARGUMENT
    assert library.nvfp4_gemm_plan_create(None, 0, 0, 8, 8, 32, 1, None) == native.E_INVALID_ARGUMENT
    shapes = (ctypes.c_int * 3)(8, 12, 32)
    assert library.nvfp4_group_gemm_plan_create(ctypes.byref(plan), 0, 1, shapes, None) == \
        native.E_UNSUPPORTED_SHAPE
    assert library.nvfp4_group_gemm_plan_create(ctypes.byref(plan), 0, 0, shapes, None) == \
        native.E_INVALID_ARGUMENT
    assert library.nvfp4_gemm_launch(None, 0, 0, 0, 0, 0, 0, 0, 0) == native.E_INVALID_ARGUMENT
    assert library.nvfp4_group_gemm_launch(None, 0, 0) == native.E_INVALID_ARGUMENT
    assert library.nvfp4_pack_scales(None, None, 1, 1, 1, None) == native.E_INVALID_ARGUMENT
    assert library.nvfp4_pack_scales(16, 16, 0, 1, 1, None) == native.E_UNSUPPORTED_SHAPE
    assert library.nvfp4_silu_product(16, 16, 16, 0, None) == native.E_UNSUPPORTED_SHAPE
    assert library.nvfp4_silu_product(18, 16, 16, 4, None) == native.E_MISALIGNED
    assert library.nvfp4_plan_workspace_bytes(None) == 0
    # The quantisers and the routing kernels check their arguments before they touch CUDA.
    assert library.nvfp4_quantize(None, 0, 16, 16, 8, 32, 1, None) == native.E_INVALID_ARGUMENT
    assert library.nvfp4_quantize(16, 5, 16, 16, 8, 32, 1, None) == native.E_INVALID_ARGUMENT
    assert library.nvfp4_quantize(16, 0, 16, 16, 8, 24, 1, None) == native.E_UNSUPPORTED_SHAPE
    assert library.nvfp4_quantize(24, 0, 16, 16, 8, 32, 1, None) == native.E_MISALIGNED
    assert library.nvfp4_quantize_blocks(16, 0, 16, 16, 8, 32, None, None) == native.E_INVALID_ARGUMENT
    assert library.nvfp4_quantize_gather(16, 0, 16, 16, 8, 32, 6, None) == native.E_INVALID_ARGUMENT
    assert library.nvfp4_moe_count(None, 1, 8, 4, 16, None) == native.E_INVALID_ARGUMENT
    assert library.nvfp4_moe_count(16, 1, 8, 513, 16, None) == native.E_UNSUPPORTED_SHAPE
    assert library.nvfp4_moe_count(16, 1, -1, 4, 16, None) == native.E_UNSUPPORTED_SHAPE
    starts = (ctypes.c_int * 2)(0, 256)
    assert library.nvfp4_moe_place(16, 1, 8, 0, 2, starts, 128, 16, 16, 16, None) == \
        native.E_UNSUPPORTED_SHAPE
    assert library.nvfp4_moe_place(16, 1, 8, 2, 2, starts, 128, 16, 16, 16, None) == \
        native.E_INVALID_ARGUMENT      # an expert's first row beyond the rows
    assert library.nvfp4_moe_place(16, 1, 8, 2, 2, None, 128, 16, 16, 16, None) == \
        native.E_INVALID_ARGUMENT
    with pytest.raises(ValueError):
        native.check(native.E_UNSUPPORTED_SHAPE)
    with pytest.raises(RuntimeError):
        native.check(native.E_UNSUPPORTED_DEVICE)
    with pytest.raises(native.NativeError):
        native.check(700)
