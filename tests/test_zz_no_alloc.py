"""The allocation-free dense launch, ``nvfp4_gemm_launch_static``.

Some callers of this library cannot give it a workspace because they may not allocate
device memory where they call it (all of HBM belongs to their own pool, or cudaMalloc is
banned on their hot path because it synchronises the device). For them the library keeps
24 MiB of scratch inside itself. This test drives that entry point through the C ABI with
a stream-K plan, which really uses the scratch (partial tiles and arrival counters), and
checks that it gives the same result as the ordinary launch with a caller workspace — on
two calls in a row, because the array keeps the previous call's contents — and that a
plan too large for the array is refused. Collected last so that a failure here cannot
hide any other test."""

import ctypes

import pytest
import torch

from harness import CaseSpec, get_workload, native

pytestmark = pytest.mark.gpu


def dense_inputs(m, n, k, seed, scales):
    workload = get_workload("nvfp4_gemm")(None, device="cuda")
    case = CaseSpec("static", {"m": m, "n": n, "k": k, "l": 1, "scales": scales}, seed)
    inputs = workload.get_inputs(case)
    (ref,) = workload.get_reference(inputs)
    return inputs, ref


def test_static_scratch_launch_matches_workspace_launch_twice():
    torch.backends.cuda.matmul.allow_tf32 = False
    library = native.load()
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    assert library.nvfp4_static_scratch_bytes() == 24 << 20
    m, n, k = 200, 520, 8192
    # A different plan first, so that the array holds foreign data where the next plan's
    # counters live.
    first, _ = dense_inputs(128, 1024, 4096, 40, "int0_3")
    warm = native.Plan.dense(0, native.OUT_F16, 128, 1024, 4096, 1, schedule=2)
    out = torch.empty((1, 128, 1024), dtype=torch.float16, device=dev)
    warm.launch_dense_static(*(t.data_ptr() for t in first), out.data_ptr(), stream)
    torch.cuda.synchronize()

    plan = native.Plan.dense(0, native.OUT_F16, m, n, k, 1, schedule=2)
    info = plan.info()
    assert info["schedule"] == "stream_k" and info["ctas"] > info["tiles"]
    assert 0 < plan.workspace_bytes() <= library.nvfp4_static_scratch_bytes()
    workspace = torch.empty(plan.workspace_bytes(), dtype=torch.uint8, device=dev)
    plan.init_workspace(workspace.data_ptr(), stream)
    for seed, scales in ((41, "int0_3"), (42, "uniform")):
        inputs, ref = dense_inputs(m, n, k, seed, scales)
        pointers = [t.data_ptr() for t in inputs]
        expected = torch.full((1, m, n), float("nan"), dtype=torch.float16, device=dev)
        plan.launch_dense(*pointers, expected.data_ptr(), workspace.data_ptr(), stream)
        assert plan.status(workspace.data_ptr(), stream) == 0
        torch.testing.assert_close(expected.permute(1, 2, 0), ref, rtol=1e-3, atol=1e-3)
        for call in range(2):
            got = torch.full((1, m, n), float("nan"), dtype=torch.float16, device=dev)
            blocks = torch.cuda.memory_stats()["allocation.all.allocated"]
            plan.launch_dense_static(*pointers, got.data_ptr(), stream)
            assert torch.cuda.memory_stats()["allocation.all.allocated"] == blocks
            torch.cuda.synchronize()
            torch.testing.assert_close(got, expected, rtol=1e-3, atol=1e-3)
            assert torch.equal(got, expected), f"call {call}: differs from the workspace launch"
            # The array's status word: no wait was abandoned, and reading it allocates nothing.
            blocks = torch.cuda.memory_stats()["allocation.all.allocated"]
            assert native.static_status(0, stream) == 0
            assert torch.cuda.memory_stats()["allocation.all.allocated"] == blocks
    plan.destroy()
    warm.destroy()


def test_static_scratch_launch_refuses_oversized_plans():
    library = native.load()
    stream = torch.cuda.current_stream().cuda_stream
    # 256-column tiles, stream-K on every SM: 2 x 148 x 128 KiB of partial slots.
    plan = native.Plan.dense(0, native.OUT_F16, 128, 7168, 16384, 1, tile_n=256, schedule=2)
    assert plan.workspace_bytes() > library.nvfp4_static_scratch_bytes()
    buffer = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = buffer.data_ptr()
    status = library.nvfp4_gemm_launch_static(plan.handle, p, p, p, p, p, p, stream)
    assert status == native.E_SCRATCH_TOO_LARGE
    assert b"scratch" in library.nvfp4_last_error()
    with pytest.raises(ValueError):
        plan.launch_dense_static(p, p, p, p, p, p, stream)
    dual = native.Plan.dual(0, 128, 128, 128, 1)
    assert library.nvfp4_gemm_launch_static(dual.handle, p, p, p, p, p, p, stream) == \
        native.E_INVALID_ARGUMENT
    assert isinstance(ctypes.c_void_p(p).value, int)
    plan.destroy()
    dual.destroy()
