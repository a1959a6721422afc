"""Parity of the CUDA path on a B200, through the operator API and the C ABI: the
acceptance loop of every workload in a worker process of its own (every smoke case against
the harness's torch reference and the numpy oracle, see ``acceptance_worker.py``), then
golden fixtures through raw pointers, every tile width and schedule, the 2-CTA kernel,
plan sharing across threads, the status word and the abandoned-wait self-test, the
quantiser and the NVFP4-output epilogues."""

import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import load_golden
from gpu_util import (assert_matches_oracle, blocked_storage, integer_scaled, oracle_dense,
                      storage)
from harness import get_workload, native
from oracle import nvfp4_oracle as o

pytestmark = pytest.mark.gpu

WORKLOADS = ("nvfp4_gemm", "nvfp4_gemm_bf16", "nvfp4_gemm_bf16_shuffled", "nvfp4_dual_gemm_gemm",
             "nvfp4_dual_gemm",
             "nvfp4_group_gemm", "nvfp4_dual_gemm_pack_scales", "nvfp4_dual_gemm_silu_product")


@pytest.fixture(scope="module", autouse=True)
def exact_matmul():
    previous = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    yield
    torch.backends.cuda.matmul.allow_tf32 = previous


WORKER = Path(__file__).resolve().parent / "acceptance_worker.py"
WORKER_TIMEOUT_S = 900


@pytest.fixture(scope="module")
def acceptance_workers():
    """One child process per workload, started together (each has its own CUDA context, so
    a sticky error in one cannot fail another); a test waits for its own child."""
    children = {name: subprocess.Popen([sys.executable, str(WORKER), name],
                                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
                for name in WORKLOADS}
    yield children
    for child in children.values():
        if child.poll() is None:
            child.kill()


@pytest.mark.parametrize("name", WORKLOADS)
def test_smoke_cases_match_reference_and_oracle(name, acceptance_workers):
    """Every smoke case of the workload, in a worker process of its own
    (``acceptance_worker.py``): torch reference, numpy oracle, inputs unchanged, library
    re-bind, prepared launches, status word."""
    child = acceptance_workers[name]
    try:
        output, _ = child.communicate(timeout=WORKER_TIMEOUT_S)
    except subprocess.TimeoutExpired:
        child.kill()
        output, _ = child.communicate()
        pytest.fail(f"{name}: worker exceeded {WORKER_TIMEOUT_S} s\n{output[-4000:]}")
    assert child.returncode == 0, f"{name}: worker exit code {child.returncode}\n{output[-4000:]}"
    assert output.strip().splitlines()[-1].startswith(f"ok {name} "), output[-2000:]


def test_golden_fixtures_through_the_c_abi():
    """Inputs and outputs recorded from the reference itself; the kernel is called with
    raw pointers, as a foreign-language binding would."""
    data = load_golden("nvfp4_gemm_cases.npz")
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    for name in sorted({key.split("/")[0] for key in data}):
        t = {f: torch.from_numpy(data[f"{name}/{f}"]).to(dev) for f in ("a", "b", "sfa", "sfb", "alpha")}
        batches, m, half_k = t["a"].shape
        n, k = t["b"].shape[1], 2 * half_k
        d = torch.full((batches, m, n), float("nan"), dtype=torch.float16, device=dev)
        plan = native.Plan.dense(0, native.OUT_F16, m, n, k, batches)
        ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
        plan.init_workspace(ws.data_ptr(), stream)
        plan.launch_dense(t["a"].data_ptr(), t["b"].data_ptr(), t["sfa"].data_ptr(),
                          t["sfb"].data_ptr(), t["alpha"].data_ptr(), d.data_ptr(),
                          ws.data_ptr(), stream)
        assert plan.status(ws.data_ptr(), stream) == 0
        np.testing.assert_allclose(d.cpu().numpy().astype(np.float32),
                                   data[name + "/d"].astype(np.float32), rtol=1e-3, atol=1e-3,
                                   err_msg=name)
        plan.destroy()

    dual = load_golden("nvfp4_dual_gemm_cases.npz")
    for name in sorted({key.split("/")[0] for key in dual}):
        g = {f: dual[f"{name}/{f}"] for f in ("a", "b1", "b2", "sa", "s1", "s2", "out")}
        batches, m, half_k = g["a"].shape
        n, k = g["b1"].shape[1], 2 * half_k
        ops = [torch.from_numpy(x).to(dev) for x in (
            g["a"], g["b1"], g["b2"], o.to_blocked(g["sa"]), o.to_blocked(g["s1"]), o.to_blocked(g["s2"]))]
        alpha = torch.full((1,), float(dual[name + "/alpha"]), device=dev)
        d = torch.full((batches, m, n), float("nan"), dtype=torch.float16, device=dev)
        plan = native.Plan.dual(0, m, n, k, batches)
        ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
        plan.init_workspace(ws.data_ptr(), stream)
        plan.launch_dual(*(x.data_ptr() for x in ops), alpha.data_ptr(), d.data_ptr(),
                         ws.data_ptr(), stream)
        assert plan.status(ws.data_ptr(), stream) == 0
        np.testing.assert_allclose(d.cpu().numpy().astype(np.float32), g["out"].astype(np.float32),
                                   rtol=1e-3, atol=1e-3, err_msg=name)
        plan.destroy()


@pytest.mark.parametrize("tile_n", (64, 128, 256))
@pytest.mark.parametrize("schedule", (1, 2, 3))
def test_every_tile_width_and_schedule(tile_n, schedule):
    """The dense kernel's three tile widths under every schedule (whole tiles, stream-K
    with its workspace fix-up, cluster split-K with its shared-memory reduction; a plan
    falls back to another schedule when the requested one does not apply) on shapes with
    partial tiles, batches and a K tail; integer scales, so results must equal the oracle
    bit for bit however K is split."""
    workload = get_workload("nvfp4_gemm")(None, device="cuda")
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    cases = [c for c in workload.get_cases() if c.suite == "smoke"
             and integer_scaled(c, "int0_3") and c.params.get("alpha", 1.0) == 1.0]
    assert len(cases) >= 5
    for case in cases:
        inputs = workload.get_inputs(case)
        a, b, sfa, sfb, alpha = inputs
        m, n, k, batches = (case.params[key] for key in "mnkl")
        d = torch.full((batches, m, n), float("nan"), dtype=torch.float16, device=dev)
        plan = native.Plan.dense(0, native.OUT_F16, m, n, k, batches, tile_n=tile_n,
                                 schedule=schedule)
        info = plan.info()
        assert info["tile_n"] == tile_n
        ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
        plan.init_workspace(ws.data_ptr(), stream)
        for _ in range(2):  # the second launch reuses the self-resetting tile counters
            d.fill_(float("nan"))
            plan.launch_dense(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
                              alpha.data_ptr(), d.data_ptr(), ws.data_ptr(), stream)
            assert plan.status(ws.data_ptr(), stream) == 0
            assert_matches_oracle(d.permute(1, 2, 0), oracle_dense(inputs),
                                  f"{case.name}/bn{tile_n}/{info['schedule']}", True)
        plan.destroy()


@pytest.mark.parametrize("m,n,k,l,tile_n", [(128, 256, 4096, 1, 128), (300, 264, 2080, 2, 128),
                                             (128, 1024, 8192, 1, 256), (17, 520, 4096, 1, 64),
                                             (128, 7168, 2048, 1, 128)])
def test_cluster_split_k(m, n, k, l, tile_n):  # noqa: E741
    """Few tiles and a long K: the plan splits each tile's K over a thread-block cluster
    and reduces through peer shared memory. Unit-range scales: the result must match the
    torch reference within the tolerance, and two launches must agree bit for bit."""
    from harness import CaseSpec
    workload = get_workload("nvfp4_gemm")(None, device="cuda")
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    for scales, exact in (("int0_3", True), ("uniform", False)):
        case = CaseSpec("cluster", {"m": m, "n": n, "k": k, "l": l, "scales": scales}, 21)
        inputs = workload.get_inputs(case)
        a, b, sfa, sfb, alpha = inputs
        plan = native.Plan.dense(0, native.OUT_F16, m, n, k, l, tile_n=tile_n, schedule=3)
        info = plan.info()
        assert info["schedule"] == "cluster_split_k", info
        assert info["ctas"] % info["tiles"] == 0 and info["ctas"] > info["tiles"]
        ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
        plan.init_workspace(ws.data_ptr(), stream)
        outs = []
        for _ in range(2):
            d = torch.full((l, m, n), float("nan"), dtype=torch.float16, device=dev)
            plan.launch_dense(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
                              alpha.data_ptr(), d.data_ptr(), ws.data_ptr(), stream)
            assert plan.status(ws.data_ptr(), stream) == 0
            outs.append(d)
        assert torch.equal(outs[0], outs[1])
        (ref,) = workload.get_reference(inputs)
        if exact:
            assert torch.equal(outs[0].permute(1, 2, 0), ref)
        else:
            torch.testing.assert_close(outs[0].permute(1, 2, 0), ref, rtol=1e-3, atol=1e-3)
        plan.destroy()


@pytest.mark.parametrize("m,n,k,l", [(256, 256, 256, 1), (300, 520, 608, 2), (512, 768, 2080, 1),
                                     (129, 264, 96, 1), (1024, 2048, 1024, 1)])
@pytest.mark.parametrize("out_kind", (native.OUT_F16, native.OUT_F32))
def test_pair_kernel(m, n, k, l, out_kind):  # noqa: E741
    """The 2-CTA kernel (256 x 256 tiles, tcgen05.mma.cta_group::2), forced on shapes with
    partial tiles in M, N and K, batches, and more tiles than one wave of pairs would hold
    is not needed: bit-exact with integer scales, within tolerance otherwise."""
    from harness import CaseSpec
    workload = get_workload("nvfp4_gemm")(None, device="cuda")
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    dtype = torch.float16 if out_kind == native.OUT_F16 else torch.float32
    for scales, exact in (("int0_3", True), ("unit", False)):
        case = CaseSpec("pair", {"m": m, "n": n, "k": k, "l": l, "scales": scales,
                                 "alpha": 0.5}, 51)
        inputs = workload.get_inputs(case)
        a, b, sfa, sfb, alpha = inputs
        plan = native.Plan.dense(0, out_kind, m, n, k, l, pair=1)
        info = plan.info()
        assert info["tile_m"] == 256 and info["tile_n"] == 256 and info["ctas"] % 2 == 0, info
        ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
        plan.init_workspace(ws.data_ptr(), stream)
        d = torch.full((l, m, n), float("nan"), dtype=dtype, device=dev)
        plan.launch_dense(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
                          alpha.data_ptr(), d.data_ptr(), ws.data_ptr(), stream)
        assert plan.status(ws.data_ptr(), stream) == 0
        from harness.workloads.quantization import fp4_matmul
        from harness.workloads.nvfp4_gemm import from_task_scales
        ref = fp4_matmul(a, b, from_task_scales(sfa, m, k // 16), from_task_scales(sfb, n, k // 16),
                         alpha=0.5, out_dtype=dtype)
        if exact:
            assert torch.equal(d.permute(1, 2, 0), ref)
        else:
            torch.testing.assert_close(d.permute(1, 2, 0), ref, rtol=1e-3, atol=1e-3)
        plan.destroy()


@pytest.mark.parametrize("tile_n", (128, 256))
@pytest.mark.parametrize("schedule", (1, 2, 3))
def test_dual_gemm_under_every_schedule(schedule, tile_n):
    """The fused dual GEMM with whole tiles, the workspace fix-up and the cluster
    reduction (both accumulator halves travel to the owner of the output columns), on
    2 x 128-column and 2 x 64-column B tiles (the latter reads half a scale atom of each
    B; n = 264 and 136 end in partial and odd-numbered 64-column tiles)."""
    from harness import CaseSpec
    workload = get_workload("nvfp4_dual_gemm")(None, device="cuda")
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    for m, n, k, l in ((200, 264, 2080, 1), (256, 512, 7168, 1), (130, 136, 1024, 2)):  # noqa: E741
        case = CaseSpec("dual", {"m": m, "n": n, "k": k, "l": l, "alpha": 0.25}, 31)
        inputs = workload.get_inputs(case)
        (ref,) = workload.get_reference(inputs)
        plan = native.Plan.dual(0, m, n, k, l, schedule=schedule, tile_n=tile_n)
        info = plan.info()
        if schedule == 3:
            assert info["schedule"] == "cluster_split_k", info
        ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
        plan.init_workspace(ws.data_ptr(), stream)
        d = torch.full((l, m, n), float("nan"), dtype=torch.float16, device=dev)
        plan.launch_dual(*(t.data_ptr() for t in inputs), d.data_ptr(), ws.data_ptr(), stream)
        assert plan.status(ws.data_ptr(), stream) == 0
        torch.testing.assert_close(d.permute(1, 2, 0), ref, rtol=1e-3, atol=1e-3)
        plan.destroy()


def test_grouped_stream_k_and_rebinding():
    """One grouped plan bound to two operand sets (two workspaces), stream-K forced so
    that tiles of different groups share CTAs and the fix-up runs across groups."""
    workload = get_workload("nvfp4_group_gemm")(None, device="cuda")
    case = next(c for c in workload.get_cases() if c.name == "skewed_full")
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    plan = native.Plan.grouped(0, case.params["groups"], schedule=2)
    assert plan.info()["schedule"] == "stream_k"
    sets = []
    for seed in (5, 6):
        inputs = workload.get_inputs(type(case)(case.name, case.params, seed, case.suite))
        outputs = workload.allocate_outputs(inputs)
        config = workload.launch_config(inputs, outputs)
        ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
        plan.init_workspace(ws.data_ptr(), stream)
        plan.bind_groups(*config.pointers, ws.data_ptr(), stream)
        sets.append((inputs, outputs, ws))
    for inputs, outputs, ws in sets + sets[::-1]:
        for out in outputs:
            out.fill_(float("nan"))
        plan.launch_groups(ws.data_ptr(), stream)
        assert plan.status(ws.data_ptr(), stream) == 0
        ref = workload.get_reference(inputs)
        for got, want in zip(outputs, ref):
            assert torch.equal(got, want)
    plan.destroy()


def test_one_plan_launched_from_two_threads_on_two_streams():
    """A plan is immutable after creation: two host threads launch the same stream-K plan
    at the same time, each on its own stream with its own workspace and operands, and
    alternate between two operand sets (so the plan's tensor-map cache is looked up and
    filled concurrently). Every result must be bit-identical to the oracle."""
    import threading

    from harness import CaseSpec
    workload = get_workload("nvfp4_gemm")(None, device="cuda")
    dev = torch.device("cuda:0")
    m, n, k = 256, 384, 4096
    plan = native.Plan.dense(0, native.OUT_F16, m, n, k, 1, schedule=2, tile_n=128)
    assert plan.info()["schedule"] == "stream_k"
    jobs, errors = [], []
    for t in range(2):
        stream = torch.cuda.Stream(device=dev)
        sets = []
        for seed in (40 + 2 * t, 41 + 2 * t):
            inputs = workload.get_inputs(CaseSpec("threads", {"m": m, "n": n, "k": k, "l": 1}, seed))
            want = oracle_dense(inputs)
            d = torch.full((1, m, n), float("nan"), dtype=torch.float16, device=dev)
            sets.append((inputs, d, want))
        ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
        plan.init_workspace(ws.data_ptr(), torch.cuda.current_stream().cuda_stream)
        jobs.append((stream, sets, ws))
    torch.cuda.synchronize()
    start = threading.Barrier(2)

    def worker(stream, sets, ws):
        try:
            start.wait()
            for i in range(200):
                inputs, d, _ = sets[i % 2]
                plan.launch_dense(*(t.data_ptr() for t in inputs), d.data_ptr(), ws.data_ptr(),
                                  stream.cuda_stream)
            stream.synchronize()
        except Exception as error:  # surfaced in the main thread below
            errors.append(error)

    threads = [threading.Thread(target=worker, args=job) for job in jobs]
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join()
    assert not errors, errors
    for stream, sets, ws in jobs:
        assert plan.status(ws.data_ptr(), stream.cuda_stream) == 0
        for inputs, d, want in sets:
            assert np.array_equal(d.cpu().numpy(), want)
    plan.destroy()


def test_status_word_and_counters_are_reset_after_a_reported_timeout():
    """nvfp4_plan_status on a workspace whose status word is set (written here by the host,
    standing in for a kernel that abandoned a wait) reports the timeout once and
    re-initialises the status word *and* the stream-K tile counters, so that the next
    launch on that workspace is correct again."""
    from harness import CaseSpec
    workload = get_workload("nvfp4_gemm")(None, device="cuda")
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    m, n, k = 128, 256, 4096
    plan = native.Plan.dense(0, native.OUT_F16, m, n, k, 1, schedule=2, tile_n=128)
    inputs = workload.get_inputs(CaseSpec("reset", {"m": m, "n": n, "k": k, "l": 1}, 9))
    want = oracle_dense(inputs)
    ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
    plan.init_workspace(ws.data_ptr(), stream)
    # What an abandoned stream-K launch leaves behind: a status code and arrival counters
    # that never reached their reset.
    words = ws[:512].view(torch.int32)
    words[0] = 2
    words[64:66] = 1
    with pytest.raises(native.NativeError):
        plan.status(ws.data_ptr(), stream)
    torch.cuda.synchronize()
    assert int(words[0]) == 0 and int(words[64]) == 0 and int(words[65]) == 0
    d = torch.full((1, m, n), float("nan"), dtype=torch.float16, device=dev)
    plan.launch_dense(*(t.data_ptr() for t in inputs), d.data_ptr(), ws.data_ptr(), stream)
    assert plan.status(ws.data_ptr(), stream) == 0
    assert np.array_equal(d.cpu().numpy(), want)
    plan.destroy()


@pytest.mark.parametrize("schedule", (1, 2))
def test_abandoned_wait_is_reported_and_the_context_stays_usable(schedule):
    """The bounded waits, exercised without a fault: in the self-test build of the dense
    kernel the producer issues no copy, so the MMA, scale-mover and epilogue roles wait on
    barriers that nothing completes and give up after a few milliseconds. The kernel must
    return by itself (tensor memory freed: the launch that follows allocates it again),
    leave a code in the status word, and nvfp4_plan_status must report the timeout once and
    re-initialise the workspace, after which the same workspace gives the exact result."""
    from harness import CaseSpec
    workload = get_workload("nvfp4_gemm")(None, device="cuda")
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    m, n, k = 256, 384, 2048
    plan = native.Plan.dense(0, native.OUT_F16, m, n, k, 1, schedule=schedule, tile_n=128)
    inputs = workload.get_inputs(CaseSpec("stall", {"m": m, "n": n, "k": k, "l": 1}, 13))
    want = oracle_dense(inputs)
    ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
    plan.init_workspace(ws.data_ptr(), stream)
    d = torch.full((1, m, n), float("nan"), dtype=torch.float16, device=dev)
    pointers = [t.data_ptr() for t in inputs]
    for _ in range(2):
        plan.selftest_abandoned_wait(*pointers, d.data_ptr(), ws.data_ptr(), stream)
        with pytest.raises(native.NativeError) as caught:
            plan.status(ws.data_ptr(), stream)
        assert caught.value.status == native.E_DEVICE_TIMEOUT
        assert torch.isnan(d).all(), "an abandoned launch must not have written D"
        assert plan.status(ws.data_ptr(), stream) == 0  # reported once, then clear
        plan.launch_dense(*pointers, d.data_ptr(), ws.data_ptr(), stream)
        assert plan.status(ws.data_ptr(), stream) == 0
        assert np.array_equal(d.cpu().numpy(), want)
        d.fill_(float("nan"))
    with pytest.raises(ValueError):
        other = native.Plan.dense(0, native.OUT_F16, m, n, k, 1, tile_n=256, schedule=1)
        try:
            other.selftest_abandoned_wait(*pointers, d.data_ptr(), ws.data_ptr(), stream)
        finally:
            other.destroy()
    plan.destroy()


@pytest.mark.parametrize("block,out_kind,config", [
    (32, native.OUT_BF16, {}), (16, native.OUT_F16, {}), (32, native.OUT_F16, {"pair": 1}),
    (32, native.OUT_F32, {"schedule": 2, "tile_n": 128}), (16, native.OUT_BF16, {"schedule": 3}),
    (32, native.OUT_F16, {"tile_n": 64, "schedule": 1}),
])
def test_shuffled_weights_give_the_logical_result_bit_for_bit(block, out_kind, config):
    """B and its scales in FlashInfer's epilogue-shuffled row order (blocks of 32 and of 16
    rows) through every epilogue that undoes the permutation: whole tiles, the stream-K
    fix-up, the cluster reduction, the 2-CTA kernel. The same plan kind on the logical
    operands must give the same bits (the products and their order are the same; only
    the column a value is stored in differs), and the oracle agrees exactly."""
    from harness import CaseSpec
    from harness.workloads.nvfp4_gemm import from_task_scales, to_task_scales
    from harness.workloads.quantization import shuffle_rows
    workload = get_workload("nvfp4_gemm")(None, device="cuda")
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    m, n, k = (512, 768, 2048) if config.get("pair") else (200, 416, 4096)
    dtype = {native.OUT_F16: torch.float16, native.OUT_BF16: torch.bfloat16,
             native.OUT_F32: torch.float32}[out_kind]
    a, b, sfa, sfb, alpha = workload.get_inputs(
        CaseSpec("shuffled", {"m": m, "n": n, "k": k, "l": 1, "alpha": 0.5}, 61))
    idx = shuffle_rows(n, block).to(dev)
    b_physical = b[idx].permute(2, 0, 1).contiguous().permute(1, 2, 0)
    sfb_physical = to_task_scales(from_task_scales(sfb, n, k // 16)[idx].contiguous())
    results = []
    for shuffled in (False, True):
        plan = (native.Plan.dense_shuffled(0, out_kind, m, n, k, 1, block, **config) if shuffled
                else native.Plan.dense(0, out_kind, m, n, k, 1, **config))
        ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
        plan.init_workspace(ws.data_ptr(), stream)
        d = torch.full((1, m, n), float("nan"), dtype=dtype, device=dev)
        operands = (a, b_physical, sfa, sfb_physical, alpha) if shuffled else (a, b, sfa, sfb, alpha)
        plan.launch_dense(*(t.data_ptr() for t in operands), d.data_ptr(), ws.data_ptr(), stream)
        assert plan.status(ws.data_ptr(), stream) == 0
        results.append(d)
        plan.destroy()
    assert torch.equal(results[0], results[1])
    if out_kind == native.OUT_F16:
        want = o.shuffled_gemm(storage(a), storage(b_physical), storage(from_task_scales(sfa, m, k // 16)),
                               storage(from_task_scales(sfb_physical, n, k // 16)), block, 0.5,
                               np.float16)
        assert np.array_equal(results[1].cpu().numpy(), want)
    with pytest.raises(ValueError):
        native.Plan.dense_shuffled(0, out_kind, m, n + 8, k, 1, block)
    with pytest.raises(ValueError):
        native.Plan.dense_shuffled(0, native.OUT_FP4, m, n, k, 1, block)


def test_native_rejects_misaligned_and_wrong_plans():
    stream = torch.cuda.current_stream().cuda_stream
    plan = native.Plan.dense(0, native.OUT_F16, 128, 128, 128, 1)
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    base = buf.data_ptr()
    with pytest.raises(ValueError):
        plan.launch_dense(base + 8, base, base, base, base, base, base, stream)
    with pytest.raises(ValueError):
        plan.launch_dual(base, base, base, base, base, base, base, base, base, stream)
    with pytest.raises(ValueError):
        native.Plan.dense(0, native.OUT_F16, 128, 128, 128, 1, tile_n=96)
    assert native.device_supported(0)
    plan.destroy()
    # Fused dual GEMM: D at 8 modulo 16 is accepted only when rows are n % 8 == 4 elements
    # long (8-byte stores); with n % 8 == 0 the kernel stores 16 bytes at a time. The
    # checks come before any launch, so the buffer's contents do not matter.
    for n, accepted in ((128, False), (132, True)):
        dual = native.Plan.dual(0, 128, n, 128, 1)
        ws = torch.zeros(max(dual.workspace_bytes(), 256), dtype=torch.uint8, device="cuda")
        dual.init_workspace(ws.data_ptr(), stream)
        args = (base, base + 65536, base + 131072, base + 196608, base + 262144, base + 327680,
                base + 393216)
        if accepted:
            dual.launch_dual(*args, base + 458752 + 8, ws.data_ptr(), stream)
            torch.cuda.synchronize()
            assert dual.status(ws.data_ptr(), stream) == 0
        else:
            with pytest.raises(ValueError):
                dual.launch_dual(*args, base + 458752 + 8, ws.data_ptr(), stream)
        dual.destroy()


@pytest.mark.parametrize("rows,k,batches", [(128, 256, 1), (200, 96, 2), (1, 32, 1), (1000, 4096, 1)])
@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
def test_quantiser_kernel_matches_torch_quantiser_bytes(rows, k, batches, dtype):
    """FP32/BF16 -> packed E2M1 + blocked UE4M3 scales in one kernel: byte-identical to the
    torch quantiser (pinned against the reference's convention) followed by the relayout,
    including zero blocks, saturating scales, ties and the zero padding of partial atoms."""
    from harness.workloads import quantization as q
    g = torch.Generator().manual_seed(rows + k)
    x = torch.randn(batches, rows, k, generator=g)
    x[0, 0, :16] = 0.0
    if rows > 1:
        x[0, 1, :16] *= 4000.0
        x[0, rows - 1, -16:] = torch.linspace(-6, 6, 16)
    x = x.to(dtype).cuda().permute(1, 2, 0)
    packed, blocked = q.quantize_nvfp4_native(x)
    torch.cuda.synchronize()
    want_packed, want_scales = q.quantize_nvfp4(x.float())
    assert torch.equal(packed, want_packed)
    assert torch.equal(blocked.view(torch.uint8), q.to_blocked_scales(want_scales).view(torch.uint8))
    # And the oracle agrees on the FP32 path.
    if dtype == torch.float32:
        host = x.permute(2, 0, 1).contiguous().cpu().numpy()
        o_packed, o_scales = o.quantize_nvfp4(host)
        assert np.array_equal(packed.permute(2, 0, 1).cpu().numpy(), o_packed)
        assert np.array_equal(blocked.view(torch.uint8).cpu().numpy(), o.to_blocked(o_scales))


def test_quantiser_kernel_on_ties_and_their_neighbours():
    """Every E4M3 scale with every E2M1 rounding boundary: blocks whose maximum pins the scale
    and whose other elements sit exactly on a boundary times the scale, and one float above
    and below it, with both signs; plus infinities, which take the kernel's other division
    path. Bytes must equal the torch quantiser's (a true division)."""
    from harness.workloads import quantization as q
    bits = torch.arange(1, 127, dtype=torch.uint8)
    scales = bits.view(torch.float8_e4m3fn).float()                       # 126 positive scales
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    exact = (scales[:, None] * bounds[None, :]).reshape(-1)               # exact products
    up = torch.nextafter(exact, torch.tensor(float("inf")))
    down = torch.nextafter(exact, torch.tensor(0.0))
    values = torch.stack([exact, up, down, -exact, -up, -down], dim=1)    # [126 * 7, 6]
    blocks = torch.zeros(values.shape[0], 16)
    blocks[:, 0] = 6.0 * scales.repeat_interleave(7)                      # amax / 6 == scale
    blocks[:, 1:7] = values
    blocks[:, 7:] = torch.randn(values.shape[0], 9) * scales.repeat_interleave(7)[:, None]
    k = 16 * 7
    x = blocks.reshape(126, k)
    special = torch.randn(2, k)
    special[0, 3], special[0, 40], special[1, 100] = float("inf"), float("-inf"), float("inf")
    x = torch.cat([x, special]).reshape(1, 128, k).cuda().permute(1, 2, 0)
    packed, blocked = q.quantize_nvfp4_native(x)
    torch.cuda.synchronize()
    want_packed, want_scales = q.quantize_nvfp4(x)
    assert torch.equal(blocked.view(torch.uint8), q.to_blocked_scales(want_scales).view(torch.uint8))
    assert torch.equal(packed, want_packed)


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
def test_quantiser_on_ragged_blocks_leaves_the_other_rows_alone(dtype):
    """nvfp4_quantize_blocks: the leading rows of every 128-row block are quantised exactly as
    nvfp4_quantize does; rows beyond a block's count keep what the buffers held (here a
    marker), in the codes and in the scales."""
    from harness.workloads import quantization as q
    filled = [128, 5, 0, 77, 128, 1]
    rows, k = 128 * len(filled), 7168
    x = torch.randn((1, rows, k), generator=torch.Generator().manual_seed(3)).to(dtype).cuda()
    want_packed, want_blocked = q.quantize_nvfp4_native(x.permute(1, 2, 0))
    packed = torch.full((rows, k // 2), 0xAB, dtype=torch.uint8, device="cuda")
    blocked = torch.full((len(filled), k // 64, 32, 4, 4), 0xCD, dtype=torch.uint8, device="cuda")
    counts = torch.tensor(filled, dtype=torch.int32, device="cuda")
    native.quantize_blocks(x.data_ptr(), native.IN_F32 if dtype == torch.float32 else native.IN_BF16,
                           packed.data_ptr(), blocked.data_ptr(), rows, k, counts.data_ptr(),
                           torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    live = torch.zeros(rows, dtype=torch.bool, device="cuda")
    for b, count in enumerate(filled):
        live[128 * b:128 * b + count] = True
    assert torch.equal(packed[live], want_packed[..., 0][live])
    assert (packed[~live] == 0xAB).all()
    # Scale byte (r, c) sits at [r / 128][c / 4][r % 32][(r / 32) % 4][c % 4].
    got = blocked.permute(0, 3, 2, 1, 4).reshape(rows, k // 16)      # [block][r/32%4][r%32] -> row
    want = want_blocked.view(torch.uint8)[0].permute(0, 3, 2, 1, 4).reshape(rows, k // 16)
    assert torch.equal(got[live], want[live])
    assert (got[~live] == 0xCD).all()
    with pytest.raises(ValueError):
        native.quantize_blocks(x.data_ptr(), native.IN_F32, packed.data_ptr(), blocked.data_ptr(),
                               rows, k, 0, 0)


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
def test_gathering_quantiser(dtype):
    """nvfp4_quantize_gather: output row r is the quantised row source[r] of x (rows used
    several times, in any order), rows with source[r] < 0 keep what the buffers held."""
    from harness.workloads import quantization as q
    tokens, rows, k = 300, 640, 2048
    g = torch.Generator().manual_seed(4)
    x = torch.randn((tokens, k), generator=g).to(dtype).cuda()
    source = torch.randint(-1, tokens, (rows,), generator=g, dtype=torch.int32)
    source[128:256] = -1                                   # a whole block without data
    source = source.cuda()
    packed = torch.full((rows, k // 2), 0xAB, dtype=torch.uint8, device="cuda")
    blocked = torch.full((rows // 128, k // 64, 32, 4, 4), 0xCD, dtype=torch.uint8, device="cuda")
    native.quantize_gather(x.data_ptr(), native.IN_F32 if dtype == torch.float32 else native.IN_BF16,
                           packed.data_ptr(), blocked.data_ptr(), rows, k, source.data_ptr(),
                           torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    live = source >= 0
    gathered = x[source.clamp(min=0).long()].float()
    want_packed, want_scales = q.quantize_nvfp4(gathered[..., None])
    assert torch.equal(packed[live], want_packed[..., 0][live])
    assert (packed[~live] == 0xAB).all()
    got = blocked.permute(0, 3, 2, 1, 4).reshape(rows, k // 16)
    assert torch.equal(got[live], want_scales[..., 0].view(torch.uint8)[live])
    assert (got[~live] == 0xCD).all()


def _fp4_out_inputs(m, n, k, batches, scales, seed):
    from harness.workloads import quantization as q
    workload = get_workload("nvfp4_gemm")(None, device="cuda")
    g = torch.Generator(device=workload.device).manual_seed(seed)
    a, sa = q.make_fp4(workload, g, m, k, batches, scales=scales)
    b, sb = q.make_fp4(workload, g, n, k, batches, scales=scales)
    return a, b, sa, sb


@pytest.mark.parametrize("m,n,k,batches", [(128, 256, 512, 1), (200, 192, 96, 2), (1, 64, 32, 1),
                                           (384, 1024, 1024, 1)])
@pytest.mark.parametrize("tile_n", (0, 64, 256))
def test_gemm_with_nvfp4_output_equals_quantised_fp32_product(m, n, k, batches, tile_n):
    """Dense GEMM whose epilogue quantises D to NVFP4: with integer scales every FP32 sum is
    exact, so packed codes and blocked scale bytes must equal the oracle's quantiser applied
    to the oracle's FP32 product, byte for byte (alpha a power of two)."""
    from harness.workloads import quantization as q
    a, b, sa, sb = _fp4_out_inputs(m, n, k, batches, "int0_3", seed=m + n + k)
    alpha = torch.tensor([0.015625], dtype=torch.float32, device=a.device)
    sfa, sfb = q.to_blocked_scales(sa), q.to_blocked_scales(sb)
    if tile_n:
        plan = native.Plan.dense(0, native.OUT_FP4, m, n, k, batches, tile_n=tile_n)
        ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=a.device)
        stream = torch.cuda.current_stream().cuda_stream
        plan.init_workspace(ws.data_ptr(), stream)
        packed = torch.empty((batches, m, n // 2), dtype=torch.uint8, device=a.device)
        blocked = torch.zeros((batches, -(-m // 128), n // 64, 32, 4, 4), dtype=torch.uint8,
                              device=a.device)
        plan.launch_dense_fp4(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
                              alpha.data_ptr(), packed.data_ptr(), blocked.data_ptr(),
                              ws.data_ptr(), stream)
        assert plan.status(ws.data_ptr(), stream) == 0
        assert plan.info()["tile_n"] == tile_n and plan.info()["schedule"] == "data_parallel"
        packed = packed.permute(1, 2, 0)
    else:
        packed, blocked = q.fp4_matmul_quantized_native(a, b, sfa, sfb, alpha)
        blocked = blocked.view(torch.uint8)
    torch.cuda.synchronize()
    want_packed, want_scales = o.gemm_quantized(
        storage(a), storage(b), storage(sa), storage(sb), alpha=0.015625)
    assert np.array_equal(packed.permute(2, 0, 1).cpu().numpy(), want_packed)
    assert np.array_equal(blocked.cpu().numpy(), o.to_blocked(want_scales))


def test_gemm_with_nvfp4_output_feeds_the_next_gemm():
    """Two chained GEMMs, D1 = A @ B1^T quantised in the epilogue, D2 = D1q @ B2^T: the
    second GEMM consumes the first one's packed output and blocked scales as they are.
    Checked against the oracle run on the same quantised intermediate (bit-exact inputs to
    the second GEMM because the first has integer scales), at the reference's tolerance."""
    from harness.workloads import quantization as q
    m, n1, k1, n2 = 256, 512, 256, 384
    a, b1, sa, sb1 = _fp4_out_inputs(m, n1, k1, 1, "int0_3", seed=7)
    alpha1 = torch.tensor([0.0078125], dtype=torch.float32, device=a.device)
    d1, sfd1 = q.fp4_matmul_quantized_native(a, b1, q.to_blocked_scales(sa),
                                             q.to_blocked_scales(sb1), alpha1)
    workload = get_workload("nvfp4_gemm").from_arch("sm_100a", device="cuda")
    g = torch.Generator(device=workload.device).manual_seed(8)
    b2, sb2 = q.make_fp4(workload, g, n2, n1, 1)
    one = torch.ones(1, dtype=torch.float32, device=a.device)
    sfd1_task = sfd1.permute(3, 4, 1, 5, 2, 0)
    sfb2_task = q.to_blocked_scales(sb2).permute(3, 4, 1, 5, 2, 0)
    (d2,) = workload.run((d1, b2, sfd1_task, sfb2_task, one))
    torch.cuda.synchronize()
    p1, s1 = o.gemm_quantized(storage(a), storage(b1), storage(sa), storage(sb1), alpha=0.0078125)
    assert np.array_equal(d1.permute(2, 0, 1).cpu().numpy(), p1)
    want = o.gemm(p1, storage(b2), s1, storage(sb2), 1.0, np.float16)
    assert_matches_oracle(d2, want, "chained", exact=False)


def test_nvfp4_output_plan_rejects_what_it_cannot_do():
    with pytest.raises(ValueError):
        native.Plan.dense(0, native.OUT_FP4, 128, 96, 64, 1)      # n not a multiple of 64
    with pytest.raises(ValueError):
        native.Plan.dense(0, native.OUT_FP4, 128, 128, 64, 1, schedule=2)
    plan = native.Plan.dense(0, native.OUT_F16, 128, 128, 64, 1)
    with pytest.raises(ValueError):
        plan.launch_dense_fp4(256, 256, 256, 256, 256, 256, 256, 256, 0)


@pytest.mark.parametrize("m,n,k,l", [(300, 264, 2080, 1), (512, 1024, 1024, 1), (130, 328, 512, 2)])
def test_dual_gemm_on_cta_pairs(m, n, k, l):  # noqa: E741
    """The fused dual GEMM on the 2-CTA kernel: the leader loads B1's tile, its peer B2's, one
    256-column MMA per pair; partial tiles in M and N (also a last 64-column box that is
    partly and one that is wholly outside D), a K tail, batches. The kernel stores D through
    a tensor map, so rows of D that are only 8-byte aligned (n = 260) are refused for it."""
    from harness import CaseSpec
    with pytest.raises(ValueError):
        native.Plan.dual(0, 130, 260, 512, 2, pair=1)
    workload = get_workload("nvfp4_dual_gemm")(None, device="cuda")
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    case = CaseSpec("dual_pair", {"m": m, "n": n, "k": k, "l": l, "alpha": 0.25}, 41)
    inputs = workload.get_inputs(case)
    (ref,) = workload.get_reference(inputs)
    plan = native.Plan.dual(0, m, n, k, l, pair=1)
    assert plan.info()["tile_m"] == 256, plan.info()
    ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
    plan.init_workspace(ws.data_ptr(), stream)
    d = torch.full((l, m, n), float("nan"), dtype=torch.float16, device=dev)
    for _ in range(2):
        plan.launch_dual(*(t.data_ptr() for t in inputs), d.data_ptr(), ws.data_ptr(), stream)
    assert plan.status(ws.data_ptr(), stream) == 0
    torch.testing.assert_close(d.permute(1, 2, 0), ref, rtol=1e-3, atol=1e-3)
    plan.destroy()


def test_mma_issue_peak_measurement_is_plausible():
    """The library's own FP4 MMA issue-rate microbenchmark: near the nominal 9 PFLOP/s on a
    B200 at full clocks, and never below what the GEMM kernels reach."""
    value = native.measure_mma_peak(0, 2048)
    assert 4000.0 < value < 12000.0, value
    with pytest.raises(ValueError):
        native.measure_mma_peak(0, 0)


@pytest.mark.parametrize("m,n,k,batches", [(256, 256, 256, 1), (300, 576, 608, 2), (1024, 2048, 1024, 1)])
@pytest.mark.parametrize("scales", ("int0_3", "uniform"))
def test_pair_kernel_with_nvfp4_output(m, n, k, batches, scales):
    """The 2-CTA kernel's NVFP4 epilogue (partial tiles in M, N and K, batches): packed codes
    and blocked scales equal, byte for byte, the quantiser kernel applied to the FP32 output
    of the same kernel, and (integer scales: sums exact in any order) the single-CTA plan's."""
    from harness.workloads import quantization as q
    a, b, sa, sb = _fp4_out_inputs(m, n, k, batches, scales, seed=m + n + k + 1)
    alpha = torch.tensor([0.25], dtype=torch.float32, device=a.device)
    sfa, sfb = q.to_blocked_scales(sa), q.to_blocked_scales(sb)
    stream = torch.cuda.current_stream().cuda_stream

    def run(out_kind, **config):
        plan = native.Plan.dense(0, out_kind, m, n, k, batches, **config)
        ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=a.device)
        plan.init_workspace(ws.data_ptr(), stream)
        if out_kind == native.OUT_FP4:
            packed = torch.full((batches, m, n // 2), 0xEE, dtype=torch.uint8, device=a.device)
            blocked = torch.zeros((batches, -(-m // 128), n // 64, 32, 4, 4), dtype=torch.uint8,
                                  device=a.device)
            plan.launch_dense_fp4(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
                                  alpha.data_ptr(), packed.data_ptr(), blocked.data_ptr(),
                                  ws.data_ptr(), stream)
            out = (packed, blocked)
        else:
            d = torch.empty((batches, m, n), dtype=torch.float32, device=a.device)
            plan.launch_dense(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
                              alpha.data_ptr(), d.data_ptr(), ws.data_ptr(), stream)
            out = d
        assert plan.status(ws.data_ptr(), stream) == 0
        info = plan.info()
        plan.destroy()
        return out, info

    (packed, blocked), info = run(native.OUT_FP4, pair=1)
    assert info["tile_m"] == 256 and info["tile_n"] == 256, info
    product, _ = run(native.OUT_F32, pair=1)
    want_packed, want_scales = q.quantize_nvfp4_native(product.permute(1, 2, 0))
    assert torch.equal(packed, want_packed.permute(2, 0, 1))
    assert torch.equal(blocked, want_scales.view(torch.uint8))
    if scales == "int0_3":
        (single_packed, single_blocked), single = run(native.OUT_FP4, pair=-1)
        assert single["tile_m"] == 128
        assert torch.equal(packed, single_packed) and torch.equal(blocked, single_blocked)


@pytest.mark.parametrize("m,n,k,l", [(256, 128, 256, 1), (300, 320, 608, 2), (512, 1024, 2080, 1)])
def test_dual_pair_kernel_with_nvfp4_output(m, n, k, l):  # noqa: E741
    """Gate/up dual GEMM with NVFP4 output on the 2-CTA kernel against the single-CTA plan:
    integer scales, so both epilogues see the same FP32 sums and must write the same bytes."""
    from harness import CaseSpec
    workload = get_workload("nvfp4_dual_gemm")(None, device="cuda")
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    case = CaseSpec("dual_fp4_pair", {"m": m, "n": n, "k": k, "l": l, "alpha": 0.0625,
                                      "scales": "int0_3"}, 52)
    inputs = workload.get_inputs(case)
    results = []
    for config in ({"pair": 1}, {"pair": -1}):
        plan = native.Plan.dual_fp4(0, m, n, k, l, **config)
        ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
        plan.init_workspace(ws.data_ptr(), stream)
        packed = torch.zeros((l, m, n // 2), dtype=torch.uint8, device=dev)
        blocked = torch.zeros((l, -(-m // 128), n // 64, 32, 4, 4), dtype=torch.uint8, device=dev)
        plan.launch_dual_fp4(*(t.data_ptr() for t in inputs), packed.data_ptr(),
                             blocked.data_ptr(), ws.data_ptr(), stream)
        assert plan.status(ws.data_ptr(), stream) == 0
        results.append((packed, blocked, plan.info()))
        plan.destroy()
    assert results[0][2]["tile_m"] == 256 and results[1][2]["tile_m"] == 128
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
    assert results[0][0].any()


@pytest.mark.parametrize("m,n,k,l,tile_n", [(256, 512, 1024, 1, 0), (200, 192, 2080, 2, 128), (130, 320, 512, 1, 256)])
def test_dual_gemm_with_nvfp4_output(m, n, k, l, tile_n):  # noqa: E741
    """Gate/up dual GEMM quantised to NVFP4 in its epilogue. The kernel's silu uses
    approximate exp and reciprocal, so codes may differ from the oracle's at E2M1 rounding
    boundaries: nearly all bytes equal, and the dequantised tensors agree to well inside one
    quantisation step of the tensor's scale."""
    from harness import CaseSpec
    workload = get_workload("nvfp4_dual_gemm")(None, device="cuda")
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    case = CaseSpec("dual_fp4", {"m": m, "n": n, "k": k, "l": l, "alpha": 0.0625}, 51)
    inputs = workload.get_inputs(case)
    a, b1, b2, sfa, sfb1, sfb2, alpha = inputs
    plan = native.Plan.dual_fp4(0, m, n, k, l, **({"tile_n": tile_n} if tile_n else {}))
    ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
    plan.init_workspace(ws.data_ptr(), stream)
    packed = torch.zeros((l, m, n // 2), dtype=torch.uint8, device=dev)
    blocked = torch.zeros((l, -(-m // 128), n // 64, 32, 4, 4), dtype=torch.uint8, device=dev)
    plan.launch_dual_fp4(*(t.data_ptr() for t in inputs), packed.data_ptr(), blocked.data_ptr(),
                         ws.data_ptr(), stream)
    assert plan.status(ws.data_ptr(), stream) == 0
    sa = o.from_blocked(blocked_storage(sfa), m, k // 16)
    s1 = o.from_blocked(blocked_storage(sfb1), n, k // 16)
    s2 = o.from_blocked(blocked_storage(sfb2), n, k // 16)
    want_packed, want_scales = o.dual_gemm_quantized(storage(a), storage(b1), storage(b2), sa, s1,
                                                     s2, float(alpha.item()))
    got_packed = packed.cpu().numpy()
    got_scales = o.from_blocked(blocked.cpu().numpy(), m, n // 16)
    assert (got_packed != want_packed).mean() < 5e-3
    assert (got_scales != want_scales).mean() < 5e-3
    got = o.dequant(got_packed, got_scales)
    want = o.dequant(want_packed, want_scales)
    assert np.linalg.norm(got - want) <= 2e-2 * np.linalg.norm(want)
    plan.destroy()
