"""The plan the library picks by itself against every plan that can be forced, timed on the
GPU: the schedule model is a handful of measured constants, and a kernel change must not be
able to make it pick a clearly slower plan without a test noticing."""

import pytest
import torch

from harness import native

pytestmark = pytest.mark.gpu

SETS = 3       # operand sets that rotate (more than L2 for the large shapes)
LAUNCHES = 30  # per timed graph replay
TOLERANCE = 1.30  # candidates within 15 % of each other swap places from GPU to GPU


def random_operands(kind, m, n, k, device):
    """Random E2M1 bytes and scale bytes in [0.5, 1): timing does not depend on the values."""
    g = torch.Generator(device=device).manual_seed(m + n + k)

    def rnd(shape, lo, hi):
        return torch.randint(lo, hi, shape, dtype=torch.uint8, device=device, generator=g)

    atoms = lambda rows: (-(-rows // 128)) * (-(-k // 64)) * 512  # noqa: E731
    sets = []
    for _ in range(SETS):
        a, sfa = rnd((1, m, k // 2), 0, 256), rnd((atoms(m),), 0x30, 0x38)
        bs = [(rnd((1, n, k // 2), 0, 256), rnd((atoms(n),), 0x30, 0x38))
              for _ in range(2 if kind == "dual" else 1)]
        d = torch.zeros((1, m, n), dtype=torch.float16, device=device)
        sets.append((a, sfa, bs, d))
    return sets


def time_plan(kind, plan, sets, device):
    """Microseconds per launch of ``plan`` replayed from a CUDA graph over the operand sets."""
    stream = torch.cuda.current_stream(device).cuda_stream
    ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=device)
    plan.init_workspace(ws.data_ptr(), stream)
    alpha = torch.ones(1, device=device)

    def launch(i):
        a, sfa, bs, d = sets[i % SETS]
        s = torch.cuda.current_stream(device).cuda_stream
        if kind == "dual":
            plan.launch_dual(a.data_ptr(), bs[0][0].data_ptr(), bs[1][0].data_ptr(), sfa.data_ptr(),
                             bs[0][1].data_ptr(), bs[1][1].data_ptr(), alpha.data_ptr(),
                             d.data_ptr(), ws.data_ptr(), s)
        else:
            plan.launch_dense(a.data_ptr(), bs[0][0].data_ptr(), sfa.data_ptr(), bs[0][1].data_ptr(),
                              alpha.data_ptr(), d.data_ptr(), ws.data_ptr(), s)

    for i in range(SETS):
        launch(i)
    torch.cuda.synchronize(device)
    assert plan.status(ws.data_ptr(), stream) == 0
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(LAUNCHES):
            launch(i)
    graph.replay()
    torch.cuda.synchronize(device)
    best = float("inf")
    for _ in range(3):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize(device)
        best = min(best, start.elapsed_time(stop) * 1e3 / LAUNCHES)
    assert plan.status(ws.data_ptr(), stream) == 0
    return best


def describe(info):
    return (info["tile_m"], info["tile_n"], info["schedule"], info["ctas"])


@pytest.mark.parametrize("kind,m,n,k", [
    ("dense", 128, 7168, 16384),    # decode: cluster split-K
    ("dense", 16, 7168, 2048),      # a few rows on many columns
    ("dense", 512, 4096, 7168),     # one wave of tiles
    ("dense", 2048, 2048, 2048),    # mid-size, several candidates close together
    ("dense", 4096, 8192, 7168),    # compute bound: the 2-CTA kernel
    ("dual", 256, 4096, 7168),      # gate/up at decode size
    ("dual", 4096, 4096, 7168),     # gate/up at prefill size
])
def test_the_chosen_plan_is_not_clearly_slower_than_a_forced_one(kind, m, n, k):
    device = torch.device("cuda:0")
    sets = random_operands(kind, m, n, k, device)

    def make(**config):
        if kind == "dual":
            return native.Plan.dual(0, m, n, k, 1, **config)
        return native.Plan.dense(0, native.OUT_F16, m, n, k, 1, **config)

    chosen = make()
    chosen_info = describe(chosen.info())
    chosen_us = time_plan(kind, chosen, sets, device)
    chosen.destroy()

    seen = {chosen_info: chosen_us}
    candidates = [dict(tile_n=t, schedule=s) for t in ((128, 256) if kind == "dual" else (64, 128, 256))
                  for s in (1, 2, 3)] + [dict(pair=1)]
    for config in candidates:
        try:
            plan = make(**config)
        except ValueError:
            continue  # not available for this shape
        info = describe(plan.info())
        if info not in seen:  # a forced plan may fall back to one already timed
            seen[info] = time_plan(kind, plan, sets, device)
        plan.destroy()
    best_info = min(seen, key=seen.get)
    table = ", ".join(f"{key}: {value:.1f} us" for key, value in sorted(seen.items(), key=lambda kv: kv[1]))
    print(f"{kind} {m}x{n}x{k}: chose {chosen_info} at {chosen_us:.1f} us; measured {table}")
    assert chosen_us <= TOLERANCE * seen[best_info], (
        f"{kind} {m}x{n}x{k}: chose {chosen_info} at {chosen_us:.1f} us; measured {table}")
