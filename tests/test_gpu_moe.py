"""The mixture-of-experts layer built on the grouped GEMM and the quantiser kernel, against
the same computation done stage by stage with the harness's torch quantiser and GEMM
reference."""

import numpy as np
import pytest
import torch

from gpu_util import blocked_storage, storage
from harness import CaseSpec, get_workload, moe, native
from harness.workloads import quantization as q
from oracle import nvfp4_oracle as o

pytestmark = pytest.mark.gpu


def quantised_weights(experts, rows, k, seed, device):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(experts, rows, k, generator=g) * 0.05
    packed, scales = q.quantize_nvfp4(w.permute(1, 2, 0))
    packed = packed.permute(2, 0, 1).contiguous().to(device)          # [E, rows, k/2]
    scales = scales.permute(2, 0, 1).contiguous().to(device)          # [E, rows, k/16] logical
    blocked = q.to_blocked_scales(scales.permute(1, 2, 0))            # [E, rb, cb, 32, 4, 4]
    return packed, scales, blocked


def routing(tokens, experts, choices, seed, device):
    g = torch.Generator().manual_seed(seed)
    scores = torch.rand(tokens, experts, generator=g)
    scores[:, experts - 1] = -1.0                      # one expert gets no token at all
    weights, ids = torch.topk(scores, choices, dim=1)
    weights = (weights / weights.sum(dim=1, keepdim=True)).to(device)
    return ids.to(device), weights


@pytest.mark.parametrize("tokens,hidden,inter,experts,choices,fused", [
    (200, 256, 128, 6, 2, True), (200, 256, 128, 6, 2, False), (33, 512, 256, 4, 1, True),
    (33, 512, 192, 4, 1, False), (700, 1024, 512, 8, 2, True)])
def test_moe_layer_matches_stagewise_reference(tokens, hidden, inter, experts, choices, fused):
    """The layer on the grouped kernels (gate/up as the grouped dual GEMM with NVFP4 output
    when ``fused``, else grouped GEMM + torch gate + quantiser) against the same stages in
    torch; a second forward with the same routing pattern reuses the cached plans and gives
    the same bits."""
    device = torch.device("cuda:0")
    g = torch.Generator().manual_seed(tokens)
    x = torch.randn(tokens, hidden, generator=g).to(device)
    ids, weights = routing(tokens, experts, choices, tokens, device)
    w13, w13_logical, w13_blocked = quantised_weights(experts, 2 * inter, hidden, 1, device)
    w2, w2_logical, w2_blocked = quantised_weights(experts, hidden, inter, 2, device)

    layer = moe.MoELayer(w13, w13_blocked, w2, w2_blocked, fused)
    out = layer.forward(x, ids, weights)
    layer.check_status()
    plans = len(layer._plans)
    again = layer.forward(x, ids, weights)
    layer.check_status()
    assert len(layer._plans) == plans == 1 and torch.equal(out, again)
    layer.close()
    ref = moe.moe_reference(x, ids, weights, w13, w13_logical, w2, w2_logical, fused)

    assert out.shape == ref.shape == (tokens, hidden) and torch.isfinite(out).all()
    scale = ref.abs().max().item()
    assert scale > 0
    # Each stage rounds the same FP32 values except for the summation order inside a GEMM
    # (and the fused kernel's approximate silu); a last-bit difference there can move an
    # intermediate across an E2M1 rounding boundary, which changes single terms of a few
    # outputs.
    assert (out - ref).norm().item() <= 3e-3 * ref.norm().item()
    assert (out - ref).abs().max().item() <= 2e-2 * scale
    with pytest.raises(ValueError):
        moe.MoELayer(w13, w13_blocked, w2[:, :, :-8], w2_blocked)


def test_forward_of_a_known_pattern_can_be_captured_in_a_graph():
    """A forward with a routing pattern seen before allocates, encodes and binds nothing: it
    can be captured in a CUDA graph, and the replay gives the same bits on new activations."""
    device = torch.device("cuda:0")
    tokens, hidden, inter, experts, choices = 300, 512, 256, 5, 2
    ids, _ = routing(tokens, experts, choices, 8, device)
    w13, _, w13_blocked = quantised_weights(experts, 2 * inter, hidden, 1, device)
    w2, _, w2_blocked = quantised_weights(experts, hidden, inter, 2, device)
    layer = moe.MoELayer(w13, w13_blocked, w2, w2_blocked)
    source, counts, starts = moe.route_rows(ids, experts)
    gen = torch.Generator().manual_seed(9)
    first = moe._gather(torch.randn(tokens, hidden, generator=gen).to(device), source, choices)
    second = moe._gather(torch.randn(tokens, hidden, generator=gen).to(device), source, choices)
    rows = first.clone()
    side = torch.cuda.Stream(device)
    with torch.cuda.stream(side):
        want_first = layer.forward_rows(rows, counts, starts).clone()   # creates the pattern
        rows.copy_(second)
        want_second = layer.forward_rows(rows, counts, starts).clone()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            y = layer.forward_rows(rows, counts, starts)
        rows.copy_(first)
        graph.replay()
        side.synchronize()
        assert torch.equal(y, want_first)
        rows.copy_(second)
        graph.replay()
        side.synchronize()
        assert torch.equal(y, want_second) and not torch.equal(want_first, want_second)
    layer.check_status()
    assert len(layer._plans) == 1
    layer.close()


@pytest.mark.parametrize("tokens,experts,choices,dtype", [
    (1000, 8, 2, torch.int64), (37, 5, 1, torch.int32), (4096, 256, 8, torch.int64), (1, 3, 1, torch.int64)])
def test_device_routing_places_every_pair_in_its_experts_block(tokens, experts, choices, dtype):
    """nvfp4_moe_count / nvfp4_moe_place: counts equal a bincount; every pair gets its own row
    inside its expert's 128-row-padded block; the rows remember their token; all other rows
    are padding."""
    g = torch.Generator().manual_seed(tokens + experts)
    scores = torch.rand(tokens, experts, generator=g)
    if experts > 2:
        scores[:, 1] = -1.0                                  # an expert without any pair
    ids = torch.topk(scores, choices, dim=1).indices.to(dtype).cuda()
    routing = moe.DeviceRouting(ids, experts)
    torch.cuda.synchronize()
    flat = ids.reshape(-1).long()
    assert routing.counts == torch.bincount(flat, minlength=experts).tolist()
    assert all(start % 128 == 0 for start in routing.starts)
    rows = routing.row_of_pair.long()
    starts = torch.tensor(routing.starts, device="cuda")[flat]
    counts = torch.tensor(routing.counts, device="cuda")[flat]
    assert ((rows >= starts) & (rows < starts + counts)).all()
    assert rows.unique().numel() == rows.numel()
    pairs = torch.arange(flat.numel(), device="cuda")
    assert torch.equal(routing.token_of_row[rows].long(), pairs // choices)
    padding = torch.ones_like(routing.token_of_row, dtype=torch.bool)
    padding[rows] = False
    assert (routing.token_of_row[padding] == -1).all()
    assert routing.token_of_row.numel() == max(128, sum(-(-c // 128) * 128 for c in routing.counts))


def test_routed_layer_needs_no_host_read_and_equals_the_planned_layer():
    """RoutedMoELayer (row counts, layout, placement on the device; one pair of plans for any
    routing) against MoELayer (plans per routing pattern) on several routings, with experts
    that get nothing and experts that get more than one 128-row block: every row is computed
    on its own, so the two must agree bit for bit. Then the routed forward captured once in a
    CUDA graph is replayed on other tokens and other expert choices."""
    device = torch.device("cuda:0")
    hidden, inter, experts, choices, tokens = 512, 256, 7, 2, 400
    w13, _, w13_blocked = quantised_weights(experts, 2 * inter, hidden, 1, device)
    w2, _, w2_blocked = quantised_weights(experts, hidden, inter, 2, device)
    planned = moe.MoELayer(w13, w13_blocked, w2, w2_blocked, fused=True)
    routed = moe.RoutedMoELayer(w13, w13_blocked, w2, w2_blocked, max_pairs=tokens * choices)
    g = torch.Generator().manual_seed(21)
    cases = []
    for seed in (1, 2, 3):
        x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).to(device)
        ids, weights = routing(tokens, experts, choices, seed, device)
        if seed == 3:
            ids = torch.zeros_like(ids)           # everything to one expert (and a duplicate)
            ids[:, 1] = 3
        want = planned.forward(x, ids, weights)
        got = routed.forward(x, ids, weights)
        assert torch.equal(got, want) and torch.isfinite(got).all() and got.abs().max() > 0
        cases.append((x, ids, weights, want))
    planned.check_status()
    routed.check_status()
    fewer = routed.forward(cases[0][0][:50], cases[0][1][:50], cases[0][2][:50])
    assert torch.equal(fewer, planned.forward(cases[0][0][:50], cases[0][1][:50], cases[0][2][:50]))

    side = torch.cuda.Stream(device)
    x_in, ids_in, w_in = (t.clone() for t in cases[0][:3])
    with torch.cuda.stream(side):
        routed.forward(x_in, ids_in, w_in)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            out = routed.forward(x_in, ids_in, w_in)
        for x, ids, weights, want in reversed(cases):
            x_in.copy_(x)
            ids_in.copy_(ids)
            w_in.copy_(weights)
            graph.replay()
            side.synchronize()
            assert torch.equal(out, want)
    routed.check_status()
    with pytest.raises(ValueError):
        routed.forward(torch.cat([x_in, x_in]), torch.cat([ids_in, ids_in]), torch.cat([w_in, w_in]))
    planned.close()
    routed.close()


def test_routed_layout_that_does_not_fit_is_reported():
    """A routed plan whose shared buffers are too small for the counts it is given cuts the
    groups and says so through the status call, once; a layout that fits clears nothing else."""
    device = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    plan = native.Plan.routed(0, native.OUT_F16, 3, 256, 256, 256)
    ws = torch.zeros(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=device)
    plan.init_workspace(ws.data_ptr(), stream)
    a = torch.zeros((256, 128), dtype=torch.uint8, device=device)
    sfa = torch.zeros((2, 4, 512), dtype=torch.uint8, device=device)
    b = torch.zeros((3, 256, 128), dtype=torch.uint8, device=device)
    sfb = torch.zeros((3, 2, 4, 512), dtype=torch.uint8, device=device)
    d = torch.zeros((256, 256), dtype=torch.float16, device=device)
    plan.bind_routed(a.data_ptr(), sfa.data_ptr(), [b[e].data_ptr() for e in range(3)],
                     [sfb[e].data_ptr() for e in range(3)], d.data_ptr(), ws.data_ptr(), stream)
    fits = torch.tensor([100, 0, 128], dtype=torch.int32, device=device)
    plan.layout_routed(fits.data_ptr(), ws.data_ptr(), stream)
    plan.launch_groups(ws.data_ptr(), stream)
    assert plan.status(ws.data_ptr(), stream) == 0
    too_many = torch.tensor([100, 100, 100], dtype=torch.int32, device=device)
    plan.layout_routed(too_many.data_ptr(), ws.data_ptr(), stream)
    plan.launch_groups(ws.data_ptr(), stream)
    with pytest.raises(ValueError):
        plan.status(ws.data_ptr(), stream)
    plan.layout_routed(fits.data_ptr(), ws.data_ptr(), stream)
    assert plan.status(ws.data_ptr(), stream) == 0
    plan.destroy()


def test_combine_kernel_matches_a_gather_and_a_batched_product():
    """nvfp4_moe_combine: the weighted sum of each token's rows in FP32, padding rows (-1)
    adding nothing."""
    device = torch.device("cuda:0")
    tokens, choices, hidden, rows = 333, 4, 1032, 2000
    g = torch.Generator().manual_seed(11)
    y = torch.randn(rows, hidden, generator=g).half().to(device)
    picks = torch.randint(0, rows, (tokens, choices), generator=g, dtype=torch.int32)
    picks[5, 1] = -1
    picks = picks.to(device)
    weights = torch.rand(tokens, choices, generator=g).to(device)
    out = torch.full((tokens, hidden), float("nan"), device=device)
    native.moe_combine(y.data_ptr(), picks.data_ptr(), weights.data_ptr(), out.data_ptr(), tokens,
                       choices, hidden, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    picked = y.float()[picks.clamp(min=0).long().reshape(-1)].view(tokens, choices, hidden)
    used = (picks >= 0).float() * weights
    want = torch.einsum("tk,tkh->th", used.double(), picked.double())
    assert torch.allclose(out.double(), want, rtol=1e-6, atol=1e-6)
    with pytest.raises(ValueError):
        native.moe_combine(y.data_ptr(), picks.data_ptr(), weights.data_ptr(), out.data_ptr(),
                           tokens, choices, 1030, 0)


def test_fused_and_unfused_layers_agree():
    device = torch.device("cuda:0")
    tokens, hidden, inter, experts, choices = 300, 512, 256, 5, 2
    x = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(5)).to(device)
    ids, weights = routing(tokens, experts, choices, 6, device)
    w13, _, w13_blocked = quantised_weights(experts, 2 * inter, hidden, 1, device)
    w2, _, w2_blocked = quantised_weights(experts, hidden, inter, 2, device)
    fused = moe.moe_forward(x, ids, weights, w13, w13_blocked, w2, w2_blocked, fused=True)
    plain = moe.moe_forward(x, ids, weights, w13, w13_blocked, w2, w2_blocked, fused=False)
    # They differ by the FP16 rounding of the two projections that the fused kernel skips.
    assert (fused - plain).norm().item() <= 1e-2 * plain.norm().item()


EP_WORKER = """
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, {package!r}); sys.path.insert(0, {repo!r}); sys.path.insert(0, {tests!r})
from harness import moe
from test_gpu_moe import quantised_weights, routing
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
device = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=device)
experts, hidden, inter, tokens, choices = 8, 512, 256, 150 + 20 * rank, 2
per_rank = experts // world
w13, w13_logical, w13_blocked = quantised_weights(experts, 2 * inter, hidden, 1, device)
w2, w2_logical, w2_blocked = quantised_weights(experts, hidden, inter, 2, device)
x = torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(50 + rank)).to(device)
ids, weights = routing(tokens, experts, choices, 60 + rank, device)
mine = slice(rank * per_rank, (rank + 1) * per_rank)
layer = moe.MoELayer(w13[mine].contiguous(), w13_blocked[mine].contiguous(),
                     w2[mine].contiguous(), w2_blocked[mine].contiguous())
out = moe.moe_forward_ep(x, ids, weights, experts, moe.ep_local_experts(layer))
layer.check_status()
routed = moe.RoutedMoELayer(w13[mine].contiguous(), w13_blocked[mine].contiguous(),
                            w2[mine].contiguous(), w2_blocked[mine].contiguous(), max_pairs=4096)
again = moe.moe_forward_ep(x, ids, weights, experts, moe.ep_local_experts(routed))
routed.check_status()
ref = moe.moe_reference(x, ids, weights, w13, w13_logical, w2, w2_logical, fused=True)
ok = (out - ref).norm().item() <= 3e-3 * ref.norm().item() and bool(torch.isfinite(out).all())
ok = ok and torch.equal(out, again)
routed.close()
flag = torch.tensor([1.0 if ok else 0.0], device=device)
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
layer.close()
dist.destroy_process_group()
if rank == 0:
    print("EP_OK" if flag.item() == 1.0 else "EP_MISMATCH", flush=True)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_layer_on_all_gpus(tmp_path):
    """Expert-parallel forward over every GPU of the box (one process per GPU, NCCL
    all-to-all for dispatch and combine, each rank's experts on the grouped kernels): every
    rank's tokens against the single-GPU reference of the whole layer."""
    import subprocess
    import sys
    from pathlib import Path

    world = min(torch.cuda.device_count(), 8)
    while 8 % world:
        world -= 1
    tests = Path(__file__).resolve().parent
    script = tmp_path / "ep_worker.py"
    script.write_text(EP_WORKER.format(package=str(tests.parent / "flashinfer-cubins_b200"),
                                       repo=str(tests.parent), tests=str(tests)))
    run = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
         "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
        capture_output=True, text=True, timeout=600,
        env={**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"})
    assert run.returncode == 0 and "EP_OK" in run.stdout, run.stdout[-2000:] + run.stderr[:6000]


def test_route_rows_pads_every_expert_to_whole_scale_atoms():
    ids = torch.tensor([[0, 2], [2, 1], [2, 0], [0, 2]], device="cuda")
    source, counts, starts = moe.route_rows(ids, 4)
    assert counts == [3, 1, 4, 0] and starts == [0, 128, 256, 384]
    assert source.numel() == 384
    assert source[:3].tolist() == [0, 5, 6] and source[128].item() == 3
    assert source[256:260].tolist() == [1, 2, 4, 7] and (source[3:128] == -1).all()


@pytest.mark.parametrize("tile_n", (128, 256))
def test_grouped_dual_gemm_with_nvfp4_output(tile_n):
    """The grouped gate/up kernel: every group's packed E2M1 bytes and blocked scales equal
    what the dense fused dual GEMM with NVFP4 output gives for that group alone (same
    arithmetic, same tile order inside a group), and agree with the oracle's quantised dual
    GEMM up to E2M1 rounding boundaries of the approximate silu. Groups of 1 to 300 rows,
    partial tiles in M and N, a K tail."""
    workload = get_workload("nvfp4_dual_gemm")(None, device="cuda")
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    n, k = 192, 1056
    groups = []
    for g, m in enumerate((1, 130, 300, 64)):
        case = CaseSpec("group", {"m": m, "n": n, "k": k, "l": 1, "alpha": 1.0}, 70 + g)
        groups.append((m, workload.get_inputs(case)))
    plan = native.Plan.grouped_dual_fp4(0, [(m, n, k) for m, _ in groups], tile_n=tile_n)
    ws = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
    plan.init_workspace(ws.data_ptr(), stream)
    outs = [(torch.zeros((1, m, n // 2), dtype=torch.uint8, device=dev),
             torch.zeros((1, -(-m // 128), n // 64, 32, 4, 4), dtype=torch.uint8, device=dev))
            for m, _ in groups]
    columns = list(zip(*[[t.data_ptr() for t in inputs[:6]] for _, inputs in groups]))
    a, b1, b2, sfa, sfb1, sfb2 = columns
    plan.bind_dual_groups_fp4(a, b1, b2, sfa, sfb1, sfb2, [p.data_ptr() for p, _ in outs],
                              [s.data_ptr() for _, s in outs], ws.data_ptr(), stream)
    plan.launch_groups(ws.data_ptr(), stream)
    assert plan.status(ws.data_ptr(), stream) == 0
    for (m, inputs), (packed, blocked) in zip(groups, outs):
        single = native.Plan.dual_fp4(0, m, n, k, 1, tile_n=tile_n)
        sws = torch.empty(max(single.workspace_bytes(), 256), dtype=torch.uint8, device=dev)
        single.init_workspace(sws.data_ptr(), stream)
        want_packed = torch.zeros_like(packed)
        want_blocked = torch.zeros_like(blocked)
        single.launch_dual_fp4(*(t.data_ptr() for t in inputs), want_packed.data_ptr(),
                               want_blocked.data_ptr(), sws.data_ptr(), stream)
        assert single.status(sws.data_ptr(), stream) == 0
        single.destroy()
        assert torch.equal(packed, want_packed), f"group of {m} rows: packed bytes differ"
        got_scales = o.from_blocked(blocked.cpu().numpy(), m, n // 16)
        assert np.array_equal(got_scales, o.from_blocked(want_blocked.cpu().numpy(), m, n // 16))
        a_t, b1_t, b2_t, sfa_t, s1_t, s2_t, alpha = inputs
        oracle_packed, oracle_scales = o.dual_gemm_quantized(
            storage(a_t), storage(b1_t), storage(b2_t),
            o.from_blocked(blocked_storage(sfa_t), m, k // 16),
            o.from_blocked(blocked_storage(s1_t), n, k // 16),
            o.from_blocked(blocked_storage(s2_t), n, k // 16), 1.0)
        assert (packed.cpu().numpy() != oracle_packed).mean() < 5e-3
        assert (got_scales != oracle_scales).mean() < 5e-3
    with pytest.raises(ValueError):
        native.Plan.grouped_dual_fp4(0, [(16, 96, 64)])      # n not a multiple of 64
    with pytest.raises(ValueError):
        native.Plan.grouped_dual_fp4(0, [(16, 128, 64)], schedule=2)
    plan.destroy()

