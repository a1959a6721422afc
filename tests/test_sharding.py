"""Host logic of the multi-GPU path: shard boundaries, group balancing, and a
world-size-2 gloo run on CPU in which every rank computes its N-shard with the torch
reference and the all-gathered result equals the unsharded one."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from harness import CaseSpec, get_workload
from harness import sharding


def test_row_shards_split_on_atom_boundaries():
    for n, world in ((7168, 8), (7168, 2), (8192, 4), (4104, 4), (136, 2), (128, 4), (1, 1)):
        spans = sharding.row_shards(n, world)
        assert len(spans) == world and spans[0][0] == 0 and spans[-1][1] == n
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            assert a1 == b0 and a1 % 128 == 0 or a1 == n
        widths = [b - a for a, b in spans if b > a]
        assert max(widths) - min(widths) <= 128 or n % 128
    assert sharding.row_shards(7168, 8) == [(896 * r, 896 * (r + 1)) for r in range(8)]
    with pytest.raises(ValueError):
        sharding.row_shards(0, 2)


def test_group_balancing_numbers():
    ms = (40, 96, 128, 256, 384, 512, 768, 1024)
    problems = [(m, 4096, 7168) for m in ms]
    owned = sharding.balance_groups(problems, 2)
    assert sorted(i for part in owned for i in part) == list(range(8))
    # Whole-group placement cannot pass total / largest group.
    assert abs(sharding.balance_speedup(problems, 2) - 3208 / 1632) < 1e-9
    assert abs(sharding.balance_speedup(problems, 8) - 3208 / 1024) < 1e-9
    # Cutting every group along N balances exactly.
    for rank in range(8):
        units = sharding.slice_groups(problems, rank, 8)
        assert [stop - start for _, start, stop in units] == [512] * 8


def free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def shard_worker(rank: int, world: int, port: int, queue) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        dense = get_workload("nvfp4_gemm")(None, device="cpu")
        case = CaseSpec("sharded", {"m": 70, "n": 392, "k": 160, "l": 2, "alpha": 0.5}, 11)
        inputs = dense.get_inputs(case)
        (full,) = dense.get_reference(inputs)
        part, span = sharding.shard_dense_inputs(inputs, rank, world)
        spans = sharding.row_shards(392, world)
        assert span == spans[rank]
        # The shard is a valid dense problem of its own (shapes and layouts check out).
        (out,) = dense.allocate_outputs(part)
        dense.operands(part, out)
        (local,) = dense.get_reference(part)
        gathered = sharding.all_gather_columns(local, spans)
        ok_dense = torch.equal(gathered, full)

        dual = get_workload("nvfp4_dual_gemm")(None, device="cpu")
        case = CaseSpec("sharded", {"m": 33, "n": 264, "k": 96, "l": 1}, 12)
        inputs = dual.get_inputs(case)
        (full,) = dual.get_reference(inputs)
        part, span = sharding.shard_dual_inputs(inputs, rank, world)
        (local,) = dual.get_reference(part)
        gathered = sharding.all_gather_columns(local, sharding.row_shards(264, world))
        ok_dual = torch.equal(gathered, full)

        group = get_workload("nvfp4_group_gemm")(None, device="cpu")
        case = CaseSpec("sharded", {"groups": [(17, 256, 128), (65, 384, 64)]}, 13)
        inputs = group.get_inputs(case)
        full = group.get_reference(inputs)
        part, spans_g = sharding.shard_group_inputs(inputs, rank, world)
        local = group.get_reference(part)
        ok_group = all(torch.equal(out, full[g][:, start:stop])
                       for out, (g, start, stop) in zip(local, spans_g))
        queue.put((rank, ok_dense, ok_dual, ok_group))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_sharded_gemm_equals_unsharded():
    context = mp.get_context("spawn")
    queue = context.Queue()
    port = free_port()
    procs = [context.Process(target=shard_worker, args=(rank, 2, port, queue)) for rank in range(2)]
    for proc in procs:
        proc.start()
    results = [queue.get(timeout=240) for _ in procs]
    for proc in procs:
        proc.join(timeout=60)
        assert proc.exitcode == 0
    assert sorted(results) == [(0, True, True, True), (1, True, True, True)]
