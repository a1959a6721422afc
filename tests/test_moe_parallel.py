"""Expert-parallel mixture-of-experts forward on two gloo ranks on the CPU: the routing,
the two all-to-all exchanges and the weighted recombination of ``harness.moe.moe_forward_ep``,
with the torch reference standing in for the experts' kernels. Every rank's output must
equal the single-process reference of its own tokens bit for bit (each (token, expert) row
is computed alone, so nothing depends on which rank computes it or in which order). Also
the routing table itself. No GPU."""

import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from harness import moe
from harness.workloads import quantization as q


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def weights(experts, rows, k, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(experts, rows, k, generator=g) * 0.05
    packed, scales = q.quantize_nvfp4(w.permute(1, 2, 0))
    return packed.permute(2, 0, 1).contiguous(), scales.permute(2, 0, 1).contiguous()


def ep_worker(rank: int, world: int, port: int, queue) -> None:
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank,
                            world_size=world)
    try:
        experts, hidden, inter, tokens, choices = 6, 128, 64, 37 + 5 * rank, 2
        w13, s13 = weights(experts, 2 * inter, hidden, 1)
        w2, s2 = weights(experts, hidden, inter, 2)
        g = torch.Generator().manual_seed(100 + rank)      # every rank has its own tokens
        x = torch.randn(tokens, hidden, generator=g)
        scores = torch.rand(tokens, experts, generator=g)
        scores[:, 4] = -1.0                                 # an expert nobody routes to
        topk_weights, topk_ids = torch.topk(scores, choices, dim=1)
        per_rank = -(-experts // world)
        first = rank * per_rank

        def local_experts(rows, local_ids):
            out = torch.zeros_like(rows)
            for e in range(per_rank):
                picked = torch.nonzero(local_ids == e, as_tuple=True)[0]
                if picked.numel():
                    # One row at a time: identical to the reference whatever the batch.
                    for i in picked.tolist():
                        out[i] = moe.expert_reference(rows[i:i + 1], w13[first + e], s13[first + e],
                                                      w2[first + e], s2[first + e]).float()
            return out

        got = moe.moe_forward_ep(x, topk_ids, topk_weights, experts, local_experts)
        want = torch.zeros_like(got)
        for t in range(tokens):
            for j in range(choices):
                e = int(topk_ids[t, j])
                y = moe.expert_reference(x[t:t + 1], w13[e], s13[e], w2[e], s2[e]).float()
                want[t] += y[0] * topk_weights[t, j]
        owners = moe.expert_owner(torch.arange(experts), experts, world).tolist()
        queue.put((rank, torch.allclose(got, want, rtol=0, atol=1e-6), bool(got.abs().sum() > 0),
                   owners))
    finally:
        dist.destroy_process_group()


def test_two_rank_expert_parallel_forward_equals_reference():
    context = mp.get_context("spawn")
    queue = context.Queue()
    port = free_port()
    procs = [context.Process(target=ep_worker, args=(rank, 2, port, queue)) for rank in range(2)]
    for proc in procs:
        proc.start()
    results = [queue.get(timeout=240) for _ in procs]
    for proc in procs:
        proc.join(timeout=60)
        assert proc.exitcode == 0
    owners = [0, 0, 0, 1, 1, 1]
    assert sorted(results) == [(0, True, True, owners), (1, True, True, owners)]


def test_route_rows_orders_pairs_by_expert_in_padded_blocks():
    ids = torch.tensor([[0, 2], [2, 1], [2, 0], [0, 2]])
    source, counts, starts = moe.route_rows(ids, 4)
    assert counts == [3, 1, 4, 0] and starts == [0, 128, 256, 384]
    assert source.numel() == 384
    assert source[:3].tolist() == [0, 5, 6] and source[128].item() == 3
    assert source[256:260].tolist() == [1, 2, 4, 7] and (source[3:128] == -1).all()
    # An expert with exactly one block of rows, and the last expert non-empty.
    ids = torch.cat([torch.zeros(128, dtype=torch.long), torch.ones(3, dtype=torch.long)])[:, None]
    source, counts, starts = moe.route_rows(ids, 2)
    assert counts == [128, 3] and starts == [0, 128] and source.numel() == 256
    assert source[:128].tolist() == list(range(128)) and source[128:131].tolist() == [128, 129, 130]
