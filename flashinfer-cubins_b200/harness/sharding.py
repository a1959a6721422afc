"""Multi-GPU decomposition of the NVFP4 GEMMs: one process per GPU, no collective on
the data path.

The reference is single-device (no collective call site anywhere in it), so this layer
is new. The path shards by independent units:

* dense and dual GEMM: rank r keeps rows ``[start_r, stop_r)`` of B (columns of D) and
  the matching scale atoms; A, SFA and alpha are replicated (small). Boundaries are
  multiples of 128 rows so that the blocked scale layout, which stores 128-row atoms
  row-block-major, splits on whole atoms and a shard is a plain slice of the original
  tensors. Each rank writes its own ``[m, n_r, l]`` output;
* grouped GEMM: either whole groups placed by longest-processing-time on FLOPs
  (``balance_groups``) or, when one group dominates, every group's B cut along N the
  same way as the dense rule (``slice_groups``), which balances FLOPs and B bytes.

``all_gather_columns`` is the one optional exchange: it reassembles the full D on every
rank with ``torch.distributed.all_gather`` (NCCL over NVLink on GPUs, gloo on CPU) when
a caller needs it.
"""

from __future__ import annotations

from collections.abc import Sequence

import torch
import torch.distributed as dist

ATOM_ROWS = 128


def row_shards(n: int, world: int, multiple: int = ATOM_ROWS) -> list[tuple[int, int]]:
    """``world`` contiguous row ranges covering ``[0, n)`` whose inner boundaries are
    multiples of ``multiple``, as even as that allows; trailing ranks may be empty when
    ``n`` has fewer than ``world`` blocks."""
    if n < 1 or world < 1:
        raise ValueError("n and world must be positive")
    blocks = -(-n // multiple)
    bounds = [min(n, (blocks * rank // world) * multiple) for rank in range(world)] + [n]
    return [(bounds[rank], bounds[rank + 1]) for rank in range(world)]


def shard_dense_inputs(inputs: tuple, rank: int, world: int) -> tuple[tuple, tuple[int, int]]:
    """Rank ``rank``'s operands of a dense launch ``(a, b, sfa, sfb, alpha)`` with the
    scales in the blocked 6-D view, and its column range of D. B and SFB are sliced
    (no copy beyond making B's slice contiguous in storage order)."""
    a, b, sfa, sfb, alpha = inputs
    start, stop = row_shards(b.shape[0], world)[rank]
    if stop <= start:
        raise ValueError(f"rank {rank} of {world} has no rows of n={b.shape[0]}")
    b_part = b[start:stop].permute(2, 0, 1).contiguous().permute(1, 2, 0)
    first, last = start // ATOM_ROWS, -(-stop // ATOM_ROWS)
    sfb_part = (sfb[:, :, first:last].permute(5, 2, 4, 0, 1, 3).contiguous()
                .permute(3, 4, 1, 5, 2, 0))
    return (a, b_part, sfa, sfb_part, alpha), (start, stop)


def shard_dual_inputs(inputs: tuple, rank: int, world: int) -> tuple[tuple, tuple[int, int]]:
    """As ``shard_dense_inputs`` for ``(a, b1, b2, sfa, sfb1, sfb2, alpha)``: B1 and B2
    are cut identically, so the fused gate stays local to the rank."""
    a, b1, b2, sfa, sfb1, sfb2, alpha = inputs
    (_, b1_part, _, s1_part, _), span = shard_dense_inputs((a, b1, sfa, sfb1, alpha), rank, world)
    (_, b2_part, _, s2_part, _), _ = shard_dense_inputs((a, b2, sfa, sfb2, alpha), rank, world)
    return (a, b1_part, b2_part, sfa, s1_part, s2_part, alpha), span


def group_flops(problem: Sequence[int]) -> int:
    m, n, k = problem
    return 2 * m * n * k


def balance_groups(problems: Sequence[Sequence[int]], world: int) -> list[list[int]]:
    """Whole groups to ranks, longest processing time first on FLOPs: returns the group
    indices of every rank (in ascending order)."""
    loads = [0] * world
    owned: list[list[int]] = [[] for _ in range(world)]
    for index in sorted(range(len(problems)), key=lambda i: (-group_flops(problems[i]), i)):
        rank = min(range(world), key=lambda r: (loads[r], r))
        owned[rank].append(index)
        loads[rank] += group_flops(problems[index])
    return [sorted(indices) for indices in owned]


def balance_speedup(problems: Sequence[Sequence[int]], world: int) -> float:
    """Total FLOPs over the most loaded rank's FLOPs under ``balance_groups``."""
    owned = balance_groups(problems, world)
    total = sum(group_flops(p) for p in problems)
    worst = max(sum(group_flops(problems[i]) for i in indices) for indices in owned)
    return total / worst


def slice_groups(problems: Sequence[Sequence[int]], rank: int, world: int):
    """Every group's B cut along N with ``row_shards``: a list of
    ``(group, start, stop)`` for ``rank`` (groups narrower than ``world`` atoms leave
    some ranks without a slice of them)."""
    units = []
    for index, (_, n, _) in enumerate(problems):
        start, stop = row_shards(n, world)[rank]
        if stop > start:
            units.append((index, start, stop))
    return units


def shard_group_inputs(inputs: tuple, rank: int, world: int):
    """Rank ``rank``'s operands of a grouped launch under ``slice_groups`` and, per kept
    group, ``(group, start, stop)``."""
    groups = [tuple(inputs[i:i + 4]) for i in range(0, len(inputs), 4)]
    problems = [(a.shape[0], b.shape[0], 2 * a.shape[1]) for a, b, _, _ in groups]
    tensors, spans = [], []
    for index, start, stop in slice_groups(problems, rank, world):
        a, b, sfa, sfb = groups[index]
        first, last = start // ATOM_ROWS, -(-stop // ATOM_ROWS)
        tensors += [a, b[start:stop].contiguous(), sfa, sfb[first:last].contiguous()]
        spans.append((index, start, stop))
    return tuple(tensors), spans


def all_gather_columns(local: torch.Tensor, spans: Sequence[tuple[int, int]],
                       group=None) -> torch.Tensor:
    """Full ``[m, n, l]`` D on every rank from each rank's ``[m, n_r, l]`` piece
    (batch-major storage). ``spans`` are all ranks' column ranges. Pieces are padded to
    the widest shard for the collective, then cut back."""
    world = dist.get_world_size(group)
    m, _, batches = local.shape
    widest = max(stop - start for start, stop in spans)
    send = torch.zeros((batches, m, widest), dtype=local.dtype, device=local.device)
    send[:, :, : local.shape[1]] = local.permute(2, 0, 1)
    pieces = [torch.empty_like(send) for _ in range(world)]
    dist.all_gather(pieces, send, group=group)
    total = spans[-1][1]
    full = torch.empty((batches, m, total), dtype=local.dtype, device=local.device)
    for (start, stop), piece in zip(spans, pieces):
        full[:, :, start:stop] = piece[:, :, : stop - start]
    return full.permute(1, 2, 0)
