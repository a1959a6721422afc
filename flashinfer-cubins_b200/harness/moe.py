"""A mixture-of-experts feed-forward layer on the NVFP4 kernels of this package: token
permutation -> quantise -> grouped gate/up GEMM -> silu gate -> quantise -> grouped down GEMM
-> weighted un-permutation. One GPU; every expert's rows form one group of the two grouped
GEMM launches.

The reference sizes its grouped cases as expert-parallel shards of such a layer
(``harness/workloads/nvfp4_group_gemm.py:751-785`` there, ``MOE_PLAN``) but has no NVFP4 MoE
layer itself (its FP8 one is ``harness/workloads/moe.py:1-33``); this module is the step
around the grouped GEMM that a user of that path builds next. ``moe_reference`` is the same
computation with the harness's torch quantiser and GEMM reference, stage by stage, so the
two agree up to the summation order inside a GEMM.

Layout choices that keep every stage a plain kernel launch on whole buffers:

* Permuted rows are grouped by expert and every expert's block is padded to a multiple of
  128 rows (padding rows are zero). A block then starts on a scale-atom row, so ONE quantiser
  launch over the whole permuted buffer produces packed rows and blocked scales that each
  group addresses by offset, with no per-expert relayout.
* Weights arrive quantised: ``w13`` packed ``[E, 2I, H/2]`` (gate rows then up rows) with
  blocked scales ``[E, ceil(2I/128), ceil(H/64), 32, 4, 4]``; ``w2`` packed ``[E, H, I/2]``
  with ``[E, ceil(H/128), ceil(I/64), 32, 4, 4]``.
"""

from __future__ import annotations

import torch

from . import native
from .workloads import quantization as q

ROW_BLOCK = 128


def route_rows(topk_ids: torch.Tensor, experts: int) -> tuple[torch.Tensor, list[int], list[int]]:
    """Order the (token, choice) pairs by expert. Returns ``source`` (for every padded
    permuted row the flat pair index ``token * K + choice``, or -1 for padding), the row
    count per expert and each expert's first padded row."""
    flat = topk_ids.reshape(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=experts).tolist()
    starts, total = [], 0
    for count in counts:
        starts.append(total)
        total += -(-count // ROW_BLOCK) * ROW_BLOCK
    source = torch.full((max(total, ROW_BLOCK),), -1, dtype=torch.int64, device=topk_ids.device)
    done = 0
    for expert, count in enumerate(counts):
        source[starts[expert]:starts[expert] + count] = order[done:done + count]
        done += count
    return source, counts, starts


def _gather(x: torch.Tensor, source: torch.Tensor, choices: int) -> torch.Tensor:
    rows = torch.zeros((source.numel(), x.shape[1]), dtype=torch.float32, device=x.device)
    valid = source >= 0
    rows[valid] = x.float()[source[valid] // choices]
    return rows


def _scatter(y: torch.Tensor, source: torch.Tensor, weights: torch.Tensor, tokens: int) -> torch.Tensor:
    valid = source >= 0
    pairs = source[valid]
    out = torch.zeros((tokens, y.shape[1]), dtype=torch.float32, device=y.device)
    out.index_add_(0, pairs // weights.shape[1],
                   y[valid].float() * weights.reshape(-1)[pairs].float()[:, None])
    return out


def _grouped_gemm(a_packed, a_scales, w_packed, w_scales, counts, starts, n, k, stream):
    """``D[rows of e] = A[rows of e] @ W[e]^T`` for every expert with rows: one grouped
    launch. ``a_packed`` ``[R, k/2]``, ``a_scales`` blocked ``[R/128, k/64, 32, 4, 4]``."""
    device = a_packed.device
    d = torch.zeros((a_packed.shape[0], n), dtype=torch.float16, device=device)
    live = [e for e, count in enumerate(counts) if count > 0]
    if not live:
        return d
    atoms_k = -(-k // 64)
    plan = native.Plan.grouped(device.index or 0, [(counts[e], n, k) for e in live])
    workspace = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=device)
    plan.init_workspace(workspace.data_ptr(), stream)
    plan.bind_groups(
        [a_packed.data_ptr() + starts[e] * (k // 2) for e in live],
        [w_packed[e].data_ptr() for e in live],
        [a_scales.data_ptr() + (starts[e] // ROW_BLOCK) * atoms_k * 512 for e in live],
        [w_scales[e].data_ptr() for e in live],
        [d.data_ptr() + starts[e] * n * 2 for e in live],
        workspace.data_ptr(), stream)
    plan.launch_groups(workspace.data_ptr(), stream)
    if plan.status(workspace.data_ptr(), stream) != 0:
        raise native.NativeError(native.E_DEVICE_TIMEOUT, "grouped GEMM abandoned a wait")
    plan.destroy()
    return d


def moe_forward(x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor,
                w13: torch.Tensor, w13_scales: torch.Tensor, w2: torch.Tensor,
                w2_scales: torch.Tensor) -> torch.Tensor:
    """``out[t] = sum_j weight[t, j] * down_e(silu(gate_e(x_t)) * up_e(x_t))`` with
    ``e = topk_ids[t, j]``; ``x`` ``[T, H]`` FP32/BF16 on a B200, result FP32 ``[T, H]``."""
    if x.device.type != "cuda" or not native.device_supported(x.device.index or 0):
        raise RuntimeError(f"sm_100a code cannot run on {x.device}")
    experts, two_i, half_h = w13.shape
    hidden, inter = 2 * half_h, two_i // 2
    if x.shape[1] != hidden or tuple(w2.shape) != (experts, hidden, inter // 2):
        raise ValueError("weight shapes do not match the activations")
    if hidden % 64 or inter % 64:
        raise ValueError("hidden and intermediate sizes must be multiples of 64")
    tokens, choices = topk_ids.shape
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream(x.device).cuda_stream
        source, counts, starts = route_rows(topk_ids, experts)
        rows = _gather(x, source, choices)
        a1, s1 = q.quantize_nvfp4_native(rows.unsqueeze(0).permute(1, 2, 0))
        h = _grouped_gemm(a1.permute(2, 0, 1)[0], s1[0], w13, w13_scales, counts, starts,
                          two_i, hidden, stream)
        act = torch.nn.functional.silu(h[:, :inter].float()) * h[:, inter:].float()
        a2, s2 = q.quantize_nvfp4_native(act.unsqueeze(0).permute(1, 2, 0))
        y = _grouped_gemm(a2.permute(2, 0, 1)[0], s2[0], w2, w2_scales, counts, starts,
                          hidden, inter, stream)
        return _scatter(y, source, topk_weights, tokens)


def moe_reference(x, topk_ids, topk_weights, w13, w13_scales, w2, w2_scales) -> torch.Tensor:
    """The same layer with the torch quantiser and the torch GEMM reference, expert by
    expert (any device). Scales are the logical ``[E, rows, k/16]`` tensors here."""
    experts, two_i, half_h = w13.shape
    hidden, inter = 2 * half_h, two_i // 2
    tokens, choices = topk_ids.shape
    out = torch.zeros((tokens, hidden), dtype=torch.float32, device=x.device)
    for e in range(experts):
        token, choice = torch.nonzero(topk_ids == e, as_tuple=True)
        if token.numel() == 0:
            continue
        a1, s1 = q.quantize_nvfp4(x[token].float().unsqueeze(0).permute(1, 2, 0))
        h = q.fp4_matmul(a1, w13[e:e + 1].permute(1, 2, 0), s1, w13_scales[e:e + 1].permute(1, 2, 0),
                         out_dtype=torch.float16)[:, :, 0]
        act = torch.nn.functional.silu(h[:, :inter].float()) * h[:, inter:].float()
        a2, s2 = q.quantize_nvfp4(act.unsqueeze(0).permute(1, 2, 0))
        y = q.fp4_matmul(a2, w2[e:e + 1].permute(1, 2, 0), s2, w2_scales[e:e + 1].permute(1, 2, 0),
                         out_dtype=torch.float16)[:, :, 0]
        out.index_add_(0, token, y.float() * topk_weights[token, choice].float()[:, None])
    return out
