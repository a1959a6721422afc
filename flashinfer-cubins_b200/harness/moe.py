"""A mixture-of-experts feed-forward layer on the NVFP4 kernels of this package, on one GPU
or expert-parallel over several.

    tokens -> route -> quantise into rows permuted by expert (one gathering launch)
           -> grouped gate/up dual GEMM, gated and re-quantised in its epilogue   (one launch)
           -> grouped down GEMM                                                  (one launch)
           -> weighted un-permutation

The reference sizes its grouped cases as expert-parallel shards of such a layer
(``harness/workloads/nvfp4_group_gemm.py:751-785`` there, ``MOE_PLAN``) but has no NVFP4 MoE
layer itself (its FP8 one is ``harness/workloads/moe.py:1-33``); this module is the step
around the grouped GEMM that a user of that path builds next. ``moe_reference`` is the same
computation with the harness's torch quantiser and GEMM reference, stage by stage.

Layout choices that keep every stage a plain kernel launch on whole buffers:

* Permuted rows are grouped by expert and every expert's block is padded to a multiple of
  128 rows (padding rows are zero). A block then starts on a scale-atom row, so ONE quantiser
  launch over the whole permuted buffer produces packed rows and blocked scales that each
  group addresses by offset, and the gate/up kernel's NVFP4 output (packed rows + blocked
  scales) is addressed by the down projection the same way, with no relayout in between.
* Weights arrive quantised: ``w13`` packed ``[E, 2I, H/2]`` (gate rows then up rows) with
  blocked scales ``[E, 2I/128, ceil(H/64), 32, 4, 4]``; ``w2`` packed ``[E, H, I/2]``
  with ``[E, ceil(H/128), ceil(I/64), 32, 4, 4]``. With ``fused=True`` the intermediate size
  must be a multiple of 128 (the up projection's scales then start on an atom row).
* ``MoELayer`` keeps plans, workspaces and the buffers between the stages per tuple of expert
  row counts and binds them once: a forward with a routing pattern seen before is one
  quantiser launch and two grouped GEMM launches, with nothing allocated, encoded or bound.
  It reads the row counts back (the plans' shapes are the host's).
* ``RoutedMoELayer`` reads nothing back: its two plans take the experts' row counts from the
  device (``nvfp4_moe_plan_create`` and friends), all experts share buffers sized for the
  worst case, and one plan pair serves every routing, so a forward is a fixed sequence of
  launches that a CUDA graph can hold. Both layers give the same bits.

Expert parallelism (``moe_forward_ep``): rank r owns experts ``[r E/W, (r+1) E/W)``. Every
rank routes its own tokens, sends each (token, choice) row to the owner of its expert with
one all-to-all, runs the layer above on what it received with its local experts, and sends
the results back with a second all-to-all; the weighted sum happens where the token lives.
``torch.distributed`` does the exchange (NCCL on GPUs, gloo on CPU for the host-logic test).
"""

from __future__ import annotations

from collections import OrderedDict
from collections.abc import Callable

import torch

from . import native
from .workloads import quantization as q

ROW_BLOCK = 128
MAX_PATTERNS = 8  # routing patterns a layer keeps plans and buffers for


class Routing:
    """Where every (token, choice) pair goes when the pairs are ordered by expert and every
    expert's block is padded to whole 128-row blocks: ``source`` (for every padded permuted
    row the flat pair index ``token * K + choice``, or -1 for padding), ``row_of_pair`` (the
    inverse: the permuted row of every pair), the row count per expert and each expert's
    first padded row."""

    __slots__ = ("source", "row_of_pair", "counts", "starts")

    def __init__(self, source, row_of_pair, counts, starts):
        self.source, self.row_of_pair, self.counts, self.starts = source, row_of_pair, counts, starts


def route(topk_ids: torch.Tensor, experts: int) -> Routing:
    """Order the (token, choice) pairs by expert. One host read (the counts: the plans' shapes
    depend on them); everything else stays on the device, without masked indexing."""
    flat = topk_ids.reshape(-1)
    device = flat.device
    order = torch.argsort(flat, stable=True)
    counts_t = torch.bincount(flat, minlength=experts)
    counts = counts_t.tolist()
    starts, total = [], 0
    for count in counts:
        starts.append(total)
        total += -(-count // ROW_BLOCK) * ROW_BLOCK
    source = torch.full((max(total, ROW_BLOCK),), -1, dtype=torch.int64, device=device)
    row_of_pair = torch.empty_like(order)
    if flat.numel():
        # Pair i of the sorted order belongs to expert flat[order[i]] and is that expert's
        # (i - first sorted position of the expert)-th row.
        starts_t = torch.tensor(starts, dtype=torch.int64, device=device)
        first = torch.cumsum(counts_t, 0) - counts_t
        sorted_expert = flat[order]
        rows = (starts_t - first)[sorted_expert] + torch.arange(flat.numel(), device=device)
        source[rows] = order
        row_of_pair[order] = rows
    return Routing(source, row_of_pair, counts, starts)


class DeviceRouting:
    """``route`` by the library's two routing kernels (``nvfp4_moe_count`` /
    ``nvfp4_moe_place``) for ids on a GPU: ``token_of_row`` (int32, the token of every padded
    permuted row, -1 for padding; what ``MoELayer.forward_gathered`` takes), ``row_of_pair``
    (int32), the row count per expert and each expert's first padded row. Two launches and
    one host read instead of a sort and a dozen indexing kernels; which pair gets which row
    inside an expert's block is not fixed from run to run (the layer's result is)."""

    __slots__ = ("token_of_row", "row_of_pair", "counts", "starts", "_scratch")

    def __init__(self, topk_ids: torch.Tensor, experts: int):
        ids = topk_ids.contiguous()
        if ids.dtype not in (torch.int32, torch.int64):
            ids = ids.to(torch.int64)
        device = ids.device
        pairs, choices = ids.numel(), ids.shape[1]
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            scratch = torch.empty((2, experts), dtype=torch.int32, device=device)
            native.moe_count(ids.data_ptr(), ids.dtype == torch.int64, pairs, experts,
                             scratch[0].data_ptr(), stream)
            self.counts = scratch[0].tolist()
            self.starts, total = [], 0
            for count in self.counts:
                self.starts.append(total)
                total += -(-count // ROW_BLOCK) * ROW_BLOCK
            rows = max(total, ROW_BLOCK)
            self.row_of_pair = torch.empty((pairs,), dtype=torch.int32, device=device)
            self.token_of_row = torch.empty((rows,), dtype=torch.int32, device=device)
            native.moe_place(ids.data_ptr(), ids.dtype == torch.int64, pairs, choices, self.starts,
                             rows, scratch[1].data_ptr(), self.row_of_pair.data_ptr(),
                             self.token_of_row.data_ptr(), stream)
            self._scratch = scratch  # until the launches have run


def route_rows(topk_ids: torch.Tensor, experts: int) -> tuple[torch.Tensor, list[int], list[int]]:
    """``route`` as the tuple ``(source, counts, starts)``."""
    routing = route(topk_ids, experts)
    return routing.source, routing.counts, routing.starts


def _gather(x: torch.Tensor, source: torch.Tensor, choices: int) -> torch.Tensor:
    rows = torch.zeros((source.numel(), x.shape[1]), dtype=torch.float32, device=x.device)
    valid = source >= 0
    rows[valid] = x.float()[source[valid] // choices]
    return rows


def _combine(y: torch.Tensor, row_of_pair: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """``out[t] = sum_j weights[t, j] * y[row of pair (t, j)]`` in FP32, no atomics: on a GPU
    the library's combine kernel (every row of ``y`` read once), elsewhere one gather and one
    batched product."""
    tokens, choices = weights.shape
    hidden = y.shape[1]
    if y.is_cuda and y.dtype == torch.float16 and hidden % 8 == 0 and y.is_contiguous():
        rows = row_of_pair.to(torch.int32).contiguous()
        w = weights.float().contiguous()
        out = torch.empty((tokens, hidden), dtype=torch.float32, device=y.device)
        with torch.cuda.device(y.device):
            native.moe_combine(y.data_ptr(), rows.data_ptr(), w.data_ptr(), out.data_ptr(), tokens,
                               choices, hidden, torch.cuda.current_stream(y.device).cuda_stream)
        return out
    picked = y.index_select(0, row_of_pair).view(tokens, choices, hidden)
    return torch.bmm(weights.float().unsqueeze(1), picked.float()).squeeze(1)


class _Pattern:
    """What one routing pattern (row count per expert) of a layer needs on one stream: the
    two grouped plans with their workspaces, and the buffers between the stages, allocated
    once and bound to the plans once. Every expert's block starts on a 128-row boundary, so
    the buffers are whole tensors that each group addresses by offset:

    * ``a1`` / ``s1``: the quantised rows (packed ``[R, H/2]``, blocked scales), written by
      the quantiser for the rows that hold data only (``block_rows``);
    * ``a2`` / ``s2``: the gated intermediate in NVFP4 (written by the fused gate/up kernel,
      or by the quantiser after ``h`` FP16 ``[R, 2I]`` when not fused). The kernels write
      only rows that exist, so padding rows and their scales stay zero;
    * ``y``: FP16 ``[R, H]``, padding rows zero."""

    def __init__(self, layer: MoELayer, counts: tuple[int, ...], stream: int):
        device, hidden, inter = layer.device, layer.hidden, layer.inter
        live = [e for e, count in enumerate(counts) if count > 0]
        self.starts, total = [], 0
        for count in counts:
            self.starts.append(total)
            total += -(-count // ROW_BLOCK) * ROW_BLOCK
        self.total = total
        starts = self.starts
        index = device.index or 0
        if layer.fused:
            self.up_plan = native.Plan.grouped_dual_fp4(
                index, [(counts[e], inter, hidden) for e in live])
        else:
            self.up_plan = native.Plan.grouped(
                index, [(counts[e], 2 * inter, hidden) for e in live])
        self.down_plan = native.Plan.grouped(index, [(counts[e], hidden, inter) for e in live])
        self.up_ws, self.down_ws = (
            torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8, device=device)
            for plan in (self.up_plan, self.down_plan))
        self.up_plan.init_workspace(self.up_ws.data_ptr(), stream)
        self.down_plan.init_workspace(self.down_ws.data_ptr(), stream)

        atoms_h, atoms_i = -(-hidden // 64), -(-inter // 64)
        blocks = total // ROW_BLOCK
        byte = dict(dtype=torch.uint8, device=device)
        self.a1 = torch.zeros((total, hidden // 2), **byte)
        self.s1 = torch.zeros((blocks, atoms_h, 32, 4, 4), **byte)
        self.a2 = torch.zeros((total, inter // 2), **byte)
        self.s2 = torch.zeros((blocks, atoms_i, 32, 4, 4), **byte)
        self.y = torch.zeros((total, hidden), dtype=torch.float16, device=device)
        self.h = None
        # Rows that hold data in every 128-row block, for the quantiser: padding rows are
        # zero in these buffers from the start and are never read or written again.
        filled = []
        for count in counts:
            blocks_of = -(-count // ROW_BLOCK)
            filled += [min(ROW_BLOCK, count - ROW_BLOCK * b) for b in range(blocks_of)]
        self.block_rows = torch.tensor(filled, dtype=torch.int32, device=device)
        a_ptrs = [self.a1.data_ptr() + starts[e] * (hidden // 2) for e in live]
        sa_ptrs = [self.s1.data_ptr() + (starts[e] // ROW_BLOCK) * atoms_h * 512 for e in live]
        a2_ptrs = [self.a2.data_ptr() + starts[e] * (inter // 2) for e in live]
        s2_ptrs = [self.s2.data_ptr() + (starts[e] // ROW_BLOCK) * atoms_i * 512 for e in live]
        w13, w13_scales = layer.w13, layer.w13_scales
        if layer.fused:
            # Gate/up straight to the down projection's A operand.
            self.up_plan.bind_dual_groups_fp4(
                a_ptrs,
                [w13[e].data_ptr() for e in live],
                [w13[e].data_ptr() + inter * (hidden // 2) for e in live],
                sa_ptrs,
                [w13_scales[e].data_ptr() for e in live],
                [w13_scales[e].data_ptr() + (inter // ROW_BLOCK) * atoms_h * 512 for e in live],
                a2_ptrs, s2_ptrs, self.up_ws.data_ptr(), stream)
        else:
            self.h = torch.zeros((total, 2 * inter), dtype=torch.float16, device=device)
            self.up_plan.bind_groups(
                a_ptrs, [w13[e].data_ptr() for e in live], sa_ptrs,
                [w13_scales[e].data_ptr() for e in live],
                [self.h.data_ptr() + starts[e] * 2 * inter * 2 for e in live],
                self.up_ws.data_ptr(), stream)
        self.down_plan.bind_groups(
            a2_ptrs, [layer.w2[e].data_ptr() for e in live], s2_ptrs,
            [layer.w2_scales[e].data_ptr() for e in live],
            [self.y.data_ptr() + starts[e] * hidden * 2 for e in live],
            self.down_ws.data_ptr(), stream)

    def destroy(self) -> None:
        self.up_plan.destroy()
        self.down_plan.destroy()


class MoELayer:
    """The experts of one layer on one GPU with their cached plans.

    ``w13`` ``[E, 2I, H/2]``, ``w13_scales`` blocked, ``w2`` ``[E, H, I/2]``, ``w2_scales``
    blocked (see the module docstring). ``fused=True`` (default when I is a multiple of
    128) runs the gate/up projection as the grouped dual GEMM with NVFP4 output;
    ``fused=False`` runs one grouped GEMM over both halves of ``w13``, the gate in torch
    and a second quantiser launch."""

    def __init__(self, w13, w13_scales, w2, w2_scales, fused: bool | None = None):
        experts, two_i, half_h = w13.shape
        self.experts, self.hidden, self.inter = experts, 2 * half_h, two_i // 2
        if tuple(w2.shape) != (experts, self.hidden, self.inter // 2):
            raise ValueError("w2 does not match w13")
        if self.hidden % 64 or self.inter % 64:
            raise ValueError("hidden and intermediate sizes must be multiples of 64")
        self.fused = self.inter % ROW_BLOCK == 0 if fused is None else fused
        if self.fused and self.inter % ROW_BLOCK:
            raise ValueError("the fused gate/up kernel needs an intermediate size that is a "
                             "multiple of 128")
        self.w13, self.w13_scales, self.w2, self.w2_scales = w13, w13_scales, w2, w2_scales
        self.device = w13.device
        if self.device.type != "cuda" or not native.device_supported(self.device.index or 0):
            raise RuntimeError(f"sm_100a code cannot run on {self.device}")
        self._plans: OrderedDict[tuple, _Pattern] = OrderedDict()

    def close(self) -> None:
        if self._plans:
            torch.cuda.synchronize(self.device)
        for pattern in self._plans.values():
            pattern.destroy()
        self._plans.clear()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _entry(self, counts: tuple[int, ...], stream: int) -> _Pattern:
        """Plans, workspaces and buffers of this routing pattern on this stream: created and
        bound at the pattern's first forward, least recently used dropped beyond
        ``MAX_PATTERNS``."""
        key = (counts, stream)
        pattern = self._plans.get(key)
        if pattern is not None:
            self._plans.move_to_end(key)
            return pattern
        while len(self._plans) >= MAX_PATTERNS:
            _, oldest = self._plans.popitem(last=False)
            torch.cuda.synchronize(self.device)
            oldest.destroy()
        pattern = _Pattern(self, counts, stream)
        self._plans[key] = pattern
        return pattern

    def _run(self, counts: list[int], starts: list[int], total: int,
             quantise: Callable[[_Pattern, int], None]) -> torch.Tensor:
        """One forward on the pattern of ``counts``: ``quantise(pattern, stream)`` fills the
        pattern's ``a1`` / ``s1``; then the two grouped launches. Returns the pattern's ``y``."""
        hidden, inter = self.hidden, self.inter
        if not any(count > 0 for count in counts):
            return torch.zeros((total, hidden), dtype=torch.float16, device=self.device)
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            pattern = self._entry(tuple(counts), stream)
            if list(starts) != pattern.starts or total != pattern.total:
                raise ValueError("rows are not laid out in 128-row blocks per expert")
            quantise(pattern, stream)
            pattern.up_plan.launch_groups(pattern.up_ws.data_ptr(), stream)
            if not self.fused:
                h = pattern.h
                act = torch.nn.functional.silu(h[:, :inter].float()) * h[:, inter:].float()
                native.quantize_blocks(act.data_ptr(), native.IN_F32, pattern.a2.data_ptr(),
                                       pattern.s2.data_ptr(), pattern.total, inter,
                                       pattern.block_rows.data_ptr(), stream)
            pattern.down_plan.launch_groups(pattern.down_ws.data_ptr(), stream)
        return pattern.y

    def forward_rows(self, rows: torch.Tensor, counts: list[int], starts: list[int]) -> torch.Tensor:
        """The experts applied to permuted rows: ``rows`` FP32 ``[R, H]`` grouped by expert
        (expert e at ``starts[e]``, ``counts[e]`` rows, blocks padded to 128 rows). Returns
        FP16 ``[R, H]`` (padding rows zero): the pattern's own output buffer, which the next
        forward with the same row counts on the same stream overwrites.

        A pattern seen before costs one quantiser launch and two grouped GEMM launches:
        nothing is allocated, encoded or bound."""
        if rows.dim() != 2 or rows.shape[1] != self.hidden:
            raise ValueError("rows do not match the weights")
        if rows.dtype != torch.float32 or not rows.is_contiguous():
            rows = rows.float().contiguous()

        def quantise(pattern: _Pattern, stream: int) -> None:
            native.quantize_blocks(rows.data_ptr(), native.IN_F32, pattern.a1.data_ptr(),
                                   pattern.s1.data_ptr(), pattern.total, self.hidden,
                                   pattern.block_rows.data_ptr(), stream)

        return self._run(counts, starts, rows.shape[0], quantise)

    def forward_gathered(self, x: torch.Tensor, source_rows: torch.Tensor, counts: list[int],
                         starts: list[int]) -> torch.Tensor:
        """``forward_rows`` without the permuted copy: permuted row r is row
        ``source_rows[r]`` of ``x`` (``[T, H]`` FP32 or BF16, contiguous), or padding where
        ``source_rows[r] < 0`` (int32 ``[R]`` on the device). The quantiser reads the token
        rows where they are."""
        if x.dim() != 2 or x.shape[1] != self.hidden:
            raise ValueError("activations do not match the weights")
        if x.dtype not in (torch.float32, torch.bfloat16) or not x.is_contiguous():
            x = x.float().contiguous()
        kind = native.IN_F32 if x.dtype == torch.float32 else native.IN_BF16
        if source_rows.dtype != torch.int32 or not source_rows.is_contiguous():
            source_rows = source_rows.to(torch.int32).contiguous()

        def quantise(pattern: _Pattern, stream: int) -> None:
            native.quantize_gather(x.data_ptr(), kind, pattern.a1.data_ptr(),
                                   pattern.s1.data_ptr(), pattern.total, self.hidden,
                                   source_rows.data_ptr(), stream)

        return self._run(counts, starts, source_rows.numel(), quantise)

    def check_status(self) -> None:
        """Synchronise and raise ``native.NativeError`` if a kernel abandoned a wait."""
        for (_, stream), pattern in self._plans.items():
            pattern.up_plan.status(pattern.up_ws.data_ptr(), stream)
            pattern.down_plan.status(pattern.down_ws.data_ptr(), stream)

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        """``out[t] = sum_j weight[t, j] * down_e(silu(gate_e(x_t)) * up_e(x_t))`` with
        ``e = topk_ids[t, j]``; ``x`` ``[T, H]`` FP32/BF16, result FP32 ``[T, H]``."""
        if x.shape[1] != self.hidden:
            raise ValueError("activations do not match the weights")
        routing = DeviceRouting(topk_ids, self.experts)
        y = self.forward_gathered(x, routing.token_of_row, routing.counts, routing.starts)
        return _combine(y, routing.row_of_pair, topk_weights)


class RoutedMoELayer:
    """The same layer with nothing read back from the device: one pair of plans
    (``nvfp4_moe_plan_create``) and one set of buffers serve every routing of up to
    ``max_pairs`` (token, choice) pairs. A forward is nine launches (count, two layouts, place,
    gather-quantise, gate/up, down, combine) whose shapes do not depend on the routing, so it
    can be captured in a CUDA graph once and replayed on new tokens and new expert choices.

    The experts' blocks share buffers of ``max_pairs + 127 * E`` rows (rounded up to 128): the
    most rows any routing can need when every expert's block is padded to whole 128-row
    blocks. Weights as for ``MoELayer``; the intermediate size must be a multiple of 128."""

    def __init__(self, w13, w13_scales, w2, w2_scales, max_pairs: int):
        experts, two_i, half_h = w13.shape
        self.experts, self.hidden, self.inter = experts, 2 * half_h, two_i // 2
        hidden, inter = self.hidden, self.inter
        if tuple(w2.shape) != (experts, hidden, inter // 2):
            raise ValueError("w2 does not match w13")
        if hidden % 64 or inter % ROW_BLOCK or max_pairs < 1:
            raise ValueError("hidden must be a multiple of 64, the intermediate size of 128")
        self.device = device = w13.device
        if device.type != "cuda" or not native.device_supported(device.index or 0):
            raise RuntimeError(f"sm_100a code cannot run on {device}")
        self.max_pairs = max_pairs
        self.capacity = capacity = -(-(max_pairs + (ROW_BLOCK - 1) * experts) // ROW_BLOCK) * ROW_BLOCK
        self.w13, self.w13_scales, self.w2, self.w2_scales = w13, w13_scales, w2, w2_scales
        index = device.index or 0
        atoms_h, atoms_i = -(-hidden // 64), -(-inter // 64)
        byte = dict(dtype=torch.uint8, device=device)
        word = dict(dtype=torch.int32, device=device)
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            self.up_plan = native.Plan.routed(index, native.OUT_FP4, experts, inter, hidden, capacity)
            self.down_plan = native.Plan.routed(index, native.OUT_F16, experts, hidden, inter, capacity)
            self.up_ws, self.down_ws = (
                torch.zeros(max(plan.workspace_bytes(), 256), **byte)
                for plan in (self.up_plan, self.down_plan))
            self.a1 = torch.zeros((capacity, hidden // 2), **byte)
            self.s1 = torch.zeros((capacity // ROW_BLOCK, atoms_h, 32, 4, 4), **byte)
            self.a2 = torch.zeros((capacity, inter // 2), **byte)
            self.s2 = torch.zeros((capacity // ROW_BLOCK, atoms_i, 32, 4, 4), **byte)
            self.y = torch.zeros((capacity, hidden), dtype=torch.float16, device=device)
            self.counts = torch.zeros((experts,), **word)
            self.cursors = torch.zeros((experts,), **word)
            self.token_of_row = torch.full((capacity,), -1, **word)
            self.row_of_pair = torch.zeros((max_pairs,), **word)
            self.up_plan.init_workspace(self.up_ws.data_ptr(), stream)
            self.down_plan.init_workspace(self.down_ws.data_ptr(), stream)
            self.up_plan.bind_routed(
                self.a1.data_ptr(), self.s1.data_ptr(),
                [w13[e].data_ptr() for e in range(experts)],
                [w13_scales[e].data_ptr() for e in range(experts)],
                self.a2.data_ptr(), self.up_ws.data_ptr(), stream,
                b2=[w13[e].data_ptr() + inter * (hidden // 2) for e in range(experts)],
                sfb2=[w13_scales[e].data_ptr() + (inter // ROW_BLOCK) * atoms_h * 512
                      for e in range(experts)],
                d_scales=self.s2.data_ptr())
            self.down_plan.bind_routed(
                self.a2.data_ptr(), self.s2.data_ptr(),
                [w2[e].data_ptr() for e in range(experts)],
                [w2_scales[e].data_ptr() for e in range(experts)],
                self.y.data_ptr(), self.down_ws.data_ptr(), stream)

    def close(self) -> None:
        if self.up_plan is not None:
            torch.cuda.synchronize(self.device)
            self.up_plan.destroy()
            self.down_plan.destroy()
            self.up_plan = self.down_plan = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check_status(self) -> None:
        """Synchronise and raise ``native.NativeError`` if a kernel abandoned a wait."""
        stream = torch.cuda.current_stream(self.device).cuda_stream
        self.up_plan.status(self.up_ws.data_ptr(), stream)
        self.down_plan.status(self.down_ws.data_ptr(), stream)

    def _experts(self, x: torch.Tensor, topk_ids: torch.Tensor) -> None:
        """Everything up to the down projection: afterwards ``self.y[self.row_of_pair[i]]`` is
        the result of pair i."""
        tokens, choices = topk_ids.shape
        pairs = tokens * choices
        if x.shape != (tokens, self.hidden):
            raise ValueError("activations and ids do not match")
        if pairs > self.max_pairs:
            raise ValueError(f"{pairs} pairs; the layer was made for {self.max_pairs}")
        if x.dtype not in (torch.float32, torch.bfloat16) or not x.is_contiguous():
            x = x.float().contiguous()
        ids = topk_ids if topk_ids.dtype in (torch.int32, torch.int64) else topk_ids.long()
        ids = ids.contiguous()
        wide = ids.dtype == torch.int64
        kind = native.IN_F32 if x.dtype == torch.float32 else native.IN_BF16
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            native.moe_count(ids.data_ptr(), wide, pairs, self.experts, self.counts.data_ptr(), stream)
            self.up_plan.layout_routed(self.counts.data_ptr(), self.up_ws.data_ptr(), stream)
            self.down_plan.layout_routed(self.counts.data_ptr(), self.down_ws.data_ptr(), stream)
            self.up_plan.place_routed(ids.data_ptr(), wide, pairs, choices, self.up_ws.data_ptr(),
                                      self.cursors.data_ptr(), self.row_of_pair.data_ptr(),
                                      self.token_of_row.data_ptr(), stream)
            native.quantize_gather(x.data_ptr(), kind, self.a1.data_ptr(), self.s1.data_ptr(),
                                   self.capacity, self.hidden, self.token_of_row.data_ptr(), stream)
            self.up_plan.launch_groups(self.up_ws.data_ptr(), stream)
            self.down_plan.launch_groups(self.down_ws.data_ptr(), stream)

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        """As ``MoELayer.forward`` (``x`` ``[T, H]`` FP32 or BF16, ids int32/int64 ``[T, K]`` in
        ``[0, E)``, weights ``[T, K]``; FP32 ``[T, H]`` out), asynchronous from start to end."""
        tokens, choices = topk_ids.shape
        if topk_weights.shape != topk_ids.shape:
            raise ValueError("ids and weights do not match")
        weights = topk_weights.float().contiguous()
        self._experts(x, topk_ids)
        out = torch.empty((tokens, self.hidden), dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            native.moe_combine(self.y.data_ptr(), self.row_of_pair.data_ptr(), weights.data_ptr(),
                               out.data_ptr(), tokens, choices, self.hidden,
                               torch.cuda.current_stream(self.device).cuda_stream)
        return out

    def apply_rows(self, rows: torch.Tensor, expert_ids: torch.Tensor) -> torch.Tensor:
        """Every row through its one expert (``expert_ids`` ``[R]``): FP16 ``[R, H]`` in the
        order the rows came. What a rank does with the rows an all-to-all delivered
        (``moe_forward_ep``)."""
        if rows.shape[0] == 0:
            return torch.empty((0, self.hidden), dtype=torch.float16, device=self.device)
        self._experts(rows, expert_ids.reshape(-1, 1))
        return self.y.index_select(0, self.row_of_pair[:rows.shape[0]])


def moe_forward(x, topk_ids, topk_weights, w13, w13_scales, w2, w2_scales,
                fused: bool | None = None) -> torch.Tensor:
    """One forward of a throw-away ``MoELayer`` (keep the layer to keep its plans)."""
    if x.device.type != "cuda" or not native.device_supported(x.device.index or 0):
        raise RuntimeError(f"sm_100a code cannot run on {x.device}")
    layer = MoELayer(w13, w13_scales, w2, w2_scales, fused)
    try:
        out = layer.forward(x, topk_ids, topk_weights)
        layer.check_status()
        return out
    finally:
        layer.close()


def expert_reference(rows: torch.Tensor, w13_e, w13_scales_e, w2_e, w2_scales_e,
                     fused: bool = True) -> torch.Tensor:
    """One expert applied to FP32 ``rows`` with the torch quantiser and GEMM reference (any
    device): packed ``w13_e`` ``[2I, H/2]`` / ``w2_e`` ``[H, I/2]`` with logical scales
    ``[rows, k/16]``. ``fused`` follows the fused kernel (the gate is applied to the FP32
    products); otherwise both products are rounded to FP16 first, as the unfused path does.
    Returns FP16 ``[rows, H]``."""
    inter = w13_e.shape[0] // 2
    a1, s1 = q.quantize_nvfp4(rows.float().unsqueeze(0).permute(1, 2, 0))
    h = q.fp4_matmul(a1, w13_e[None].permute(1, 2, 0), s1, w13_scales_e[None].permute(1, 2, 0),
                     out_dtype=torch.float32 if fused else torch.float16)[:, :, 0]
    act = torch.nn.functional.silu(h[:, :inter].float()) * h[:, inter:].float()
    a2, s2 = q.quantize_nvfp4(act.unsqueeze(0).permute(1, 2, 0))
    return q.fp4_matmul(a2, w2_e[None].permute(1, 2, 0), s2, w2_scales_e[None].permute(1, 2, 0),
                        out_dtype=torch.float16)[:, :, 0]


def moe_reference(x, topk_ids, topk_weights, w13, w13_scales, w2, w2_scales,
                  fused: bool = False) -> torch.Tensor:
    """The same layer expert by expert with ``expert_reference`` (any device). Scales are
    the logical ``[E, rows, k/16]`` tensors here."""
    experts, hidden = w13.shape[0], 2 * w13.shape[2]
    tokens, _ = topk_ids.shape
    out = torch.zeros((tokens, hidden), dtype=torch.float32, device=x.device)
    for e in range(experts):
        token, choice = torch.nonzero(topk_ids == e, as_tuple=True)
        if token.numel() == 0:
            continue
        y = expert_reference(x[token], w13[e], w13_scales[e], w2[e], w2_scales[e], fused)
        out.index_add_(0, token, y.float() * topk_weights[token, choice].float()[:, None])
    return out


# -- expert parallelism -------------------------------------------------------------------


def expert_owner(expert: torch.Tensor, experts: int, world: int) -> torch.Tensor:
    """Rank that owns each expert: contiguous blocks of ``ceil(E / W)`` experts."""
    per_rank = -(-experts // world)
    return expert // per_rank


def _group_by(keys: torch.Tensor, groups: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Positions that put equal ``keys`` (in ``[0, groups)``) next to each other, groups in
    order: ``(order, place, counts)`` with ``order[p]`` the item at position p, ``place`` its
    inverse and ``counts`` the items per group (a device tensor). On a GPU the library's
    routing kernels do it in two launches (the order inside a group is then not fixed); on the
    CPU a stable sort."""
    if keys.is_cuda:
        device, items = keys.device, keys.numel()
        keys = keys.contiguous()
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            scratch = torch.empty((2, groups), dtype=torch.int32, device=device)
            wide = keys.dtype == torch.int64
            native.moe_count(keys.data_ptr(), wide, items, groups, scratch[0].data_ptr(), stream)
            counts = scratch[0].tolist()
            firsts, total = [], 0
            for count in counts:
                firsts.append(total)
                total += count
            place = torch.empty((items,), dtype=torch.int32, device=device)
            order = torch.empty((max(items, 1),), dtype=torch.int32, device=device)
            native.moe_place(keys.data_ptr(), wide, items, 1, firsts, items, scratch[1].data_ptr(),
                             place.data_ptr(), order.data_ptr(), stream)
        return order[:items].long(), place.long(), scratch[0].long()
    order = torch.argsort(keys, stable=True)
    place = torch.empty_like(order)
    place[order] = torch.arange(order.numel(), device=order.device)
    return order, place, torch.bincount(keys, minlength=groups)


def moe_forward_ep(x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor,
                   experts: int,
                   local_experts: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
                   group=None) -> torch.Tensor:
    """Expert-parallel forward of this rank's tokens. ``experts`` is the global expert
    count; ``local_experts(rows, local_ids)`` applies this rank's experts to ``rows``
    ``[R, H]`` (in the type of ``x``) whose expert (numbered from 0 within the rank) is
    ``local_ids[R]`` and returns ``[R, H]``, every rank in the same type (on a GPU:
    ``ep_local_experts(layer)`` below, FP16; the CPU test passes the torch reference). Two ``all_to_all_single`` exchanges carry the rows out and back; one
    small one carries the row counts. Returns FP32 ``[T, H]``."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    tokens, choices = topk_ids.shape
    hidden = x.shape[1]
    per_rank = -(-experts // world)
    flat = topk_ids.reshape(-1)
    owner = expert_owner(flat, experts, world)
    # Pairs grouped by destination rank: `order` (the pair at every position of the send
    # buffer) and `place` (its inverse).
    order, place, send_counts = _group_by(owner, world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    send_split, recv_split = send_counts.tolist(), recv_counts.tolist()
    # Rows travel in the activations' own type (BF16 activations as BF16) and come back in the
    # experts' output type (FP16 from the GPU kernels).
    send_rows = x[order // choices].contiguous()
    send_ids = (flat[order] % per_rank).contiguous()
    recv_rows = torch.empty((sum(recv_split), hidden), dtype=send_rows.dtype, device=x.device)
    recv_ids = torch.empty((sum(recv_split),), dtype=send_ids.dtype, device=x.device)
    dist.all_to_all_single(recv_rows, send_rows, recv_split, send_split, group=group)
    dist.all_to_all_single(recv_ids, send_ids, recv_split, send_split, group=group)
    done = local_experts(recv_rows, recv_ids)
    if done.device.type == "cpu":
        done = done.float()   # gloo has no half-precision all-to-all
    done = done.contiguous()
    back = torch.empty((sum(send_split), hidden), dtype=done.dtype, device=x.device)
    dist.all_to_all_single(back, done, send_split, recv_split, group=group)
    # back[i] is the result of pair order[i]: put the pairs back in token order and combine.
    return _combine(back, place, topk_weights)


def ep_local_experts(layer: MoELayer | RoutedMoELayer) -> Callable[[torch.Tensor, torch.Tensor], torch.Tensor]:
    """``local_experts`` for ``moe_forward_ep`` on a GPU: the rank's layer applied to the
    received rows (each row has exactly one expert, weight 1). A ``RoutedMoELayer`` (made for
    as many pairs as can arrive) does it without reading anything back."""
    if isinstance(layer, RoutedMoELayer):
        return layer.apply_rows

    def apply(rows: torch.Tensor, local_ids: torch.Tensor) -> torch.Tensor:
        if rows.shape[0] == 0:
            return torch.empty((0, rows.shape[1]), dtype=torch.float16, device=rows.device)
        routing = DeviceRouting(local_ids[:, None], layer.experts)
        y = layer.forward_gathered(rows, routing.token_of_row, routing.counts, routing.starts)
        return y.index_select(0, routing.row_of_pair)   # FP16, in the order the rows came

    return apply
