#!/usr/bin/env python
"""Benchmark of the NVFP4 block-scaled GEMM family on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]
                    [--workload square|decode|dual|grouped|latency]
                    [--scaling strong|weak] [--no-configs] [--no-cpu-baseline]

One JSON line on stdout (rank 0). A *step* is one GEMM call on one set of synthetic
operands. The headline workload is the largest single-GPU configuration, the
compute-bound M = N = K = 8192 GEMM with FP16 output; the same line carries, under
``configs``, the other configurations (latency 128x256x512, decode 128x7168x16384, fused
dual GEMM 256x4096x7168, ragged grouped GEMM with eight groups) measured the same way.
Operands are N(0,1) drawn from seeded CPU generators, quantised per 16-element K block to
E2M1 with an E4M3 scale amax/6, scales in the blocked 128x4 layout, alpha = 1; several
operand sets rotate so that together they exceed the 126 MB L2.

* ``validated``: before anything is timed every operand set is run once through the
  prepared launch and compared with the workload's torch reference on the same device
  (dequantise, FP32 matmul, one rounding; rtol = atol = 1e-3); after the timed region one
  output is compared again. A mismatch raises.
* ``value``: whole-job TFLOP/s with operands resident in HBM: K prepared launches replayed
  from a CUDA graph between two CUDA events (back-to-back launches; with programmatic
  dependent launch a kernel's prologue overlaps its predecessor's tail), max over ranks.
  ``isolated_us`` is the median of single launches bracketed by events one at a time, the
  way the reference's own benchmark times a kernel.
* ``e2e``: the same metric through the operator API (``Workload.run``) with host buffers:
  every step copies the operands from pinned host memory, runs the workload and copies D
  back to pinned host memory; the copies of neighbouring steps overlap on separate streams
  (``serial_ms_per_step``: one step at a time).
* ``roofline``: tensor-bound workloads against the nominal dense FP4 peak and the rate at
  which this GPU issues the same MMAs with nothing else running; HBM-bound workloads:
  algorithmic bytes of one call / call duration against the measured HBM copy bandwidth.
* ``cpu_baseline``: the numpy oracle (a port of the reference's torch oracle, pinned to the
  reference's outputs) timed on this host's cores on a bounded sample of the same problem;
  ``torch_path`` inside it is the package's torch restatement of the same arithmetic on all
  cores. A reported baseline, not the target.
* ``competitors``: library NVFP4 GEMMs on the same GPU, same timing method (cuBLASLt
  through ``torch._scaled_mm``, cuDNN and the prebuilt trtllm-gen kernels through FlashInfer
  ``mm_fp4``), for context; the package never imports them.
* ``next_rows``: the rows beside the GEMM path, validated and timed the same way: the
  activation quantiser, the GEMMs whose epilogue writes NVFP4 (dense and gate/up), BF16
  output on weights in the trtllm-gen row order, and one rank's share of a DeepSeek-V3 MoE
  layer on the grouped kernels.
* ``--impl reference``: the reference arm, that CPU path alone on bounded samples.

With N > 1 (launched by torch.distributed.run) the default is strong scaling: the
workload's own N is cut into 128-row shards of B, one per rank, with no collective on the
data path (the grouped GEMM cuts every group's N the same way; ``grouped_lpt`` places
whole groups by FLOPs); every rank validates its own shard; ``all_gather_us`` times the one
optional exchange (all ranks' columns of D gathered over NCCL), outside ``value``.
``--scaling weak`` gives every rank the whole shape instead.
"""

from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO / "flashinfer-cubins_b200"))
sys.path.insert(0, str(REPO))

WORKLOADS = {
    # name: (kind, shape)
    "latency": ("dense", dict(m=128, n=256, k=512)),
    "decode": ("dense", dict(m=128, n=7168, k=16384)),
    "square": ("dense", dict(m=8192, n=8192, k=8192)),
    "dual": ("dual", dict(m=256, n=4096, k=7168)),
    "grouped": ("grouped", dict(ms=(40, 96, 128, 256, 384, 512, 768, 1024), n=4096, k=7168)),
}
BOUND = {"latency": "latency", "decode": "hbm", "square": "tensor", "dual": "hbm",
         "grouped": "hbm"}
# ncu summary that holds the DRAM traffic of one launch of the workload's kernel.
TRAFFIC_SUMMARY = {
    "decode": "nvfp4_gemm_decode_m128_n7168_k16384.md",
    "square": "nvfp4_gemm_square_m8192_n8192_k8192.md",
    "dual": "nvfp4_dual_gemm_m256_n4096_k7168.md",
    "grouped": "nvfp4_group_gemm_8groups_n4096_k7168.md",
}
L2_BYTES = 126 << 20
FALLBACK_HBM_GBS = 6650.0
NOMINAL_FP4_TFLOPS = 9000.0


def algorithmic_work(kind: str, shape: dict) -> tuple[float, float]:
    """(FLOPs, bytes) of one call: 2*M*N*K per GEMM; every operand read once and the
    output written once, logical (unpadded) scale sizes."""
    if kind == "grouped":
        flops = byts = 0.0
        for m in shape["ms"]:
            f, b = algorithmic_work("dense", dict(m=m, n=shape["n"], k=shape["k"]))
            flops, byts = flops + f, byts + b
        return flops, byts
    m, n, k = shape["m"], shape["n"], shape["k"]
    gemms = 2 if kind == "dual" else 1
    flops = 2.0 * m * n * k * gemms
    byts = m * k / 2 + m * k / 16 + gemms * (n * k / 2 + n * k / 16) + 2.0 * m * n
    return flops, byts


def measured_hbm_peak() -> tuple[float, str]:
    path = REPO / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (KeyError, ValueError):
            pass
    return FALLBACK_HBM_GBS, "fallback"


def summary_traffic(file: str):
    """The ``dram_bytes_per_launch:`` line of an ncu summary under ``profiles/``: the sum of
    its byte counts (one per kernel of the step), or None."""
    path = REPO / "profiles" / file
    if not path.is_file():
        return None
    found = re.search(r"dram_bytes_per_launch:([^\n]*)", path.read_text())
    counts = re.findall(r"\b[0-9][0-9_,]{5,}\b", found.group(1)) if found else []
    return sum(int(re.sub(r"[_,]", "", c)) for c in counts) or None


def recorded_traffic(name: str):
    """DRAM bytes of one launch from the workload's ncu summary, or None."""
    file = TRAFFIC_SUMMARY.get(name)
    return summary_traffic(file) if file else None


# -- synthetic operands ---------------------------------------------------------------------


def normal_fp4(rows: int, k: int, seed: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """N(0,1) from a CPU generator -> packed E2M1 (rows, k/2, 1) and logical scales."""
    from harness.workloads import quantization as q

    x = torch.randn(rows, k, generator=torch.Generator().manual_seed(seed))
    packed, scales = q.quantize_nvfp4(x.to(device))
    return packed[..., None], scales[..., None]


def make_operand_set(kind: str, shape: dict, index: int, device) -> tuple:
    """One full (unsharded) operand set: seeds A = 1, B = 2 (dual: B1 = 2, B2 = 3), group g
    A = 10 + g and B = 20 + g, plus 1000 per further set."""
    from harness.workloads.nvfp4_gemm import to_task_scales
    from harness.workloads.nvfp4_group_gemm import to_blocked

    base = 1000 * index
    if kind == "grouped":
        tensors = []
        for g, m in enumerate(shape["ms"]):
            a, sa = normal_fp4(m, shape["k"], base + 10 + g, device)
            b, sb = normal_fp4(shape["n"], shape["k"], base + 20 + g, device)
            tensors += [a[..., 0].contiguous(), b[..., 0].contiguous(),
                        to_blocked(sa[..., 0]), to_blocked(sb[..., 0])]
        return tuple(tensors)
    a, sa = normal_fp4(shape["m"], shape["k"], base + 1, device)
    b, sb = normal_fp4(shape["n"], shape["k"], base + 2, device)
    alpha = torch.ones(1, device=device)
    if kind == "dense":
        return (a, b, to_task_scales(sa), to_task_scales(sb), alpha)
    b2, s2 = normal_fp4(shape["n"], shape["k"], base + 3, device)
    return (a, b, b2, to_task_scales(sa), to_task_scales(sb), to_task_scales(s2), alpha)


def shard_operands(kind: str, inputs: tuple, rank: int, world: int, placement: str):
    """This rank's operands of ``inputs`` and a description of what it owns; ``None`` if
    the rank owns nothing."""
    from harness import sharding

    if world == 1:
        return inputs, "whole problem"
    if kind == "dense":
        local, span = sharding.shard_dense_inputs(inputs, rank, world)
        return local, f"columns {span[0]}:{span[1]}"
    if kind == "dual":
        local, span = sharding.shard_dual_inputs(inputs, rank, world)
        return local, f"columns {span[0]}:{span[1]}"
    if placement == "lpt":
        groups = [tuple(inputs[i:i + 4]) for i in range(0, len(inputs), 4)]
        problems = [(a.shape[0], b.shape[0], 2 * a.shape[1]) for a, b, _, _ in groups]
        owned = sharding.balance_groups(problems, world)[rank]
        if not owned:
            return None, "no group"
        return tuple(t for g in owned for t in groups[g]), f"groups {owned}"
    local, spans = sharding.shard_group_inputs(inputs, rank, world)
    return (local or None), f"{len(spans)} (group, column range) units"


def work_of(kind: str, inputs) -> tuple[float, float]:
    """(FLOPs, algorithmic bytes) of the launch on ``inputs`` (a rank's shard)."""
    if inputs is None:
        return 0.0, 0.0
    if kind == "grouped":
        flops = byts = 0.0
        for i in range(0, len(inputs), 4):
            a, b = inputs[i], inputs[i + 1]
            f, by = algorithmic_work("dense", dict(m=a.shape[0], n=b.shape[0], k=2 * a.shape[1]))
            flops, byts = flops + f, byts + by
        return flops, byts
    a, b = inputs[0], inputs[1]
    return algorithmic_work(kind, dict(m=a.shape[0], n=b.shape[0], k=2 * a.shape[1]))


def workload_class(kind: str):
    from harness import get_workload

    return get_workload({"dense": "nvfp4_gemm", "dual": "nvfp4_dual_gemm",
                         "grouped": "nvfp4_group_gemm"}[kind])


# -- clocks ---------------------------------------------------------------------------------


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) on a
    thread while the measurements run."""

    REASONS = {
        "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
        "hw_power_brake": 0x80, "sw_power_cap": 0x4,
    }

    def __init__(self, index: int, interval: float = 0.002):
        self.samples: list[tuple[float, int, int, int]] = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._interval = interval
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _run(self):
        nvml = self._nvml
        while not self._stop.is_set():
            try:
                mhz = nvml.nvmlDeviceGetClockInfo(self._handle, nvml.NVML_CLOCK_SM)
                util = nvml.nvmlDeviceGetUtilizationRates(self._handle).gpu
                reasons = nvml.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                self.samples.append((time.perf_counter(), mhz, util, reasons))
            except Exception:
                pass
            self._stop.wait(self._interval)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self, since: float = 0.0, until: float = float("inf")) -> dict:
        samples = [s for s in self.samples if since <= s[0] <= until]
        if not samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        # "Under load": samples taken while NVML reported the GPU at least half busy (all
        # samples if none was: the timed regions are shorter than NVML's averaging window).
        loaded = [s[1] for s in samples if s[2] >= 50] or [s[1] for s in samples]
        seen = 0
        for _, _, _, reasons in samples:
            seen |= reasons
        names = [name for name, bit in self.REASONS.items() if seen & bit]
        return {"sm_mhz": statistics.median(loaded), "sm_min_mhz": min(loaded),
                "sm_max_mhz": self.max_mhz, "reasons": names, "samples": len(samples),
                "samples_under_load": len(loaded)}


# -- CPU baseline (the oracle port) ---------------------------------------------------------


def host_dense_operands(m: int, n: int, k: int, seed_a: int = 1, seed_b: int = 2):
    """Storage-order numpy operands (packed bytes, logical scale bytes) of one GEMM, made
    on the CPU with the harness quantiser."""
    a, sa = normal_fp4(m, k, seed_a, "cpu")
    b, sb = normal_fp4(n, k, seed_b, "cpu")

    def store(t):
        t = t.permute(2, 0, 1).contiguous()
        return (t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t).numpy()

    return store(a), store(b), store(sa), store(sb)


def cpu_problem(kind: str, shape: dict) -> tuple[int, int, int, int, str]:
    """(m, n, k, gemms per row sample, description): the GEMM whose rows of B the CPU arm
    samples. The dual GEMM is two GEMMs over the same A (its gate is negligible); the
    grouped GEMM is represented by its largest group (same N and K for every group)."""
    if kind == "grouped":
        m = max(shape["ms"])
        return m, shape["n"], shape["k"], 1, (
            f"largest group m={m} of the grouped GEMM n={shape['n']} k={shape['k']}")
    gemms = 2 if kind == "dual" else 1
    what = "both GEMMs of the dual GEMM" if kind == "dual" else "the GEMM"
    return shape["m"], shape["n"], shape["k"], gemms, (
        f"{what} m={shape['m']} n={shape['n']} k={shape['k']}")


def oracle_rows(operands, rows: slice, gemms: int):
    from oracle import nvfp4_oracle as o

    a, b, sa, sb = operands
    for _ in range(gemms):
        o.gemm(a, b[:, rows], sa, sb[:, rows], 1.0, np.float16)


def rows_within(operands, n: int, gemms: int, seconds: float) -> int:
    """How many rows of B one oracle call can take within ``seconds``: the call costs a fixed
    part (dequantising A) plus a part per row of B, estimated from two probes. All of B
    when the whole problem fits."""
    small, large = min(n, 32), min(n, 256)
    timings = []
    for rows in (small, large):
        t0 = time.perf_counter()
        oracle_rows(operands, slice(0, rows), gemms)
        timings.append(time.perf_counter() - t0)
    if large == small:
        return n
    per_row = max((timings[1] - timings[0]) / (large - small), 1e-9)
    fixed = max(timings[0] - per_row * small, 0.0)
    return int(min(n, max(large, (seconds - fixed) / per_row)))


def cpu_baseline(kind: str, shape: dict, budget_s: float = 18.0) -> dict:
    """TFLOP/s of the CPU path on this host for a bounded sample of the workload (the whole
    problem when it fits the budget)."""
    m, n, k, gemms, what = cpu_problem(kind, shape)
    operands = host_dense_operands(m, n, k)
    rows = rows_within(operands, n, gemms, budget_s / 3)
    times = []
    for _ in range(3):
        t0 = time.perf_counter()
        oracle_rows(operands, slice(0, rows), gemms)
        times.append(time.perf_counter() - t0)
    best = statistics.median(times)
    result = {
        "value": 2.0 * m * rows * k * gemms / best / 1e12, "unit": "TFLOP/s",
        "cores": os.cpu_count(), "kind": "port",
        "sample": f"numpy oracle (dequantise, FP32 matmul, FP16 cast) on {rows} of {n} rows of "
                  f"B of {what}, median of 3, {best:.3f} s each",
    }
    # The package's torch restatement of the reference's oracle (the workloads'
    # get_reference) on all cores, on the same rows.
    try:
        from harness.workloads.quantization import fp4_matmul

        threads = torch.get_num_threads()
        torch.set_num_threads(os.cpu_count() or threads)
        a, sa = normal_fp4(m, k, 1, "cpu")
        b, sb = normal_fp4(rows, k, 2, "cpu")
        fp4_matmul(a, b, sa, sb, out_dtype=torch.float16)
        t0 = time.perf_counter()
        for _ in range(gemms):
            fp4_matmul(a, b, sa, sb, out_dtype=torch.float16)
        elapsed = time.perf_counter() - t0
        torch.set_num_threads(threads)
        result["torch_path"] = {"value": 2.0 * m * rows * k * gemms / elapsed / 1e12,
                                "unit": "TFLOP/s", "threads": os.cpu_count(),
                                "seconds": elapsed}
    except Exception as error:  # the baseline above stands on its own
        result["torch_path"] = {"unavailable": repr(error)[:200]}
    return result


def reference_arm(args, name: str, kind: str, shape: dict, rank: int) -> None:
    """``--impl reference``: the CPU path alone. Only rank 0 works."""
    if rank != 0:
        return
    m, n, k, gemms, what = cpu_problem(kind, shape)
    operands = host_dense_operands(m, n, k)
    total = args.steps + args.warmup
    rows = rows_within(operands, n, gemms, 120.0 / total)
    rows -= rows % 16 if rows > 16 else 0
    starts = [(i * rows) % max(n - rows, 1) for i in range(total)]
    for i in range(args.warmup):
        oracle_rows(operands, slice(starts[i], starts[i] + rows), gemms)
    t0 = time.perf_counter()
    for i in range(args.warmup, total):
        oracle_rows(operands, slice(starts[i], starts[i] + rows), gemms)
    elapsed = time.perf_counter() - t0
    value = 2.0 * m * rows * k * gemms * args.steps / elapsed / 1e12
    sample = (f"each step: numpy oracle on {rows} of {n} rows of B of {what} "
              f"(host operands, no device)")
    line = {
        "impl": "reference", "metric": "nvfp4_gemm_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "nvfp4", "data": "synthetic",
        "config": {"workload": f"{name}: nvfp4 {kind} GEMM {shape} l=1 (CPU oracle, bounded sample)",
                   "sample_rows": rows},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": os.cpu_count(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), file=args.json_out, flush=True)


# -- GPU arm --------------------------------------------------------------------------------


class Distributed:
    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))

    def barrier(self):
        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(self, values: list[float], device) -> list[float]:
        t = torch.tensor(values, dtype=torch.float64, device=device)
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def sum_over_ranks(self, values: list[float], device) -> list[float]:
        t = torch.tensor(values, dtype=torch.float64, device=device)
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return [float(v) for v in t.tolist()]


class Measured:
    """One workload on this rank: operand sets, prepared launches, validation, timing."""

    def __init__(self, name, kind, shape, dist_info, device, scaling, placement="slices",
                 max_sets=8):
        self.name, self.kind, self.shape = name, kind, shape
        self.dist, self.device = dist_info, device
        world = dist_info.world if scaling == "strong" else 1
        _, byts = algorithmic_work(kind, shape)
        self.sets = min(max_sets, max(3, int(2 * L2_BYTES // max(byts / world, 1)) + 1))
        cls = workload_class(kind)
        self.workload = cls.from_arch("sm_100a", device=device)
        self.operands, self.owned = [], "nothing"
        for index in range(self.sets):
            full = make_operand_set(kind, shape, index, device)
            local, self.owned = shard_operands(kind, full, dist_info.rank, world, placement)
            self.operands.append(local)
            del full
        self.active = self.operands[0] is not None
        self.flops, self.bytes = work_of(kind, self.operands[0])
        self.launches, self.outputs, self.references = [], [], []
        self.max_abs_err = 0.0
        self.validated = False
        self.info = {}
        if self.active:
            for inputs in self.operands:
                launch, outputs = self.workload.prepare(inputs)
                self.launches.append(launch)
                self.outputs.append(outputs)
            self.info = self.workload.plan_info(self.operands[0])

    def close(self):
        self.launches, self.outputs, self.references, self.operands = [], [], [], []
        self.workload.close()
        torch.cuda.empty_cache()

    def validate(self, keep_reference: bool = True) -> None:
        """Every operand set once through its prepared launch against the workload's torch
        reference on this device (rtol = atol = 1e-3); raises on a mismatch."""
        if not self.active:
            self.validated = True
            return
        previous = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            for index, (inputs, launch) in enumerate(zip(self.operands, self.launches)):
                outputs = launch()
                torch.cuda.synchronize()
                reference = self.workload.get_reference(inputs)
                self.workload.validate(reference, outputs)
                self._track_error(reference, outputs)
                if keep_reference and index == 0:
                    self.references = [r.clone() for r in reference]
                del reference
            self.workload.check_status()
        finally:
            torch.backends.cuda.matmul.allow_tf32 = previous
        self.validated = True

    def _track_error(self, reference, outputs) -> None:
        for r, o in zip(reference, outputs):
            diff = (r.float() - o.float()).abs()
            finite = torch.isfinite(diff)
            if finite.any():
                self.max_abs_err = max(self.max_abs_err, float(diff[finite].max().item()))

    def revalidate_first(self) -> None:
        """After the timed region: set 0's output (last written by the timed launches)
        against the reference kept from ``validate``."""
        if self.active and self.references:
            torch.cuda.synchronize()
            self.workload.validate(tuple(self.references), self.outputs[0])
            self.workload.check_status()

    def run(self, count: int, offset: int = 0) -> None:
        if self.active:
            for i in range(count):
                self.launches[(offset + i) % self.sets]()

    def time_replay(self, steps: int, warmup: int, use_graph: bool = True):
        """(elapsed ms of ``steps`` back-to-back launches, how)."""
        self.run(warmup)
        self.dist.barrier()
        graph = None
        if use_graph and self.active:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    self.run(steps)
                graph.replay()  # warm the instantiated graph once
            except Exception as error:  # capture unsupported: time direct launches
                print(f"[bench] CUDA graph capture failed ({error}); timing direct launches",
                      file=sys.stderr)
                graph = None
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.dist.barrier()
        start.record()
        if graph is not None:
            graph.replay()
        else:
            self.run(steps)
        stop.record()
        self.dist.barrier()
        self.graph = graph
        return start.elapsed_time(stop), ("cuda_graph_replay" if graph is not None
                                          else "direct_launches")

    def time_isolated(self, samples: int = 20) -> float:
        """Median microseconds of single launches, each bracketed by its own event pair
        (the reference's method, harness/benchmark.py:19-43 there), rotating operand sets."""
        if not self.active:
            return 0.0
        times = []
        for i in range(samples + 5):
            start, stop = (torch.cuda.Event(enable_timing=True),
                           torch.cuda.Event(enable_timing=True))
            torch.cuda.synchronize()
            start.record()
            self.launches[i % self.sets]()
            stop.record()
            torch.cuda.synchronize()
            if i >= 5:
                times.append(start.elapsed_time(stop) * 1e3)
        return statistics.median(times)

    def time_sustained(self, seconds: float, steps: int):
        """Replays the captured graph back to back for about ``seconds``: microseconds per
        call at whatever clock the power limit leaves, with the wall-clock window."""
        if not self.active or getattr(self, "graph", None) is None:
            return None
        per_replay = max(self.last_ms, 1e-3) * 1e-3
        replays = max(2, int(seconds / per_replay))
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        start.record()
        for _ in range(replays):
            self.graph.replay()
        stop.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        return start.elapsed_time(stop) * 1e3 / (replays * steps), t0, t1

    def roofline(self, name: str, per_call_us: float, world_flops: float, world_bytes: float,
                 issue_tflops):
        bound = BOUND[name]
        if bound == "tensor":
            tf = world_flops / (per_call_us * 1e-6) / 1e12
            peak = NOMINAL_FP4_TFLOPS * self.dist.world
            line = {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s",
                    "frac": tf / peak, "traffic": recorded_traffic(name),
                    "peak_source": "nominal dense FP4 (9 PFLOP/s per GPU)",
                    "algorithmic_flops_per_launch": world_flops / self.dist.world}
            if issue_tflops:
                line["measured_mma_issue_tflops"] = issue_tflops
                line["frac_of_measured_mma_issue"] = tf / (issue_tflops * self.dist.world)
            return line
        peak, peak_kind = measured_hbm_peak()
        achieved = world_bytes / (per_call_us * 1e-6) / 1e9
        return {"bound": "hbm" if bound == "hbm" else "latency", "achieved": achieved,
                "peak": peak * self.dist.world, "unit": "GB/s",
                "frac": achieved / (peak * self.dist.world),
                "traffic": recorded_traffic(name) if self.dist.world == 1 else None,
                "peak_source": f"{peak_kind} HBM copy bandwidth",
                "algorithmic_bytes_per_launch": world_bytes / self.dist.world}


def measure_config(name, dist_info, device, scaling, steps, warmup, issue_tflops,
                   placement="slices", use_graph=True):
    """One entry of ``configs``: validated, graph-replay and isolated timings."""
    kind, shape = WORKLOADS[name]
    measured = Measured(name, kind, shape, dist_info, device, scaling, placement)
    try:
        measured.validate()
        elapsed_ms, how = measured.time_replay(steps, warmup, use_graph)
        isolated = measured.time_isolated()
        measured.revalidate_first()
        elapsed_ms, isolated = dist_info.max_over_ranks([elapsed_ms, isolated], device)
        flops, byts = dist_info.sum_over_ranks([measured.flops, measured.bytes], device)
        err, = dist_info.max_over_ranks([measured.max_abs_err], device)
        per_call_us = elapsed_ms * 1e3 / steps
        entry = {
            "config": name + ("_lpt" if placement == "lpt" else ""),
            "workload": f"nvfp4 {kind} GEMM {shape} l=1, fp16 out",
            "us_per_call": per_call_us, "isolated_us": isolated,
            "timing": f"{how}, back-to-back (PDL overlap); isolated_us: single launches, median",
            "tflops": flops / (per_call_us * 1e-6) / 1e12,
            "roofline": measured.roofline(name, per_call_us, flops, byts, issue_tflops),
            "plan": measured.info, "operand_sets": measured.sets,
            "validated": measured.validated, "max_abs_err": err, "steps": steps,
            "owned_by_rank0": measured.owned,
        }
        return entry
    finally:
        measured.close()


def replay_us(fn, sets: int, iters: int, sustain_s: float = 0.0):
    """Microseconds per call of ``fn(i % sets)`` launched ``iters`` times back to back from a
    CUDA graph between two CUDA events (five warm-up calls and one warm replay first). With
    ``sustain_s`` the graph is then replayed for about that long and the pair (burst,
    sustained) is returned: the second figure is at whatever clock the power limit leaves."""
    for i in range(5):
        fn(i % sets)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(iters):
            fn(i % sets)
    graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.replay()
    stop.record()
    torch.cuda.synchronize()
    burst = start.elapsed_time(stop) * 1e3 / iters
    if sustain_s <= 0.0:
        return burst
    replays = max(2, int(sustain_s / max(burst * iters * 1e-6, 1e-6)))
    start.record()
    for _ in range(replays):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return burst, start.elapsed_time(stop) * 1e3 / (replays * iters)


def competitors(device, square_iters: int) -> list[dict]:
    """Library NVFP4 GEMMs on this GPU, same event method (graph replay over rotating operand
    sets): cuBLASLt through torch._scaled_mm (the call of the task's own reference,
    resources/nvfp4_gemm/reference.py:27-53) and cuDNN through FlashInfer's mm_fp4."""
    results = []

    def operands(m, n, k, sets):
        g = torch.Generator(device=device).manual_seed(1)
        rows = lambda r: -(-r // 128) * 128  # noqa: E731
        cols = -(-(k // 16) // 4) * 4
        out = []
        for _ in range(sets):
            a = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device=device, generator=g)
            b = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=device, generator=g)
            sa = torch.randint(0x30, 0x38, (rows(m), cols), dtype=torch.uint8, device=device,
                               generator=g)
            sb = torch.randint(0x30, 0x38, (rows(n), cols), dtype=torch.uint8, device=device,
                               generator=g)
            out.append((a, b, sa, sb))
        return out

    timed = replay_us

    def scaled_mm(m, n, k, ops):
        f4, e4 = torch.float4_e2m1fn_x2, torch.float8_e4m3fn
        prepared = [(a.view(f4), b.view(f4).t(), sa.view(e4).flatten(), sb.view(e4).flatten())
                    for a, b, sa, sb in ops]
        return lambda i: torch._scaled_mm(*prepared[i], bias=None, out_dtype=torch.float16)

    def cudnn_mm(m, n, k, ops):
        import flashinfer

        alpha = torch.ones(1, device=device)
        e4 = torch.float8_e4m3fn
        prepared = [(a, b.t(), sa.view(e4), sb.view(e4).t()) for a, b, sa, sb in ops]
        outs = [torch.empty(m, n, dtype=torch.float16, device=device) for _ in ops]
        return lambda i: flashinfer.mm_fp4(*prepared[i], alpha, torch.float16, outs[i],
                                           backend="cudnn")

    def trtllm_mm(m, n, k, ops):
        # The prebuilt trtllm-gen kernels (the Gemm_Bfloat16_E2m1E2m1 family the reference
        # ships as cubins): BF16 output, weights in the shuffled layout. Random bytes time
        # the same as prepared weights.
        import flashinfer

        alpha = torch.ones(1, device=device)
        e4 = torch.float8_e4m3fn
        prepared = [(a, b.t(), sa.view(e4), sb.view(e4).t()) for a, b, sa, sb in ops]
        outs = [torch.empty(m, n, dtype=torch.bfloat16, device=device) for _ in ops]
        return lambda i: flashinfer.mm_fp4(*prepared[i], alpha, torch.bfloat16, outs[i],
                                           backend="trtllm")

    for label, make in (("cublaslt via torch._scaled_mm", scaled_mm),
                        ("cudnn via flashinfer.mm_fp4", cudnn_mm),
                        ("trtllm-gen cubins via flashinfer.mm_fp4", trtllm_mm)):
        for name in ("decode", "square"):
            shape = WORKLOADS[name][1]
            m, n, k = shape["m"], shape["n"], shape["k"]
            sets = 4 if name == "decode" else 3
            try:
                iters = square_iters if name == "square" else 200
                launch = make(m, n, k, operands(m, n, k, sets))
                entry = {"library": label, "config": name, "steps": iters}
                if name == "square" and make is scaled_mm:
                    # The same 3 s under the power limit that the headline's `sustained` has.
                    us, entry["sustained_us_per_call"] = timed(launch, sets, iters, 3.0)
                else:
                    us = timed(launch, sets, iters)
                entry.update(us_per_call=us, tflops=2.0 * m * n * k / us / 1e6)
                results.append(entry)
            except Exception as error:
                results.append({"library": label, "config": name,
                                "unavailable": f"unavailable on this box: {error!r}"[:300]})
            torch.cuda.empty_cache()
    return results


def _hbm_line(byts: float, us: float, traffic=None) -> dict:
    peak, peak_kind = measured_hbm_peak()
    achieved = byts / (us * 1e-6) / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "traffic": traffic,
            "peak_source": f"{peak_kind} HBM copy bandwidth",
            "algorithmic_bytes_per_launch": byts}


def _tensor_line(flops: float, us: float) -> dict:
    tf = flops / (us * 1e-6) / 1e12
    return {"bound": "tensor", "achieved": tf, "peak": NOMINAL_FP4_TFLOPS, "unit": "TFLOP/s",
            "frac": tf / NOMINAL_FP4_TFLOPS, "traffic": None,
            "peak_source": "nominal dense FP4 (9 PFLOP/s per GPU)",
            "algorithmic_flops_per_launch": flops}


class _NativePlan:
    """A plan with its workspace on the current stream, for the rows that go through the
    C ABI directly (``harness/native.py``)."""

    def __init__(self, plan, device):
        self.plan, self.device = plan, device
        self.workspace = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8,
                                     device=device)
        plan.init_workspace(self.workspace.data_ptr(), self.stream)
        torch.cuda.synchronize(device)

    @property
    def stream(self) -> int:
        """The stream current at the time of the call (a capturing stream inside a graph)."""
        return torch.cuda.current_stream(self.device).cuda_stream

    def status(self) -> int:
        return self.plan.status(self.workspace.data_ptr(), self.stream)

    def close(self):
        torch.cuda.synchronize()
        self.plan.destroy()


def row_quantiser(device) -> dict:
    """The activation quantiser (``nvfp4_quantize``): BF16 [8192, 8192] to packed E2M1 and
    blocked scales, against the torch quantiser on the first 1024 rows."""
    from harness.workloads import quantization as q

    rows, k, sets = 8192, 8192, 2
    xs = [torch.randn((1, rows, k), generator=torch.Generator().manual_seed(70 + i))
          .to(device=device, dtype=torch.bfloat16).permute(1, 2, 0) for i in range(sets)]
    packed, blocked = q.quantize_nvfp4_native(xs[0])
    want_packed, want_scales = q.quantize_nvfp4(xs[0][:1024].float())
    ok = (torch.equal(packed[:1024], want_packed) and
          torch.equal(blocked[:, :8].view(torch.uint8),
                      q.to_blocked_scales(want_scales).view(torch.uint8)))
    us = replay_us(lambda i: q.quantize_nvfp4_native(xs[i]), sets, 40)
    byts = rows * k * 2 + rows * k // 2 + rows * k // 16
    return {"row": "f1 activation quantiser", "entry": "nvfp4_quantize",
            "workload": f"bf16 [{rows}, {k}] -> packed e2m1 + blocked ue4m3 scales",
            "us_per_call": us, "validated": bool(ok),
            "roofline": _hbm_line(byts, us, summary_traffic("nvfp4_quantize_bf16_8192x8192.md")),
            "note": "timed with its two output allocations from torch's caching allocator"}


def row_fp4_output(device) -> list[dict]:
    """GEMMs whose epilogue quantises D to NVFP4: the square shape and the dual shape. The
    dense result must equal, byte for byte, the quantiser kernel applied to the FP32 output of
    the same plan family; the dual result (approximate silu) is checked after dequantisation
    against the FP16-output kernel."""
    from harness import native
    from harness.workloads import quantization as q

    rows_out = []
    index = device.index or 0
    # Dense, 8192^3.
    kind, shape = WORKLOADS["square"]
    m, n, k = shape["m"], shape["n"], shape["k"]
    sets = 3
    operands = [make_operand_set(kind, shape, 40 + i, device) for i in range(sets)]
    fp4 = _NativePlan(native.Plan.dense(index, native.OUT_FP4, m, n, k, 1), device)
    f32 = _NativePlan(native.Plan.dense(index, native.OUT_F32, m, n, k, 1), device)
    packed = [torch.empty((1, m, n // 2), dtype=torch.uint8, device=device) for _ in range(sets)]
    scales = [torch.zeros((1, -(-m // 128), n // 64, 32, 4, 4), dtype=torch.uint8, device=device)
              for _ in range(sets)]

    def dense(i):
        a, b, sfa, sfb, alpha = operands[i][:5]
        fp4.plan.launch_dense_fp4(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
                                  alpha.data_ptr(), packed[i].data_ptr(), scales[i].data_ptr(),
                                  fp4.workspace.data_ptr(), fp4.stream)

    dense(0)
    a, b, sfa, sfb, alpha = operands[0][:5]
    product = torch.empty((1, m, n), dtype=torch.float32, device=device)
    f32.plan.launch_dense(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
                          alpha.data_ptr(), product.data_ptr(), f32.workspace.data_ptr(),
                          f32.stream)
    want_packed, want_scales = q.quantize_nvfp4_native(product.permute(1, 2, 0))
    ok = (fp4.status() == 0 and f32.status() == 0 and
          torch.equal(packed[0], want_packed.permute(2, 0, 1)) and
          torch.equal(scales[0], want_scales.view(torch.uint8)))
    del product, want_packed, want_scales
    us = replay_us(dense, sets, 30)
    rows_out.append({"row": "f2 NVFP4-output epilogue, dense", "entry": "nvfp4_gemm_launch_fp4",
                     "workload": f"square {shape}, D packed e2m1 + blocked scales",
                     "us_per_call": us, "validated": bool(ok), "plan": fp4.plan.info(),
                     "roofline": _tensor_line(2.0 * m * n * k, us)})
    fp4.close()
    f32.close()
    del operands, packed, scales
    torch.cuda.empty_cache()

    # Dual (gate/up), the dual workload's shape.
    kind, shape = WORKLOADS["dual"]
    m, n, k = shape["m"], shape["n"], shape["k"]
    sets = 4
    # alpha = 1/32 keeps silu(h1) * h2 of N(0,1) operands inside FP16, which the check below
    # compares with.
    alpha = torch.full((1,), 1.0 / 32.0, device=device)
    operands = [make_operand_set(kind, shape, 50 + i, device)[:6] + (alpha,) for i in range(sets)]
    fp4 = _NativePlan(native.Plan.dual_fp4(index, m, n, k, 1), device)
    f16 = _NativePlan(native.Plan.dual(index, m, n, k, 1), device)
    packed = [torch.zeros((1, m, n // 2), dtype=torch.uint8, device=device) for _ in range(sets)]
    scales = [torch.zeros((1, -(-m // 128), n // 64, 32, 4, 4), dtype=torch.uint8, device=device)
              for _ in range(sets)]

    def dual(i):
        fp4.plan.launch_dual_fp4(*(t.data_ptr() for t in operands[i]), packed[i].data_ptr(),
                                 scales[i].data_ptr(), fp4.workspace.data_ptr(), fp4.stream)

    dual(0)
    half = torch.empty((1, m, n), dtype=torch.float16, device=device)
    f16.plan.launch_dual(*(t.data_ptr() for t in operands[0]), half.data_ptr(),
                         f16.workspace.data_ptr(), f16.stream)
    ok = fp4.status() == 0 and f16.status() == 0
    logical = q.from_blocked_scales(scales[0].view(torch.float8_e4m3fn), m, n // 16)
    got = q.dequant_fp4(packed[0].permute(1, 2, 0), logical)[..., 0]
    want = half[0].float()
    # One E2M1 step at a block's scale is amax/6 of the block; well inside it on average.
    error = (got - want).norm().item() / max(want.norm().item(), 1e-30)
    ok = ok and error < 0.12
    us = replay_us(dual, sets, 200)
    _, byts = algorithmic_work(kind, shape)
    byts += -2.0 * m * n + m * n / 2 + m * n / 16
    rows_out.append({"row": "f2 NVFP4-output epilogue, dual (gate/up)",
                     "entry": "nvfp4_dual_gemm_launch_fp4",
                     "workload": f"dual {shape}, D packed e2m1 + blocked scales",
                     "us_per_call": us, "validated": bool(ok),
                     "relative_error_to_fp16_output": error, "plan": fp4.plan.info(),
                     "roofline": _hbm_line(byts, us)})
    fp4.close()
    f16.close()
    del operands, packed, scales
    torch.cuda.empty_cache()
    return rows_out


def row_shuffled(device) -> dict:
    """BF16 output on weights in the trtllm row order, decode shape, through the operator
    API (workload ``nvfp4_gemm_bf16_shuffled``) against its torch reference."""
    from harness import get_workload

    kind, shape = WORKLOADS["decode"]
    sets = 4
    workload = get_workload("nvfp4_gemm_bf16_shuffled").from_arch("sm_100a", device=device)
    operands = [make_operand_set(kind, shape, 60 + i, device) for i in range(sets)]
    prepared = [workload.prepare(inputs) for inputs in operands]
    outputs = prepared[0][0]()
    torch.cuda.synchronize()
    ok = True
    try:
        workload.validate(workload.get_reference(operands[0]), outputs)
        workload.check_status()
    except AssertionError:
        ok = False
    us = replay_us(lambda i: prepared[i][0](), sets, 200)
    _, byts = algorithmic_work(kind, shape)
    info = workload.plan_info(operands[0])
    workload.close()
    return {"row": "f3 BF16 output on shuffled weights",
            "entry": "nvfp4_gemm_plan_create_shuffled + nvfp4_gemm_launch",
            "workload": f"decode {shape}, B rows in the trtllm-gen order (block 32), bf16 out",
            "us_per_call": us, "validated": ok, "plan": info, "roofline": _hbm_line(byts, us)}


def row_moe(device) -> list[dict]:
    """One rank's share of a DeepSeek-V3 MoE layer under 8-way expert parallelism (32 local
    experts, hidden 7168, intermediate 2048; the reference sizes its grouped cases the same
    way, harness/workloads/nvfp4_group_gemm.py:751-785 there): the rows routed to this rank at
    1,024 and 16,384 tokens, per-expert counts seeded log-normal. ``layer_us`` is
    ``MoELayer.forward_rows`` (quantiser and two grouped launches on the pattern's bound
    buffers) called from Python, ``layer_graph_us`` the same forward replayed from a CUDA
    graph; ``kernels_us`` the two grouped launches alone replayed from a graph;
    ``shard_forward_us`` everything a rank does with the rows an all-to-all delivered (route,
    gather-quantise, both GEMMs, un-permute; ``moe.ep_local_experts``);
    ``routed_forward_us`` / ``routed_forward_graph_us`` the same work by ``RoutedMoELayer``,
    which reads nothing back from the device. The busiest
    expert's rows are checked against the stage-by-stage torch reference."""
    from harness import moe
    from harness.models import MODELS
    from harness.throughput import skewed_lengths
    from harness.workloads import quantization as q

    spec = MODELS["deepseek_v3"]
    local = 32
    shapes = spec.linear_shapes()
    (two_i, hidden), (_, inter) = shapes["expert_gate_up"], shapes["expert_down"]
    gen = torch.Generator(device=device).manual_seed(90)

    def weights(rows, k):
        packed = torch.empty((local, rows, k // 2), dtype=torch.uint8, device=device)
        blocked = torch.empty((local, -(-rows // 128), -(-k // 64), 32, 4, 4),
                              dtype=torch.float8_e4m3fn, device=device)
        for e in range(local):
            w = torch.randn((1, rows, k), device=device, generator=gen) * 0.05
            p, s = q.quantize_nvfp4_native(w.permute(1, 2, 0))
            packed[e], blocked[e] = p[..., 0], s[0]
        return packed, blocked

    w13, w13_scales = weights(two_i, hidden)
    w2, w2_scales = weights(hidden, inter)
    layer = moe.MoELayer(w13, w13_scales, w2, w2_scales, fused=True)
    out = []
    for tokens in (1024, 16384):
        routed = tokens * spec.top_k * local // spec.experts
        counts = list(skewed_lengths(routed, local, seed=tokens, minimum=0))
        starts, total = [], 0
        for count in counts:
            starts.append(total)
            total += -(-count // 128) * 128
        rows = torch.zeros((max(total, 128), hidden), dtype=torch.float32, device=device)
        for e, count in enumerate(counts):
            rows[starts[e]:starts[e] + count] = torch.randn((count, hidden), device=device,
                                                            generator=gen)
        y = layer.forward_rows(rows, counts, starts)
        layer.check_status()
        probe = max(range(local), key=lambda e: counts[e])
        span = slice(starts[probe], starts[probe] + counts[probe])
        want = moe.expert_reference(
            rows[span], w13[probe],
            q.from_blocked_scales(w13_scales[probe][None], two_i, hidden // 16)[..., 0],
            w2[probe], q.from_blocked_scales(w2_scales[probe][None], hidden, inter // 16)[..., 0],
            fused=True)
        error = ((y[span].float() - want.float()).norm() / want.float().norm()).item()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            y = layer.forward_rows(rows, counts, starts)
        torch.cuda.synchronize()
        repeats = 10
        start.record()
        for _ in range(repeats):
            y = layer.forward_rows(rows, counts, starts)
        stop.record()
        torch.cuda.synchronize()
        layer_us = start.elapsed_time(stop) * 1e3 / repeats
        pattern = layer._entry(tuple(counts), torch.cuda.current_stream(device).cuda_stream)

        def kernels(_):
            stream = torch.cuda.current_stream(device).cuda_stream
            pattern.up_plan.launch_groups(pattern.up_ws.data_ptr(), stream)
            pattern.down_plan.launch_groups(pattern.down_ws.data_ptr(), stream)

        kernels_us = replay_us(kernels, 1, 20)
        # The whole forward of a known pattern is three launches on bound buffers, so it can be
        # captured: the layer without the host's share.
        side = torch.cuda.Stream(device)
        with torch.cuda.stream(side):
            layer.forward_rows(rows, counts, starts)  # the pattern's buffers on this stream
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(20):
                    layer.forward_rows(rows, counts, starts)
            graph.replay()
            side.synchronize()
            start.record(side)
            graph.replay()
            stop.record(side)
            side.synchronize()
        layer_graph_us = start.elapsed_time(stop) * 1e3 / 20
        del graph
        # What the rank does with the rows an all-to-all delivered (BF16 rows in arrival order,
        # one expert each): route, gather-quantise, both GEMMs, un-permute; the row counts are
        # read back on the host.
        arrived = torch.randn((routed, hidden), device=device, generator=gen).to(torch.bfloat16)
        expert_of_row = torch.repeat_interleave(
            torch.arange(local, device=device), torch.tensor(counts, device=device))
        expert_of_row = expert_of_row[torch.randperm(routed, device=device, generator=gen)]
        shard = moe.ep_local_experts(layer)
        for _ in range(3):
            shard(arrived, expert_of_row)
        torch.cuda.synchronize()
        start.record()
        for _ in range(repeats):
            shard(arrived, expert_of_row)
        stop.record()
        torch.cuda.synchronize()
        shard_us = start.elapsed_time(stop) * 1e3 / repeats
        # The same with nothing read back (RoutedMoELayer: counts, layout and placement on the
        # device, one pair of plans for any routing), called from Python and replayed from a
        # CUDA graph; it must give the planned layer's bits.
        routed_layer = moe.RoutedMoELayer(w13, w13_scales, w2, w2_scales, max_pairs=routed)
        ones = torch.ones((routed, 1), device=device)
        ids = expert_of_row[:, None].contiguous()
        same = torch.equal(routed_layer.forward(arrived, ids, ones), shard(arrived, expert_of_row).float())
        for _ in range(2):
            routed_layer.forward(arrived, ids, ones)
        torch.cuda.synchronize()
        start.record()
        for _ in range(repeats):
            routed_layer.forward(arrived, ids, ones)
        stop.record()
        torch.cuda.synchronize()
        routed_us = start.elapsed_time(stop) * 1e3 / repeats
        with torch.cuda.stream(side):
            routed_layer.forward(arrived, ids, ones)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(20):
                    routed_layer.forward(arrived, ids, ones)
            graph.replay()
            side.synchronize()
            start.record(side)
            graph.replay()
            stop.record(side)
            side.synchronize()
        routed_graph_us = start.elapsed_time(stop) * 1e3 / 20
        routed_layer.check_status()
        del graph
        routed_layer.close()
        del arrived
        layer.check_status()
        del y
        live = sum(1 for count in counts if count)
        flops = 2.0 * routed * (two_i * hidden + hidden * inter)
        weight_bytes = live * (two_i * hidden + hidden * inter) * (0.5 + 1.0 / 16)
        row_bytes = routed * (hidden * (0.5 + 1.0 / 16) + 2 * inter * (0.5 + 1.0 / 16)
                              + 2.0 * hidden)
        byts = weight_bytes + row_bytes
        traffic = (summary_traffic("nvfp4_moe_shard_deepseek_v3_1024_tokens.md")
                   if tokens == 1024 else None)
        line = (_tensor_line(flops, kernels_us) if flops / 9e15 > byts / 6.5e12
                else _hbm_line(byts, kernels_us, traffic))
        out.append({"row": "f4 MoE layer (expert-parallel shard)",
                    "entry": "nvfp4_group_dual_gemm_bind_fp4 + nvfp4_group_gemm_bind + "
                             "nvfp4_group_gemm_launch x2 + nvfp4_quantize",
                    "workload": f"deepseek_v3 experts, {local} local of {spec.experts}, "
                                f"{tokens} tokens -> {routed} routed rows, {live} live experts, "
                                f"hidden {hidden}, intermediate {inter}",
                    "layer_us": layer_us, "layer_graph_us": layer_graph_us,
                    "shard_forward_us": shard_us,
                    "routed_forward_us": routed_us, "routed_forward_graph_us": routed_graph_us,
                    "routed_equals_planned": bool(same),
                    "kernels_us": kernels_us,
                    "us_per_call": kernels_us, "tflops": flops / kernels_us / 1e6,
                    "validated": bool(error < 1e-2), "relative_error_of_probed_expert": error,
                    "roofline": line,
                    "note": "weights of one operand set (791 MB) exceed L2; kernels_us replays "
                            "the bound launches on the same operands"})
    layer.close()
    del w13, w13_scales, w2, w2_scales
    torch.cuda.empty_cache()
    return out


def row_expert_parallel(info, device) -> dict:
    """The MoE layer expert-parallel over the ranks of this run: DeepSeek-V3's 256 experts
    (hidden 7168, intermediate 2048) in contiguous blocks per rank, 2,048 BF16 tokens per rank
    routed top-8 over all experts; one forward = route, two all-to-all exchanges (rows out as
    BF16, back as FP16), the local experts on the routed grouped kernels (``RoutedMoELayer``: no
    host read on the receiving side), weighted combine. Expert e's
    weights come from seed e on whichever rank owns it, so rank 0 can rebuild any expert and
    checks a few of its tokens against the stage-by-stage torch reference."""
    from harness import moe
    from harness.models import MODELS
    from harness.workloads import quantization as q

    spec = MODELS["deepseek_v3"]
    world, rank = info.world, info.rank
    experts, hidden = spec.experts, spec.hidden
    (two_i, _), (_, inter) = spec.linear_shapes()["expert_gate_up"], spec.linear_shapes()["expert_down"]
    per_rank = -(-experts // world)
    tokens, choices = 2048, spec.top_k

    def expert_weights(e: int):
        g = torch.Generator(device=device).manual_seed(5000 + e)
        out = []
        for rows, k in ((two_i, hidden), (hidden, inter)):
            w = torch.randn((1, rows, k), device=device, generator=g) * 0.05
            p, blocked = q.quantize_nvfp4_native(w.permute(1, 2, 0))
            out += [p[..., 0], blocked[0].view(torch.uint8)]
        return out  # w13, w13 scales (blocked bytes), w2, w2 scales (blocked bytes)

    mine = range(rank * per_rank, min(experts, (rank + 1) * per_rank))
    parts = [expert_weights(e) for e in mine]
    # A layer that reads nothing back, made for as many pairs as can arrive at this rank.
    layer = moe.RoutedMoELayer(*(torch.stack([p[i] for p in parts]) for i in range(4)),
                               max_pairs=tokens * spec.top_k * world)
    del parts
    g = torch.Generator(device=device).manual_seed(7000 + rank)
    x = torch.randn((tokens, hidden), device=device, generator=g).to(torch.bfloat16)
    scores = torch.rand((tokens, experts), device=device, generator=g)
    weights, ids = torch.topk(scores, choices, dim=1)
    weights = weights / weights.sum(dim=1, keepdim=True)
    local = moe.ep_local_experts(layer)

    def forward():
        return moe.moe_forward_ep(x, ids, weights, experts, local)

    out = forward()
    layer.check_status()
    ok = bool(torch.isfinite(out).all())
    if rank == 0:
        sample = slice(0, 4)
        want = torch.zeros((4, hidden), dtype=torch.float32, device=device)
        for t in range(4):
            for j in range(choices):
                e = int(ids[t, j])
                w13, s13, w2, s2 = expert_weights(e)
                y = moe.expert_reference(
                    x[t:t + 1].float(), w13,
                    q.from_blocked_scales(s13[None].view(torch.float8_e4m3fn), two_i, hidden // 16)[..., 0],
                    w2, q.from_blocked_scales(s2[None].view(torch.float8_e4m3fn), hidden, inter // 16)[..., 0],
                    fused=True)
                want[t] += weights[t, j] * y[0].float()
        error = ((out[sample] - want).norm() / want.norm()).item()
        ok = ok and error < 1e-2
    else:
        error = 0.0
    for _ in range(2):
        forward()
    info.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    repeats = 10
    start.record()
    for _ in range(repeats):
        forward()
    stop.record()
    info.barrier()
    us, = info.max_over_ranks([start.elapsed_time(stop) * 1e3 / repeats], device)
    ok_all, = info.max_over_ranks([0.0 if ok else 1.0], device)
    layer.check_status()
    layer.close()
    torch.cuda.empty_cache()
    flops = 2.0 * tokens * world * choices * (two_i * hidden + hidden * inter)
    return {"config": "moe_expert_parallel",
            "workload": f"deepseek_v3 experts: {experts} over {world} ranks ({per_rank} each), "
                        f"{tokens} bf16 tokens per rank, top-{choices}, hidden {hidden}, "
                        f"intermediate {inter}",
            "us_per_forward": us, "tflops": flops / us / 1e6,
            "validated": ok_all == 0.0, "relative_error_of_sampled_tokens": error,
            "exchange": "torch.distributed all_to_all_single over NCCL: rows out as BF16, back as "
                        "FP16; no peer-memory kernel",
            "timing": "CUDA events around 10 forwards called from Python, max over ranks"}


def next_rows(device, only: str = "") -> list[dict]:
    """The rows beside the GEMM path (quantiser, NVFP4-output epilogues, shuffled weights, the
    MoE layer), each validated and timed like ``configs``. A row that fails says so and the
    others still run."""
    rows = []
    wanted = {name for name in only.split(",") if name}
    for make in (row_quantiser, row_fp4_output, row_shuffled, row_moe):
        if wanted and make.__name__.removeprefix("row_") not in wanted:
            continue
        try:
            made = make(device)
            rows += made if isinstance(made, list) else [made]
        except Exception as error:  # reported, not hidden
            rows.append({"row": make.__name__, "failed": repr(error)[:400]})
        torch.cuda.empty_cache()
    return rows


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="native", choices=("native", "reference"))
    parser.add_argument("--workload", default="square", choices=sorted(WORKLOADS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-graph", action="store_true")
    parser.add_argument("--no-configs", action="store_true",
                        help="headline workload only (no configs array, no competitors)")
    parser.add_argument("--next-rows-only", action="store_true",
                        help="measure only the rows beside the GEMM path (one GPU)")
    parser.add_argument("--rows", default="",
                        help="with --next-rows-only: a comma-separated subset of quantiser, "
                             "fp4_output, shuffled, moe")
    parser.add_argument("--scaling", default="strong", choices=("strong", "weak"),
                        help="strong: the workload's N is split over the ranks; weak: every "
                             "rank runs the whole shape")
    args = parser.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    name = args.workload
    kind, shape = WORKLOADS[name]
    info = Distributed()
    # Libraries print to stdout as they please (cuDNN announces its handle): everything but
    # the one JSON line goes to stderr.
    sys.stdout.flush()
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)

    args.json_out = json_out
    if args.impl == "reference":
        reference_arm(args, name, kind, shape, info.rank)
        return

    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(info.local_rank)
    device = torch.device("cuda", info.local_rank)
    world = info.world
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    from harness import native, sharding

    if args.next_rows_only:
        if info.rank == 0:
            print(json.dumps({"next_rows": next_rows(device, args.rows)}), file=json_out,
                  flush=True)
        return

    issue_tflops = None
    try:
        issue_tflops = native.measure_mma_peak(info.local_rank, 4096)
    except Exception:
        pass

    with ClockSampler(info.local_rank) as clocks:
        headline = Measured(name, kind, shape, info, device, args.scaling)
        headline.validate()
        t_begin = time.perf_counter()
        elapsed_ms, how = headline.time_replay(args.steps, args.warmup, not args.no_graph)
        t_end = time.perf_counter()
        headline.last_ms = elapsed_ms
        clock_line = clocks.summary(t_begin, t_end)

        # Direct (non-graph) launches and isolated single launches, for the record.
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        info.barrier()
        direct_steps = min(args.steps, 200)
        start.record()
        headline.run(direct_steps)
        stop.record()
        info.barrier()
        direct_us = start.elapsed_time(stop) * 1e3 / direct_steps
        isolated_us = headline.time_isolated()
        sustained = headline.time_sustained(3.0, args.steps) if BOUND[name] == "tensor" else None
        headline.revalidate_first()

        # The optional exchange: every rank's columns of D gathered on every rank.
        gather_us = None
        if world > 1 and args.scaling == "strong" and kind != "grouped":
            spans = sharding.row_shards(shape["n"], world)
            local = headline.outputs[0][0]
            for _ in range(2):
                sharding.all_gather_columns(local, spans)
            info.barrier()
            times = []
            for _ in range(5):
                start.record()
                sharding.all_gather_columns(local, spans)
                stop.record()
                torch.cuda.synchronize()
                times.append(start.elapsed_time(stop) * 1e3)
            gather_us, = info.max_over_ranks([statistics.median(times)], device)

        # End to end through the operator API: pinned host operands in, D out, per step.
        e2e_steps = max(3, min(args.steps, 10 if headline.bytes > (64 << 20) else 30))
        h2d = d2h = 0
        e2e_ms = serial_ms = 0.0
        if headline.active:
            host_sets = [tuple(t.cpu().pin_memory() for t in inputs)
                         for inputs in headline.operands[:2]]
            staging = [tuple(torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=device)
                             for t in headline.operands[0]) for _ in range(2)]
            h2d = sum(t.numel() * t.element_size() for t in host_sets[0])
            host_out = [None]

            def e2e_step(i: int) -> int:
                src, dst = host_sets[i % 2], staging[i % 2]
                for s, d in zip(src, dst):
                    d.copy_(s, non_blocking=True)
                outputs = headline.workload.run(dst)
                outs = [o.to("cpu", non_blocking=True) for o in outputs]
                torch.cuda.current_stream().synchronize()
                host_out[0] = outs
                return sum(o.numel() * o.element_size() for o in outputs)

            d2h = e2e_step(0)
            e2e_step(1)
            info.barrier()
            start.record()
            for i in range(e2e_steps):
                e2e_step(i)
            stop.record()
            info.barrier()
            serial_ms = start.elapsed_time(stop)

            # The same steps with the copies of neighbouring steps overlapped (PCIe carries
            # both directions at once): step i's operands go in on one stream while step
            # i-1's D comes out on another; two buffers each way. Every step still copies its
            # operands from pinned host memory and its D back to pinned host memory inside the
            # timed region.
            current = torch.cuda.current_stream()
            s_in, s_run, s_out = (torch.cuda.Stream(device) for _ in range(3))
            pinned_out = [None, None]
            device_out = [None, None]
            ev_in = [torch.cuda.Event() for _ in range(2)]
            ev_run = [torch.cuda.Event() for _ in range(2)]
            ev_out = [torch.cuda.Event() for _ in range(2)]

            def pipelined(steps: int) -> None:
                for i in range(steps):
                    b = i % 2
                    if i >= 2:
                        ev_out[b].synchronize()      # the host has step i-2's D
                    with torch.cuda.stream(s_in):
                        if i >= 2:
                            s_in.wait_event(ev_run[b])  # the GEMM that read staging[b] is done
                        for src_t, dst_t in zip(host_sets[b], staging[b]):
                            dst_t.copy_(src_t, non_blocking=True)
                        ev_in[b].record(s_in)
                    with torch.cuda.stream(s_run):
                        s_run.wait_event(ev_in[b])
                        device_out[b] = headline.workload.run(staging[b])
                        ev_run[b].record(s_run)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(ev_run[b])
                        if pinned_out[b] is None:
                            pinned_out[b] = [torch.empty(o.shape, dtype=o.dtype, pin_memory=True)
                                             for o in device_out[b]]
                        for o, h in zip(device_out[b], pinned_out[b]):
                            h.copy_(o, non_blocking=True)
                        ev_out[b].record(s_out)
                for stream in (s_in, s_run, s_out):
                    current.wait_stream(stream)

            for stream in (s_in, s_run, s_out):
                stream.wait_stream(current)
            pipelined(4)
            torch.cuda.synchronize()
            info.barrier()
            start.record()
            pipelined(e2e_steps)
            stop.record()
            info.barrier()
            e2e_ms = start.elapsed_time(stop)
            # The bytes that came back are the GEMM's: compare them with the reference.
            last = (e2e_steps - 1) % 2
            reference = headline.workload.get_reference(staging[last])
            reference = tuple(r.cpu() for r in reference)
            headline.workload.validate(reference, tuple(pinned_out[last]))
            headline.workload.validate(reference, tuple(host_out[0]))  # same operands, serial run
            headline.workload.check_status()
            del reference, host_sets, staging, pinned_out, device_out
        else:
            info.barrier()
            info.barrier()

        elapsed_ms, e2e_ms, serial_ms, direct_us, isolated_us = info.max_over_ranks(
            [elapsed_ms, e2e_ms, serial_ms, direct_us, isolated_us], device)
        world_flops, world_bytes, h2d_all, d2h_all = info.sum_over_ranks(
            [headline.flops, headline.bytes, float(h2d), float(d2h)], device)
        err, = info.max_over_ranks([headline.max_abs_err], device)
        plan_info, sets, owned = headline.info, headline.sets, headline.owned
        per_call_us = elapsed_ms * 1e3 / args.steps
        roofline = headline.roofline(name, per_call_us, world_flops, world_bytes, issue_tflops)
        sustained_line = None
        if sustained is not None:
            sustained_us, s0, s1 = sustained
            s_clock = clocks.summary(s0, s1)
            sustained_line = {
                "us_per_call": sustained_us,
                "tflops": world_flops / world / (sustained_us * 1e-6) / 1e12,
                "seconds": s1 - s0, "sm_mhz": s_clock.get("sm_mhz"),
                "reasons": s_clock.get("reasons"),
                "us_times_mhz": sustained_us * (s_clock.get("sm_mhz") or 0),
                "note": "graph replayed back to back for ~3 s on this rank: the clock is "
                        "whatever the power limit leaves",
            }
        headline.close()

        configs = []
        if not args.no_configs:
            for other in ("latency", "decode", "dual", "grouped"):
                if other == name:
                    continue
                steps = 1000 if other == "latency" else 200
                if world > 1 and other == "latency":
                    continue  # two 128-row shards at most: not a multi-GPU problem
                configs.append(measure_config(other, info, device, args.scaling, steps, 20,
                                              issue_tflops, use_graph=not args.no_graph))
                if other == "grouped" and world > 1 and args.scaling == "strong":
                    configs.append(measure_config(other, info, device, args.scaling, steps, 20,
                                                  issue_tflops, placement="lpt",
                                                  use_graph=not args.no_graph))
            if world > 1:
                try:
                    configs.append(row_expert_parallel(info, device))
                except Exception as error:  # reported, not hidden; every rank raises or none
                    configs.append({"config": "moe_expert_parallel", "failed": repr(error)[:400]})
        all_clock = clocks.summary()

    if info.rank == 0:
        value = world_flops * args.steps / (elapsed_ms * 1e-3) / 1e12
        e2e_value = world_flops * e2e_steps / (e2e_ms * 1e-3) / 1e12 if e2e_ms else 0.0
        split = (f" (global n = {shape.get('n')} split over {world} ranks in 128-row shards)"
                 if world > 1 and args.scaling == "strong" else
                 f" (every one of {world} ranks runs the whole shape)" if world > 1 else "")
        line = {
            "metric": "nvfp4_gemm_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": elapsed_ms / args.steps, "us_per_call": per_call_us,
            "isolated_us": isolated_us,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "nvfp4", "data": "synthetic",
            "validated": True, "max_abs_err": err,
            "config": {
                "workload": f"{name}: nvfp4 {kind} GEMM {shape} l=1, fp16 out" + split,
                "operand_sets": sets,
                "l2": f"{sets} operand sets rotate, larger than the 126 MB L2 together",
                "timing": f"{how}, back-to-back (PDL overlap); isolated_us: single launches, "
                          "median",
                "direct_launch_us_per_call": direct_us, "plan": plan_info,
                "sharding": "each rank owns an N-shard; no collective on the data path",
                "rank0_owns": owned,
            },
            "roofline": roofline,
            "sustained": sustained_line,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d_all),
                    "d2h_bytes_per_step": int(d2h_all), "steps": e2e_steps,
                    "ms_per_step": e2e_ms / e2e_steps if e2e_steps else None,
                    "serial_ms_per_step": serial_ms / e2e_steps if e2e_steps else None,
                    "how": "Workload.run on operands copied from pinned host memory, D copied "
                           "back to pinned host memory, every step; copies of neighbouring "
                           "steps overlap on separate streams (serial_ms_per_step: one step at "
                           "a time)",
                    "validated": True},
            "gpu_launches": args.steps,
            "clocks": clock_line,
            "clocks_whole_run": all_clock,
            "configs": configs,
        }
        if gather_us is not None:
            line["all_gather_us"] = gather_us
        if world == 1 and not args.no_configs:
            line["competitors"] = competitors(
                device, args.steps if name == "square" else 50)
            line["next_rows"] = next_rows(device)
        line["cpu_baseline"] = None if args.no_cpu_baseline else cpu_baseline(kind, shape)
        print(json.dumps(line), file=json_out, flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
