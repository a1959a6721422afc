#!/usr/bin/env python
"""Benchmark of the NVFP4 block-scaled GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]
                    [--workload decode|square|dual|grouped]

One JSON line on stdout (rank 0). A *step* is one GEMM call on one set of synthetic
operands. The default workload is the skinny, HBM-bound decode GEMM
(M=128, N=7168, K=16384, FP16 out): A and B are N(0,1) drawn from a seeded CPU
generator, quantised per 16-element K block to E2M1 with an E4M3 scale amax/6, scales
in the blocked 128x4 layout, alpha = 1. Steps rotate through several operand sets that
together exceed the 126 MB L2, so B is read from HBM every step.

* ``value``: whole-job TFLOP/s with operands resident in HBM, timed on the device with
  CUDA events around K prepared launches (replayed from a CUDA graph when capture
  works, so that Python launch overhead is not what is measured), max over ranks.
* ``e2e``: the same metric through the operator API with host buffers: every step
  copies the operands from pinned host memory, runs the workload and reads D back.
* ``roofline``: algorithmic bytes of one call / average call duration against the
  measured HBM copy bandwidth of this pool.
* ``cpu_baseline``: the numpy oracle (a port of the reference's torch oracle) timed on
  this host's cores on the same operands; a reported baseline, not the target.
* ``--impl reference``: the reference arm — that same CPU path, alone, on bounded
  samples of the workload.

With N > 1 (launched by torch.distributed.run) every rank holds its own N-shard of a
GEMM whose N is N_gpus x 7168 (weak scaling, no collective on the data path);
``--scaling strong`` splits the workload's own N over the ranks instead.
"""

from __future__ import annotations

import argparse
import json
import os
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
    # name: (kind, shape description)
    "decode": ("dense", dict(m=128, n=7168, k=16384)),
    "square": ("dense", dict(m=8192, n=8192, k=8192)),
    "dual": ("dual", dict(m=256, n=4096, k=7168)),
    "grouped": ("grouped", dict(ms=(40, 96, 128, 256, 384, 512, 768, 1024), n=4096, k=7168)),
}
L2_BYTES = 126 << 20
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one decode-shape launch, from the ncu
# capture summarised in profiles/nvfp4_gemm_decode_m128_n7168_k16384.md.
DECODE_DRAM_TRAFFIC_BYTES = 68_483_328


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


# -- synthetic operands ---------------------------------------------------------------------


def normal_fp4(rows: int, k: int, seed: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """N(0,1) from a CPU generator -> packed E2M1 (rows, k/2, 1) and logical scales."""
    from harness.workloads import quantization as q

    x = torch.randn(rows, k, generator=torch.Generator().manual_seed(seed))
    packed, scales = q.quantize_nvfp4(x.to(device))
    return packed[..., None], scales[..., None]


def make_operand_set(kind: str, shape: dict, index: int, rank: int, device) -> tuple:
    from harness.workloads.nvfp4_gemm import to_task_scales
    from harness.workloads.nvfp4_group_gemm import to_blocked

    base = 1000 * index + 100 * rank
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

    def __init__(self, index: int, interval: float = 0.02):
        self.samples: list[tuple[int, int, int]] = []
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
                self.samples.append((mhz, util, reasons))
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

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        # "Under load": samples taken while NVML reported the GPU at least half busy (all
        # samples if none was: the timed regions are shorter than NVML's averaging window).
        loaded = [s[0] for s in self.samples if s[1] >= 50] or [s[0] for s in self.samples]
        seen = 0
        for _, _, reasons in self.samples:
            seen |= reasons
        names = [name for name, bit in self.REASONS.items() if seen & bit]
        return {"sm_mhz": statistics.median(loaded), "sm_min_mhz": min(loaded),
                "sm_max_mhz": self.max_mhz, "reasons": names, "samples": len(self.samples),
                "samples_under_load": len(loaded)}


# -- CPU baseline (the oracle port) ---------------------------------------------------------


def oracle_dense_call(a, b, sa, sb, rows: slice | None = None):
    """One oracle GEMM on numpy storage-order operands, optionally on a row slice of B."""
    from oracle import nvfp4_oracle as o

    if rows is not None:
        b, sb = b[:, rows], sb[:, rows]
    return o.gemm(a, b, sa, sb, 1.0, np.float16)


def host_dense_operands(shape: dict, seed_base: int = 0):
    """Storage-order numpy operands (packed bytes, logical scale bytes) of the dense
    workload, made on the CPU with the harness quantiser."""
    a, sa = normal_fp4(shape["m"], shape["k"], seed_base + 1, "cpu")
    b, sb = normal_fp4(shape["n"], shape["k"], seed_base + 2, "cpu")

    def store(t):
        t = t.permute(2, 0, 1).contiguous()
        return (t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t).numpy()

    return store(a), store(b), store(sa), store(sb)


def cpu_baseline(kind: str, shape: dict, budget_s: float = 15.0) -> dict:
    """TFLOP/s of the oracle on this host for (a bounded sample of) the workload."""
    if kind != "dense":
        shape = dict(m=128, n=7168, k=16384)
    a, b, sa, sb = host_dense_operands(shape)
    m, n, k = shape["m"], shape["n"], shape["k"]
    probe_rows = min(n, 256)
    t0 = time.perf_counter()
    oracle_dense_call(a, b, sa, sb, slice(0, probe_rows))
    per_row = (time.perf_counter() - t0) / probe_rows
    rows = int(min(n, max(probe_rows, budget_s / 3 / per_row)))
    times = []
    for _ in range(3):
        t0 = time.perf_counter()
        oracle_dense_call(a, b, sa, sb, slice(0, rows))
        times.append(time.perf_counter() - t0)
    best = statistics.median(times)
    return {
        "value": 2.0 * m * rows * k / best / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(),
        "kind": "port",
        "sample": f"numpy oracle (dequantise, FP32 matmul, FP16 cast) on {rows} of {n} rows of B "
                  f"of the m={m} n={n} k={k} GEMM, median of 3, {best:.3f} s each",
    }


def reference_arm(args, kind: str, shape: dict, rank: int) -> None:
    """``--impl reference``: the CPU path alone. Only rank 0 works."""
    if rank != 0:
        return
    if kind != "dense":
        kind, shape = "dense", dict(m=128, n=7168, k=16384)
    a, b, sa, sb = host_dense_operands(shape)
    m, n, k = shape["m"], shape["n"], shape["k"]
    total = args.steps + args.warmup
    t0 = time.perf_counter()
    oracle_dense_call(a, b, sa, sb, slice(0, 128))
    per_row = (time.perf_counter() - t0) / 128
    rows = int(min(n, max(16, 90.0 / total / per_row)))
    rows -= rows % 16 if rows > 16 else 0
    starts = [(i * rows) % max(n - rows, 1) for i in range(total)]
    for i in range(args.warmup):
        oracle_dense_call(a, b, sa, sb, slice(starts[i], starts[i] + rows))
    t0 = time.perf_counter()
    for i in range(args.warmup, total):
        oracle_dense_call(a, b, sa, sb, slice(starts[i], starts[i] + rows))
    elapsed = time.perf_counter() - t0
    value = 2.0 * m * rows * k * args.steps / elapsed / 1e12
    sample = (f"each step: numpy oracle on {rows} of {n} rows of B of the m={m} n={n} k={k} "
              f"GEMM (host operands, no device)")
    line = {
        "impl": "reference", "metric": "nvfp4_gemm_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4", "data": "synthetic",
        "config": {"workload": f"nvfp4_gemm m={m} n={n} k={k} l=1 (CPU oracle, bounded sample)",
                   "sample_rows": rows},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": os.cpu_count(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# -- GPU arm --------------------------------------------------------------------------------


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=2000)
    parser.add_argument("--warmup", type=int, default=200)
    parser.add_argument("--impl", default="native", choices=("native", "reference"))
    parser.add_argument("--workload", default="decode", choices=sorted(WORKLOADS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-graph", action="store_true")
    parser.add_argument("--scaling", default="weak", choices=("weak", "strong"),
                        help="weak: every rank runs the whole shape (global N = ranks x N); "
                             "strong: the shape's N is split over the ranks")
    args = parser.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    kind, shape = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        reference_arm(args, kind, shape, rank)
        return
    global_n = shape.get("n")
    if args.scaling == "strong" and world > 1:
        if kind == "grouped" or shape["n"] % (128 * world):
            raise SystemExit("strong scaling needs a dense or dual shape whose N splits into "
                             "multiples of 128 rows per rank")
        shape = dict(shape, n=shape["n"] // world)

    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    flops, byts = algorithmic_work(kind, shape)
    set_bytes = byts  # operands + output of one set
    sets = max(3, int(2 * L2_BYTES // set_bytes) + 1)
    sets = min(sets, 8 if args.scaling == "weak" else 32)
    cls = workload_class(kind)
    # One workload (and so one native plan with cached tensor maps) per operand set.
    workloads = [cls.from_arch("sm_100a", device=device) for _ in range(sets)]
    operand_sets = [make_operand_set(kind, shape, index, rank, device) for index in range(sets)]
    prepared = [w.prepare(inputs) for w, inputs in zip(workloads, operand_sets)]
    launches = [launch for launch, _ in prepared]
    info = {}
    if kind == "dense":
        info = workloads[0].plan_info(operand_sets[0])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def run_steps(count: int, offset: int = 0):
        for i in range(count):
            launches[(offset + i) % sets]()

    with ClockSampler(local_rank) as clocks:
        run_steps(args.warmup)
        barrier()
        graph = None
        if not args.no_graph:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    run_steps(args.steps)
                graph.replay()  # warm the instantiated graph once
                barrier()
            except Exception as error:  # capture unsupported: time direct launches
                print(f"[bench] CUDA graph capture failed ({error}); timing direct launches",
                      file=sys.stderr)
                graph = None
                barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        if graph is not None:
            graph.replay()
        else:
            run_steps(args.steps)
        stop.record()
        barrier()
        elapsed_ms = start.elapsed_time(stop)
        for w in workloads:
            w.check_status()

        # Direct (non-graph) launches, for the record.
        barrier()
        start.record()
        run_steps(min(args.steps, 500))
        stop.record()
        barrier()
        direct_us = start.elapsed_time(stop) * 1e3 / min(args.steps, 500)

        # End to end through the operator API: pinned host operands in, D out, per step.
        e2e_steps = max(3, min(args.steps, 30))
        host_sets = [tuple(t.cpu().pin_memory() for t in inputs) for inputs in operand_sets[:2]]
        # Device staging tensors in the operands' memory layout.
        staging = [tuple(torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=device)
                         for t in operand_sets[0]) for _ in range(2)]
        host_out = None
        h2d = sum(t.numel() * t.element_size() for t in host_sets[0])

        def e2e_step(i: int):
            nonlocal host_out
            src, dst = host_sets[i % 2], staging[i % 2]
            for s, d in zip(src, dst):
                d.copy_(s, non_blocking=True)
            outputs = workloads[i % 2].run(dst)
            outs = [o.to("cpu", non_blocking=True) for o in outputs]
            torch.cuda.current_stream().synchronize()
            host_out = outs
            return sum(o.numel() * o.element_size() for o in outputs)

        d2h = e2e_step(0)
        e2e_step(1)
        barrier()
        start.record()
        for i in range(e2e_steps):
            e2e_step(i)
        stop.record()
        barrier()
        e2e_ms = start.elapsed_time(stop)

    times = torch.tensor([elapsed_ms, e2e_ms, direct_us], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, direct_us = (float(v) for v in times.tolist())

    if rank == 0:
        per_call_us = elapsed_ms * 1e3 / args.steps
        value = world * flops * args.steps / (elapsed_ms * 1e-3) / 1e12
        e2e_value = world * flops * e2e_steps / (e2e_ms * 1e-3) / 1e12
        peak, peak_kind = measured_hbm_peak()
        achieved = byts / (per_call_us * 1e-6) / 1e9
        bound = "tensor" if args.workload == "square" else "hbm"
        if bound == "hbm":
            roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                        "frac": achieved / peak,
                        "traffic": DECODE_DRAM_TRAFFIC_BYTES if args.workload == "decode" else None,
                        "peak_source": f"{peak_kind} HBM copy bandwidth",
                        "algorithmic_bytes_per_launch": byts}
        else:
            tf = flops / (per_call_us * 1e-6) / 1e12
            peak_tf = 9000.0
            # The rate at which this GPU issues block-scaled FP4 MMAs with nothing else
            # running (the library's own microbenchmark, after the timed region).
            from harness import native
            issue_tf = native.measure_mma_peak(local_rank, 4096)
            roofline = {"bound": "tensor", "achieved": tf, "peak": peak_tf, "unit": "TFLOP/s",
                        "frac": tf / peak_tf, "traffic": None,
                        "peak_source": "nominal dense FP4",
                        "measured_mma_issue_tflops": issue_tf,
                        "frac_of_measured_mma_issue": tf / issue_tf,
                        "algorithmic_flops_per_launch": flops}
        line = {
            "metric": "nvfp4_gemm_tflops", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": elapsed_ms / args.steps, "us_per_call": per_call_us,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "nvfp4", "data": "synthetic",
            "config": {
                "workload": f"nvfp4 {kind} GEMM {shape} l=1, fp16 out, per GPU"
                            + (f" (global n = {world} x {shape.get('n')})"
                               if world > 1 and args.scaling == "weak" else "")
                            + (f" (global n = {global_n} split over {world} ranks)"
                               if world > 1 and args.scaling == "strong" else ""),
                "operand_sets": sets, "l2": f"{sets} operand sets of {set_bytes / 2**20:.0f} MiB "
                                            "rotate, larger than the 126 MB L2 together",
                "timing": "cuda_graph_replay" if graph is not None else "direct_launches",
                "direct_launch_us_per_call": direct_us, "plan": info,
                "sharding": "each rank owns an N-shard; no collective on the data path",
            },
            "roofline": roofline,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": args.steps,
            "clocks": clocks.summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(kind, shape)
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
