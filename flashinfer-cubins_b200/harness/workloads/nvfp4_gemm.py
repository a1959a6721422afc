"""Batched NVFP4 block-scaled GEMM: ``D[:, :, l] = alpha * (A*SFA) @ (B*SFB)^T``.

Workload ``nvfp4_gemm`` of the reference (``harness/workloads/nvfp4_gemm.py:511-600``)
on the B200-native kernel. Inputs ``(a, b, sfa, sfb, alpha)``:

* ``a [m, k/2, l]`` and ``b [n, k/2, l]``: packed E2M1 ``uint8`` (low nibble first,
  K contiguous, batch outermost in memory);
* ``sfa``/``sfb``: UE4M3 scales in the blocked layout, as the ``float8_e4m3fn`` view of
  shape ``(32, 4, ceil(rows/128), 4, ceil(k/64), l)`` whose memory is the contiguous
  ``(l, ceil(rows/128), ceil(k/64), 32, 4, 4)`` array (``to_task_scales``);
* ``alpha``: one FP32 element on the device, read by the kernel's epilogue, so a value
  written by an earlier stream-ordered operation is seen without a host sync.

Output ``(d,)``: FP16 ``[m, n, l]``, batch outermost in memory. Requires
``k % 32 == 0`` (16-byte rows of packed operands) and ``n % 8 == 0`` (16-byte rows of
D). Where the reference rebuilds a 3,072-byte CUTLASS ``Params`` with nine tensor maps
per launch (``nvfp4_gemm.py:198-387``), this workload keeps a plan per problem shape
in the native library and passes six pointers.
"""

from __future__ import annotations

from collections.abc import Sequence
from typing import Any

import torch

from .. import native
from ..registry import register
from ..throughput import gemm_case, model_case, upstream_case
from ..workload import CaseSpec, Workload
from .quantization import (
    SF_COLS,
    SF_ROWS,
    SF_VEC,
    ceil_div,
    empty_fp4_output,
    fp4_matmul,
    from_blocked_scales,
    make_fp4,
    shuffle_rows,
    to_blocked_scales,
)

INT32_MAX = (1 << 31) - 1
# The NVIDIA task's input distributions: every E2M1 byte, integer scales 0..3.
TASK_DIST = {"values": "full", "scales": "int0_3"}
# Shapes (m, n, k, l) of the NVIDIA nvfp4_gemm task: its test lines (seed 1111) and
# its benchmark lines (resources/nvfp4_gemm/task.yml:43-58 in the reference).
TASK_TESTS = (
    (128, 256, 256, 1), (128, 1536, 7168, 1), (128, 3072, 1536, 1), (256, 7168, 256, 1),
    (256, 7168, 2048, 1), (2304, 4608, 7168, 1), (384, 7168, 2304, 1), (512, 512, 7168, 1),
    (512, 4096, 512, 1), (512, 1536, 7168, 1),
)
TASK_BENCHMARKS = ((128, 7168, 16384, 1), (128, 4096, 7168, 1), (128, 7168, 2048, 1))
TASK_SEED = 1111
BLOCKED_ORDER = (5, 2, 4, 0, 1, 3)  # permutation that makes a task-view scale tensor contiguous


class TaskLines:
    """The test and benchmark lines of one NVIDIA task as this package records them. The
    reference keeps a path to the task's ``task.yml`` under this name (``TASK``) and parses
    it on every use (``nvfp4_gemm.py:72,481-491`` there); here the lines are tables in the
    workload modules and ``task_shapes`` turns them into the same list of dicts."""

    def __init__(self, name: str, tests, benchmarks, seed: int = TASK_SEED):
        self.name, self.tests, self.benchmarks, self.seed = name, tuple(tests), tuple(benchmarks), seed


TASK = TaskLines("nvfp4_gemm", TASK_TESTS, TASK_BENCHMARKS)


def task_shapes(task: TaskLines, section: str) -> list[dict[str, Any]]:
    """The ``tests`` or ``benchmarks`` entries of a task: dicts with ``m, n, k, l`` (lists
    per group for the grouped task) and the task's ``seed``."""
    if section not in ("tests", "benchmarks"):
        raise ValueError(f"unknown section {section!r}")
    entries = []
    for line in getattr(task, section):
        if line and isinstance(line[0], (tuple, list)):  # grouped: (ms, ns, ks)
            ms, ns, ks = line
            entry = {"m": list(ms), "n": list(ns), "k": list(ks), "g": len(ms)}
        else:
            entry = dict(zip(("m", "n", "k", "l"), line))
        entry["seed"] = task.seed
        entries.append(entry)
    return entries


def fake_encode(*args, **kwargs):
    """The reference's deterministic stand-in for ``cuTensorMapEncodeTiled``, which its
    tests use to compare CUTLASS ``Params`` bytes (``nvfp4_gemm.py:78-102`` there). This
    package builds no ``Params`` struct, so there is nothing for it to encode."""
    raise NotImplementedError("no CUTLASS Params are built here; tensor maps are encoded "
                              "inside the native library")


def blocked_scale_shape(rows: int, k: int, batches: int) -> tuple[int, ...]:
    """Shape of the task's permuted view of the blocked scales of a rows x k operand."""
    return (32, 4, ceil_div(rows, SF_ROWS), SF_COLS, ceil_div(ceil_div(k, SF_VEC), SF_COLS), batches)


def to_task_scales(scales: torch.Tensor) -> torch.Tensor:
    """Logical ``(rows, cols, l)`` scales -> the ``(32, 4, rb, 4, cb, l)`` view of their
    blocked layout."""
    return to_blocked_scales(scales).permute(3, 4, 1, 5, 2, 0)


def from_task_scales(blocked: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Inverse of ``to_task_scales``: logical ``(rows, cols, l)`` scales."""
    return from_blocked_scales(blocked.permute(*BLOCKED_ORDER), rows, cols)


def check_layout(tensor, shape, dtype, order) -> None:
    """``tensor`` has ``shape``/``dtype`` and ``tensor.permute(*order)`` is contiguous."""
    if tuple(tensor.shape) != tuple(shape) or tensor.dtype != dtype:
        raise ValueError(
            f"expected {dtype} {tuple(shape)}, got {tensor.dtype} {tuple(tensor.shape)}"
        )
    if not tensor.permute(*order).is_contiguous():
        raise ValueError(f"{dtype} {tuple(shape)} operand has an unsupported layout")


def fp4_case(m, n, k, l=1, *, seed, suite="smoke", **extra) -> CaseSpec:  # noqa: E741
    """A plain ``(m, n, k, l)`` case; ``extra`` holds non-default distributions
    (``values``/``scales``) and ``alpha``, which also appear in the case's name."""
    params = dict(m=m, n=n, k=k, l=l, **extra)
    return CaseSpec("_".join(f"{key}{value}" for key, value in params.items()), params, seed, suite)


def task_cases(shapes, name: str, **extra) -> list[CaseSpec]:
    """One smoke case per distinct task test shape, with the task's seed. ``shapes`` is a
    sequence of ``(m, n, k, l)`` or a ``TaskLines`` (its test lines)."""
    if isinstance(shapes, TaskLines):
        shapes = shapes.tests
    cases: dict[str, CaseSpec] = {}
    for index, (m, n, k, l) in enumerate(shapes):  # noqa: E741
        label = f"task_m{m}_n{n}_k{k}_l{l}"
        if label not in cases:
            cases[label] = upstream_case(
                label, dict(m=m, n=n, k=k, l=l, **extra), f"{name}/task.yml::tests[{index}]",
                seed=TASK_SEED,
            )
    return list(cases.values())


class LaunchConfig:
    """A validated dense launch: the problem and the six device addresses."""

    def __init__(self, problem, pointers):
        self.problem = problem  # (m, n, k, l)
        self.pointers = pointers  # (a, b, sfa, sfb, alpha, d)
        self.keepalive: list[Any] = []


class Fp4GemmWorkload(Workload):
    """Host side shared by ``nvfp4_gemm`` (FP16 D) and ``nvfp4_dual_gemm_gemm`` (FP32
    D): operand checks, plan lookup and launch. Subclasses set ``OUT_DTYPE`` and
    implement ``operands`` plus the data side of the contract. The counterpart of the
    reference's ``CutlassFp4Gemm`` (``nvfp4_gemm.py:150-460``)."""

    OUT_DTYPE: torch.dtype = torch.float16
    entry_point = "nvfp4_gemm_launch"

    # -- validation -------------------------------------------------------------------

    def build_params(self, m, n, k, l, a, b, sfa, sfb, alpha, d) -> LaunchConfig:  # noqa: E741
        """Check a problem and its device addresses the way the reference's builder
        does (``nvfp4_gemm.py:226-231``) and return the launch description."""
        out_bytes = torch.empty((), dtype=self.OUT_DTYPE).element_size()
        if min(m, n, k, l) < 1 or k % 32 or (n * out_bytes) % 16:
            raise ValueError(f"unsupported problem m={m} n={n} k={k} l={l}")
        if l > 1 and max(m * k, n * k, m * n) > INT32_MAX:
            raise ValueError("batch strides exceed the 32-bit range")
        if any(p % 16 for p in (a, b, sfa, sfb, d)) or alpha % 4:
            raise ValueError("misaligned operand address")
        return LaunchConfig((m, n, k, l), (a, b, sfa, sfb, alpha, d))

    def operands(self, inputs: tuple, out: torch.Tensor) -> tuple[int, int, int, int]:
        """Check ``inputs`` (a, b, sfa, sfb, alpha) and ``out``; return (m, n, k, l)."""
        raise NotImplementedError

    def launch_config(self, inputs: tuple, out: torch.Tensor) -> LaunchConfig:
        """Check the tensors and describe the launch of ``inputs`` into ``out``."""
        m, n, k, l = self.operands(inputs, out)  # noqa: E741
        a, b, sfa, sfb, alpha = inputs
        if tuple(alpha.shape) != (1,) or alpha.dtype != torch.float32:
            raise ValueError("alpha must be one FP32 element")
        if any(t.device != out.device for t in inputs):
            raise ValueError("operands must be on one device")
        config = self.build_params(
            m, n, k, l, a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
            alpha.data_ptr(), out.data_ptr(),
        )
        config.keepalive = [inputs, out]
        return config

    # -- launch -----------------------------------------------------------------------

    def _plan(self, problem):
        out_kind = {torch.float16: native.OUT_F16, torch.bfloat16: native.OUT_BF16}.get(
            self.OUT_DTYPE, native.OUT_F32)
        return self.plan_for(
            ("dense", out_kind, problem),
            lambda: native.Plan.dense(self.device_index(), out_kind, *problem),
        )

    def _launch(self, config: LaunchConfig, entry=None) -> None:
        """Launch on the current stream with ``entry`` = (plan, workspace), or with the
        plan and workspace cached for that stream."""
        with self._lock, torch.cuda.device(self.device):
            plan, workspace = entry or self._plan(config.problem)
            plan.launch_dense(*config.pointers, workspace.data_ptr(), self.stream_handle())

    def plan_info(self, inputs: tuple) -> dict:
        """What the native plan for these inputs decided (tile, schedule, grid)."""
        (out,) = self.allocate_outputs(inputs)
        plan, _ = self._plan(self.launch_config(inputs, out).problem)
        return plan.info()

    def allocate_outputs(self, inputs):
        return (empty_fp4_output(inputs[0], inputs[1], self.OUT_DTYPE),)

    def run(self, inputs):
        self._check_supported()
        (out,) = self.allocate_outputs(inputs)
        self._launch(self.launch_config(inputs, out))
        return (out,)

    def prepare(self, inputs):
        self._check_supported()
        outputs = self.allocate_outputs(inputs)
        config = self.launch_config(inputs, outputs[0])
        entry = self._plan(config.problem)  # plan and workspace exist before the timed calls

        def launch() -> tuple:
            self._launch(config, entry)
            return outputs

        return launch, outputs


CutlassFp4Gemm = Fp4GemmWorkload  # the reference's name for this base class


@register(name="nvfp4_gemm", supported_arches=("sm_100a",))
class NVFP4GEMM(Fp4GemmWorkload):
    """Batched NT NVFP4 GEMM with UE4M3/16 block scales, alpha and FP16 output.

    Smoke cases (the reference's, ``nvfp4_gemm.py:532-544``; default distribution the
    task's): partial M, N and K tiles (k = 96 is less than one 256-wide k-tile and has
    6 scale columns, a partial scale atom), batches l = 2 and 3, a nine-k-tile loop
    ending in a partial tile, 195 output tiles (more than 148 SMs), zero (``int0_3``),
    subnormal (``unit``) and three-binade (``uniform``) scales, alpha != 1; then every
    NVIDIA task test line and the two FlashInfer ``mm_fp4`` shapes (``UPSTREAM``).
    """

    OUT_DTYPE = torch.float16

    SMOKE = (
        fp4_case(128, 128, 128, seed=1),
        fp4_case(128, 256, 256, 2, seed=2),
        fp4_case(256, 128, 512, seed=3),
        fp4_case(200, 136, 96, seed=4),
        fp4_case(200, 136, 96, seed=5, scales="uniform"),
        fp4_case(300, 264, 384, 3, seed=6, alpha=0.0123),
        fp4_case(129, 1032, 2080, 2, seed=7),
        fp4_case(640, 1544, 768, 3, seed=8),
        fp4_case(192, 520, 1024, 2, seed=9, scales="unit"),
        fp4_case(17, 4104, 4096, seed=10, scales="uniform", alpha=0.37),
        fp4_case(1000, 264, 512, seed=11, values="restricted", scales="int1_2"),
    )

    def operands(self, inputs, out):
        a, b, sfa, sfb, _ = inputs
        if a.dim() != 3 or b.dim() != 3:
            raise ValueError("A and B must be (rows, k/2, l)")
        m, half_k, l = a.shape  # noqa: E741
        n, k = b.shape[0], 2 * half_k
        check_layout(a, (m, half_k, l), torch.uint8, (2, 0, 1))
        check_layout(b, (n, half_k, l), torch.uint8, (2, 0, 1))
        check_layout(sfa, blocked_scale_shape(m, k, l), torch.float8_e4m3fn, BLOCKED_ORDER)
        check_layout(sfb, blocked_scale_shape(n, k, l), torch.float8_e4m3fn, BLOCKED_ORDER)
        check_layout(out, (m, n, l), self.OUT_DTYPE, (2, 0, 1))
        return m, n, k, l

    # -- workload contract ------------------------------------------------------------

    def get_cases(self):
        cases = [*self.SMOKE, *task_cases(TASK_TESTS, "nvfp4_gemm")]
        for index, (test, (m, n, k), alpha) in enumerate(UPSTREAM):
            cases.append(upstream_case(
                f"mm_fp4_m{m}_n{n}_k{k}", dict(m=m, n=n, k=k, l=1, alpha=alpha), test, seed=index,
            ))
        return cases + throughput_cases()

    def get_inputs(self, case):
        p, g = case.params, self.generator(case)
        dist = {key: p.get(key, TASK_DIST[key]) for key in TASK_DIST}
        a, sa = make_fp4(self, g, p["m"], p["k"], p["l"], **dist)
        b, sb = make_fp4(self, g, p["n"], p["k"], p["l"], **dist)
        alpha = torch.full((1,), p.get("alpha", 1.0), device=self.device)
        return a, b, to_task_scales(sa), to_task_scales(sb), alpha

    def get_reference(self, inputs):
        a, b, sfa, sfb, alpha = inputs
        cols = 2 * a.shape[1] // SF_VEC
        sa = from_task_scales(sfa, a.shape[0], cols)
        sb = from_task_scales(sfb, b.shape[0], cols)
        return (fp4_matmul(a, b, sa, sb, alpha=float(alpha.item()), out_dtype=self.OUT_DTYPE),)

    def validate(self, ref, impl):
        # The NVIDIA task's tolerance. Kernel and reference both add exact products in
        # FP32 and round once to FP16 after the same FP32 multiplication by alpha:
        # identical outputs for integer scales, at most one FP16 ulp apart otherwise.
        self.assert_close(ref, impl, rtol=1e-3, atol=1e-3)


@register(name="nvfp4_gemm_bf16", supported_arches=("sm_100a",))
class NVFP4GEMMBf16(NVFP4GEMM):
    """The same GEMM with BF16 output, the output type FlashInfer's ``mm_fp4`` asks for
    (the reference's ``tests/gemm/test_mm_fp4.py`` line quoted in ``UPSTREAM`` runs its m = 1
    case in BF16). Not a workload of the reference: its NVFP4 GEMM cubins write FP16. A few
    smoke cases only; same inputs, reference rounded to BF16, BF16's tolerance."""

    OUT_DTYPE = torch.bfloat16

    SMOKE = (
        fp4_case(128, 128, 128, seed=1),
        fp4_case(200, 136, 96, seed=5, scales="uniform"),
        fp4_case(300, 264, 384, 3, seed=6, alpha=0.0123),
        fp4_case(1, 128, 512, seed=12, alpha=0.0123),
        fp4_case(1000, 264, 512, seed=11, values="restricted", scales="int1_2"),
    )

    def get_cases(self):
        return list(self.SMOKE)

    def validate(self, ref, impl):
        # One BF16 rounding of the same FP32 value on both sides: equal for integer scales,
        # at most one BF16 ulp (2^-8 relative) apart otherwise.
        self.assert_close(ref, impl, rtol=8e-3, atol=1e-3)


@register(name="nvfp4_gemm_bf16_shuffled", supported_arches=("sm_100a",))
class NVFP4GEMMBf16Shuffled(NVFP4GEMMBf16):
    """``nvfp4_gemm_bf16`` on weights in the layout FlashInfer's ``mm_fp4`` takes with its
    trtllm backend: the rows of B and of B's scales permuted inside blocks of 32 rows
    (``quantization.shuffle_rows``; the reference prepares such weights in
    ``harness/workloads/batched_gemm/trtllm.py:257-288``), BF16 output in logical column
    order. Inputs ``(a, b_shuffled, sfa, sfb_shuffled, alpha)`` with the shapes and layouts
    of ``nvfp4_gemm``; n a multiple of the shuffle block. Not a workload of the reference,
    whose kernels for this layout are the prebuilt ``cubins/gemm/Gemm_Bfloat16_E2m1E2m1_*``."""

    SHUFFLE_BLOCK = 32

    SMOKE = (
        fp4_case(128, 128, 128, seed=1),
        fp4_case(200, 160, 96, seed=5, scales="uniform"),
        fp4_case(300, 288, 384, 3, seed=6, alpha=0.0123),
        fp4_case(1, 128, 512, seed=12, alpha=0.0123),
        fp4_case(16, 7168, 2048, seed=13),
        fp4_case(1000, 256, 512, seed=11, values="restricted", scales="int1_2"),
    )

    def shuffle_index(self, n: int) -> torch.Tensor:
        return shuffle_rows(n, self.SHUFFLE_BLOCK)

    def get_inputs(self, case):
        a, b, sfa, sfb, alpha = super().get_inputs(case)
        n, cols = b.shape[0], 2 * b.shape[1] // SF_VEC
        idx = self.shuffle_index(n).to(b.device)
        logical = from_task_scales(sfb, n, cols)
        b_physical = b[idx].permute(2, 0, 1).contiguous().permute(1, 2, 0)
        return a, b_physical, sfa, to_task_scales(logical[idx].contiguous()), alpha

    def get_reference(self, inputs):
        a, b_physical, sfa, sfb_physical, alpha = inputs
        n, cols = b_physical.shape[0], 2 * b_physical.shape[1] // SF_VEC
        idx = self.shuffle_index(n).to(b_physical.device)
        b = torch.empty_like(b_physical)
        b[idx] = b_physical
        physical = from_task_scales(sfb_physical, n, cols)
        logical = torch.empty_like(physical)
        logical[idx] = physical
        return super().get_reference((a, b, sfa, to_task_scales(logical), alpha))

    def _plan(self, problem):
        return self.plan_for(
            ("dense_shuffled", self.SHUFFLE_BLOCK, problem),
            lambda: native.Plan.dense_shuffled(self.device_index(), native.OUT_BF16, *problem,
                                               self.SHUFFLE_BLOCK),
        )


# FlashInfer's mm_fp4 tests that run this kernel family (cutlass backend, nvfp4, 128x4
# scale layout) with the alpha they pass; the m = 1 case asks for BF16 there and runs
# with FP16 output here.
UPSTREAM = (
    ("tests/gemm/test_mm_fp4.py::test_mm_fp4[1-128-512-bfloat16-cutlass]", (1, 128, 512), 0.0123),
    ("tests/gemm/test_mm_fp4.py::test_mm_fp4[31-256-256-float16-cutlass]", (31, 256, 256), 0.0123),
)

THROUGHPUT = "nvfp4_gemm"

# (model, m values): every linear layer of each model from decode to 16k-token prefill.
MODEL_PLAN = (
    ("deepseek_v3", (1, 16, 4096, 16384)),
    ("llama3_70b", (1, 16, 4096, 16384)),
    ("llama3_405b", (8, 8192)),
    ("qwen3_235b_a22b", (8, 8192)),
    ("gpt_oss_120b", (8, 8192)),
    ("llama4_maverick", (8, 8192)),
)


def model_gemm_cases(plan, prefix=""):
    """``model_case`` (m, n, k, l=1) for every linear layer of each planned model."""
    from ..models import MODELS

    return [
        model_case(f"{prefix}{model}_{layer}_m{m}", dict(m=m, n=n, k=k, l=1), model, layer)
        for model, ms in plan
        for layer, (n, k) in MODELS[model].linear_shapes().items()
        for m in ms
    ]


def official_source(name: str) -> dict:
    return {
        "kind": "official_shape",
        "snapshot": f"resources/{name}/task.yml",
        "url": "https://github.com/gpu-mode/reference-kernels/blob/main/problems/nvidia/"
               f"{name}/task.yml",
        "selection": "All benchmark (not just test) shapes; generated using the harness "
                     "quantization contract.",
    }


def throughput_cases():
    """Throughput cases: the task's benchmark lines, then the linear layers of
    ``MODEL_PLAN`` without repeating a shape."""
    cases = [gemm_case(THROUGHPUT, shape, official_source(THROUGHPUT)) for shape in TASK_BENCHMARKS]
    seen = {tuple(c.params.values()) for c in cases}
    for case in model_gemm_cases(MODEL_PLAN):
        key = tuple(case.params.values())
        if key not in seen:
            seen.add(key)
            cases.append(case)
    return cases
