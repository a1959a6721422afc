"""Grouped NVFP4 block-scaled GEMM: every group in one persistent launch.

Workload ``nvfp4_group_gemm`` of the reference
(``harness/workloads/nvfp4_group_gemm.py:187-665``). For each group g,
``D_g[m_g, n_g] = (A_g * SFA_g) @ (B_g * SFB_g)^T`` with packed E2M1 ``A_g [m_g, k_g/2]``
and ``B_g [n_g, k_g/2]`` (K contiguous), UE4M3 scales per 16 K elements in the blocked
layout ``(ceil(rows/128), ceil(k/64), 32, 4, 4)`` and FP16 row-major ``D_g``. Inputs are
four tensors per group in the order ``a_g, b_g, sfa_g, sfb_g``; outputs one tensor per
group. Requires ``k % 32 == 0``, ``n % 8 == 0`` and at least one row per group.

The reference hands CUTLASS per-group device arrays and lets the kernel rewrite its
TMA descriptors per group on the device (``nvfp4_group_gemm.py:250-501``). Here the
host knows every shape, so ``launch_config`` encodes two tensor maps per group once
(``nvfp4_group_gemm_bind``), copies them with the group table into the workspace in
one stream-ordered transfer, and the kernel only walks the table; tiles of all groups
share one (tile, k-tile) numbering so that stream-K can balance ragged groups.
"""

from __future__ import annotations

import random
from typing import Any

import torch

from .. import native
from ..registry import register
from ..throughput import model_case, skewed_lengths, upstream_case
from ..workload import CaseSpec, Workload
from .nvfp4_gemm import TaskLines, fake_encode, official_source
from .quantization import ceil_div, fp4_matmul, from_blocked_scales, make_fp4, to_blocked_scales

SF_VEC = 16  # K elements per scale factor
SF_BLOCK_ROWS, SF_BLOCK_COLS = 128, 4  # rows x scale columns per 512-byte atom
# The NVIDIA task's distributions: 0xBB-masked E2M1 bytes, integer scales 1..2.
TASK_DIST = {"values": "restricted", "scales": "int1_2"}
TASK_SEED = 1111
# Groups (m, n, k) of the NVIDIA nvfp4_group_gemm task: test lines and benchmark lines
# (resources/nvfp4_group_gemm/task.yml:47-63 in the reference), as (m list, n list, k list).
TASK_TESTS = (
    ((96, 128), (128, 256), (256, 512)),
    ((256, 72), (512, 384), (256, 256)),
    ((128, 128), (128, 256), (512, 256)),
    ((80, 128, 256), (384, 256, 128), (256, 512, 256)),
    ((64, 72, 96), (128, 384, 512), (512, 512, 256)),
    ((64, 256, 128), (768, 128, 256), (512, 256, 512)),
    ((128, 128, 64), (256, 512, 512), (768, 256, 768)),
    ((128, 128, 128, 128), (128, 128, 128, 128), (512, 256, 512, 256)),
    ((40, 56, 384, 512), (512, 384, 256, 128), (256, 256, 256, 256)),
    ((512, 384, 256, 128), (256, 256, 256, 256), (512, 768, 512, 768)),
)
TASK_BENCHMARKS = (
    ((80, 176, 128, 72, 64, 248, 96, 160), (4096,) * 8, (7168,) * 8),
    ((40, 76, 168, 72, 164, 148, 196, 160), (7168,) * 8, (2048,) * 8),
    ((192, 320), (3072, 3072), (4096, 4096)),
    ((128, 384), (4096, 4096), (1536, 1536)),
)


TASK = TaskLines("nvfp4_group_gemm", TASK_TESTS, TASK_BENCHMARKS, TASK_SEED)
# The reference names here the per-group device arrays of a CUTLASS grouped launch
# (``nvfp4_group_gemm.py:250-315`` there). The native library keeps one table of problems
# and two tensor maps per group in its workspace instead, so there are none to list.
ARRAYS: tuple[str, ...] = ()


def fast_divmod_u64(divisor: int) -> tuple[int, int, int, int]:
    """``(divisor, multiplier, shift, round_up)`` with which an unsigned 64-bit division is
    a multiply-high and a shift: ``x // divisor == (((x + round_up) * multiplier) >> 64)
    >> shift`` when ``multiplier`` is non-zero, ``x >> shift`` when it is zero (powers of
    two). The reference packs such constants into its grouped kernel's scheduler parameters
    (``nvfp4_group_gemm.py:113-137`` there); the persistent scheduler of this package
    divides on the device and does not use them, the function is kept for callers that do.
    With ``shift = floor(log2(divisor))`` the multiplier ``ceil(2**(64 + shift) / divisor)``
    lies in ``[2**63, 2**64)`` and the quotient is exact for every ``x < 2**63``."""
    if divisor < 1:
        raise ValueError("divisor must be positive")
    shift = divisor.bit_length() - 1
    if divisor == 1 << shift:
        return divisor, 0, shift, 0
    multiplier = -(-(1 << (64 + shift)) // divisor)
    return divisor, multiplier, shift, 0


def blocked_shape(rows: int, k: int) -> tuple[int, int, int, int, int]:
    """Shape of one group's blocked scale tensor for (rows, k/16) scales."""
    return (ceil_div(rows, SF_BLOCK_ROWS), ceil_div(k // SF_VEC, SF_BLOCK_COLS), 32, 4,
            SF_BLOCK_COLS)


def to_blocked(scales: torch.Tensor) -> torch.Tensor:
    """Logical (rows, cols) scales -> one group's zero-padded ``(rb, cb, 32, 4, 4)``."""
    return to_blocked_scales(scales[..., None])[0]


def from_blocked(blocked: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Inverse of ``to_blocked`` (drops the padding)."""
    return from_blocked_scales(blocked[None], rows, cols)[..., 0]


class LaunchConfig:
    """A validated grouped launch: the problems and the five pointer lists."""

    def __init__(self, problems, pointers):
        self.problems = problems  # ((m, n, k), ...)
        self.pointers = pointers  # (a[], b[], sfa[], sfb[], d[])
        self.plan: native.Plan | None = None
        self.workspace: torch.Tensor | None = None
        self.keepalive: list[Any] = []


@register(name="nvfp4_group_gemm", supported_arches=("sm_100a",))
class NVFP4GroupGEMM(Workload):
    """Ragged grouped NVFP4 GEMM, one FP16 output per group, one launch.

    Cases: ``SMOKE`` (see its comment), every NVIDIA task test line (task distribution
    and seed) and benchmark line, and MoE expert GEMMs with skewed per-expert token
    counts (``MOE_PLAN``)."""

    rtol, atol = 1e-3, 1e-3
    entry_point = "nvfp4_group_gemm_launch"

    @staticmethod
    def groups_of(inputs: tuple) -> list[tuple[torch.Tensor, ...]]:
        if not inputs or len(inputs) % 4:
            raise ValueError("expected four tensors (a, b, sfa, sfb) per group")
        return [tuple(inputs[i:i + 4]) for i in range(0, len(inputs), 4)]

    @staticmethod
    def problem_of(group: tuple[torch.Tensor, ...]) -> tuple[int, int, int]:
        a, b = group[:2]
        return a.shape[0], b.shape[0], a.shape[1] * 2

    def launch_config(self, inputs: tuple, outputs: tuple) -> LaunchConfig:
        """Check every tensor (shape, dtype, contiguity, device, 16-byte alignment) and
        describe the launch of ``inputs`` into ``outputs`` (one FP16 tensor per group).
        Pure host work: nothing native is called."""
        groups = self.groups_of(inputs)
        if len(outputs) != len(groups):
            raise ValueError("expected one output per group")
        device = outputs[0].device
        problems = []
        pointers: tuple[list[int], ...] = ([], [], [], [], [])
        for (a, b, sfa, sfb), out in zip(groups, outputs):
            if a.dim() != 2 or b.dim() != 2:
                raise ValueError("A and B must be (rows, k/2)")
            m, n, k = self.problem_of((a, b))
            if m < 1 or n % 8 or k % 32 or k < 32:
                raise ValueError(f"unsupported group m={m} n={n} k={k}")
            wanted = (
                (a, (m, k // 2), torch.uint8),
                (b, (n, k // 2), torch.uint8),
                (sfa, blocked_shape(m, k), torch.float8_e4m3fn),
                (sfb, blocked_shape(n, k), torch.float8_e4m3fn),
                (out, (m, n), torch.float16),
            )
            for slot, (tensor, shape, dtype) in zip(pointers, wanted):
                if tuple(tensor.shape) != shape or tensor.dtype != dtype:
                    raise ValueError(
                        f"expected {dtype} {shape}, got {tensor.dtype} {tuple(tensor.shape)}"
                    )
                if not tensor.is_contiguous() or tensor.device != device:
                    raise ValueError("operands must be contiguous and on one device")
                if tensor.data_ptr() % 16:
                    raise ValueError("operands must be 16-byte aligned")
                slot.append(tensor.data_ptr())
            problems.append((m, n, k))
        config = LaunchConfig(tuple(problems), pointers)
        config.keepalive = [inputs, outputs]
        return config

    def _bind(self, config: LaunchConfig) -> None:
        """Plan for these shapes (cached) and a bound workspace for these pointers."""
        with self._lock, torch.cuda.device(self.device):
            plan, _ = self.plan_for(
                ("group", config.problems),
                lambda: native.Plan.grouped(self.device_index(), config.problems),
            )
            # Each bound launch owns a workspace: the group table inside it holds this
            # launch's pointers.
            workspace = torch.empty(max(plan.workspace_bytes(), 256), dtype=torch.uint8,
                                    device=self.device)
            plan.init_workspace(workspace.data_ptr(), self.stream_handle())
            plan.bind_groups(*config.pointers, workspace.data_ptr(), self.stream_handle())
            config.plan, config.workspace = plan, workspace

    def plan_info(self, inputs: tuple) -> dict:
        """What the native plan for these inputs decided (tile, schedule, grid)."""
        config = self.launch_config(inputs, self.allocate_outputs(inputs))
        with self._lock, torch.cuda.device(self.device):
            plan, _ = self.plan_for(
                ("group", config.problems),
                lambda: native.Plan.grouped(self.device_index(), config.problems),
            )
        return plan.info()

    def _launch(self, config: LaunchConfig) -> None:
        with self._lock, torch.cuda.device(self.device):
            config.plan.launch_groups(config.workspace.data_ptr(), self.stream_handle())

    # -- workload contract ------------------------------------------------------------

    def get_cases(self):
        return [*SMOKE, *task_group_cases(), *throughput_cases()]

    def get_inputs(self, case):
        p, g = case.params, self.generator(case)
        dist = {key: p.get(key, TASK_DIST[key]) for key in TASK_DIST}
        tensors = []
        for m, n, k in p["groups"]:
            a, sa = make_fp4(self, g, m, k, 1, **dist)
            b, sb = make_fp4(self, g, n, k, 1, **dist)
            tensors += [a[..., 0], b[..., 0], to_blocked(sa[..., 0]), to_blocked(sb[..., 0])]
        return tuple(tensors)

    def get_reference(self, inputs):
        outputs = []
        for a, b, sfa, sfb in self.groups_of(inputs):
            m, n, k = self.problem_of((a, b))
            sa = from_blocked(sfa, m, k // SF_VEC)
            sb = from_blocked(sfb, n, k // SF_VEC)
            d = fp4_matmul(a[..., None], b[..., None], sa[..., None], sb[..., None],
                           out_dtype=torch.float16)
            outputs.append(d[..., 0])
        return tuple(outputs)

    def allocate_outputs(self, inputs):
        return tuple(
            torch.empty((a.shape[0], b.shape[0]), device=a.device, dtype=torch.float16)
            for a, b, _, _ in self.groups_of(inputs)
        )

    def run(self, inputs):
        self._check_supported()
        outputs = self.allocate_outputs(inputs)
        config = self.launch_config(inputs, outputs)
        self._bind(config)
        self._launch(config)
        return outputs

    def prepare(self, inputs):
        self._check_supported()
        outputs = self.allocate_outputs(inputs)
        config = self.launch_config(inputs, outputs)
        self._bind(config)

        def launch() -> tuple:
            self._launch(config)
            return outputs

        return launch, outputs

    def validate(self, ref, impl):
        # FP32 accumulation of exactly representable products in both; outputs differ
        # by at most one FP16 rounding step (the NVIDIA task's tolerance).
        self.assert_close(ref, impl, rtol=self.rtol, atol=self.atol)


def group_case(label, groups, seed, suite="smoke", **extra) -> CaseSpec:
    return CaseSpec(label, {"groups": [tuple(g) for g in groups], **extra}, seed, suite)


def example75_groups(seed: int = 75, count: int = 10) -> list[tuple[int, int, int]]:
    """Random problems in the style of CUTLASS example 75: ``count`` groups with
    m, n, k = 32 * (draw % 64) from a seeded generator, 0 replaced by 32."""
    rng = random.Random(seed)
    return [tuple(32 * max(rng.randrange(64), 1) for _ in range(3)) for _ in range(count)]


# Smoke cases (the reference's, nvfp4_group_gemm.py:688-727): one tile; three ragged
# groups; distinct (m, n, k) per group down to a 1-row group with k = 32, a partial
# scale atom, partial N and a nine-k-tile loop; MoE-like skewed groups (1-row groups
# included) over a shared partial-N/long-K weight shape with about 200 tiles; random
# example-75 problems; zero, subnormal and three-binade scales.
SMOKE = (
    group_case("single", [(128, 128, 128)], 1),
    group_case("ragged", [(17, 128, 128), (128, 256, 256), (65, 128, 512)], 2),
    group_case("distinct", [(1, 8, 32), (200, 136, 96), (129, 264, 384), (300, 1032, 2080)], 3),
    group_case("skewed", [(m, 2056, 1024) for m in skewed_lengths(640, 12, seed=4, sigma=1.5)], 4),
    group_case("skewed_full", [(m, 520, 2080) for m in skewed_lengths(300, 6, seed=5, sigma=1.5)],
               5, values="full", scales="int0_3"),
    group_case("distinct_unit", [(64, 72, 160), (257, 136, 512)], 6, scales="unit"),
    group_case("ragged_uniform", [(33, 264, 256), (190, 128, 768)], 7, scales="uniform"),
    CaseSpec(
        "cutlass_example75", {"groups": example75_groups()}, 75, "smoke",
        {"kind": "upstream_test",
         "test": "cutlass examples/75_blackwell_grouped_gemm/"
                 "75_blackwell_grouped_gemm_block_scaled.cu::randomize_problems "
                 "(groups=10, alpha=1, beta=0 as configured here)"},
    ),
)


def task_group_cases() -> list[CaseSpec]:
    """Every NVIDIA task test line, with the task's seed."""
    cases = []
    for index, (ms, ns, ks) in enumerate(TASK_TESTS):
        groups = list(zip(ms, ns, ks, strict=True))
        label = "task_" + "_".join(f"{m}x{n}x{k}" for m, n, k in groups)
        cases.append(upstream_case(label, {"groups": groups},
                                   f"nvfp4_group_gemm/task.yml::tests[{index}]", seed=TASK_SEED))
    return cases


THROUGHPUT = "nvfp4_group_gemm"

# (model, local experts per GPU, token counts): MoE expert GEMMs (gate_up and down);
# each local expert is one group holding its routed tokens; per-expert counts are
# seeded log-normal and experts without tokens are left out of the launch.
MOE_PLAN = (
    ("deepseek_v3", 32, (16, 1024, 16384)),
    ("qwen3_235b_a22b", 32, (16, 1024, 16384)),
    ("gpt_oss_120b", 128, (16, 1024, 16384)),
    ("llama4_maverick", 16, (16, 1024, 16384)),
)


def moe_cases() -> list[CaseSpec]:
    from ..models import MODELS

    cases = []
    for model, local, token_counts in MOE_PLAN:
        spec = MODELS[model]
        shapes = spec.linear_shapes()
        for tokens in token_counts:
            routed = tokens * spec.top_k * local // spec.experts
            counts = [m for m in skewed_lengths(routed, local, seed=tokens, minimum=0) if m]
            for layer in ("expert_gate_up", "expert_down"):
                n, k = shapes[layer]
                case = model_case(f"{model}_{layer}_t{tokens}",
                                  {"groups": [(m, n, k) for m in counts]}, model, layer)
                case.source.update(tokens=tokens, local_experts=local)
                cases.append(case)
    return cases


def throughput_cases():
    """Throughput cases: every task benchmark line and the MoE expert GEMMs."""
    cases = [
        CaseSpec(f"throughput_groups{len(ms)}_n{ns[0]}_k{ks[0]}",
                 {"groups": list(zip(ms, ns, ks, strict=True))}, TASK_SEED, "throughput",
                 official_source(THROUGHPUT))
        for ms, ns, ks in TASK_BENCHMARKS
    ]
    return cases + moe_cases()
