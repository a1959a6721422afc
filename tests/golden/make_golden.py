"""Regenerates the golden fixtures in this directory from the reference itself.

Run where the reference checkout is available (it is pure PyTorch on CPU for this
path):

    REFERENCE_ROOT=/path/to/flashinfer-cubins python tests/golden/make_golden.py

The script imports the reference's ``harness`` package (and nothing of this
repository), runs its own input generators and torch oracle on CPU, and stores inputs
and outputs in *storage order* (batch outermost) as compressed ``.npz`` files. The
tests then check this repository's oracle, its harness mirror and its CUDA kernels
against these files without needing the reference.
"""

import os
import sys
from pathlib import Path

import numpy as np
import torch

REFERENCE_ROOT = os.environ.get("REFERENCE_ROOT")
if not REFERENCE_ROOT or not Path(REFERENCE_ROOT, "harness").is_dir():
    raise SystemExit("set REFERENCE_ROOT to a checkout of the reference (it has a harness/ package)")
sys.path.insert(0, REFERENCE_ROOT)

from harness import get_workload  # noqa: E402  (the reference's package)
from harness.workloads import nvfp4_dual_gemm as ref_dual  # noqa: E402
from harness.workloads import nvfp4_gemm as ref_gemm  # noqa: E402
from harness.workloads import nvfp4_group_gemm as ref_group  # noqa: E402
from harness.workloads import quantization as q  # noqa: E402
from harness.workloads.batched_gemm import formats as fmt  # noqa: E402

OUT = Path(__file__).resolve().parent


def storage(t: torch.Tensor) -> np.ndarray:
    """A ``(rows, cols, l)`` view -> contiguous ``[l, rows, cols]`` bytes/values."""
    t = t.permute(2, 0, 1).contiguous()
    if t.dtype == torch.float8_e4m3fn:
        t = t.view(torch.uint8)
    return t.numpy()


def blocked_storage(task_view: torch.Tensor) -> np.ndarray:
    """The task's 6-D scale view -> contiguous ``[l, rb, cb, 32, 4, 4]`` bytes."""
    return task_view.permute(5, 2, 4, 0, 1, 3).contiguous().view(torch.uint8).numpy()


def known_answer():
    # tests/test_quantization.py:65-75: nibble order, sign, LUT, 16-element boundary.
    packed = torch.tensor([0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE] * 2,
                          dtype=torch.uint8).reshape(1, 16, 1)
    scales = torch.tensor([2.0, 0.5]).reshape(1, 2, 1)
    decoded = q.dequant_fp4(packed, scales)
    np.savez_compressed(
        OUT / "dequant_known_answer.npz",
        packed=storage(packed), scales=storage(scales.to(torch.float8_e4m3fn)),
        decoded=storage(decoded),
    )


def blocked_layouts():
    # tests/test_quantization.py:60,126-153: shapes with partial atoms and batches.
    data = {}
    for rows, cols, batches in ((128, 8, 1), (200, 6, 2), (1, 2, 1), (260, 32, 3), (129, 16, 3)):
        g = torch.Generator().manual_seed(rows + cols)
        raw = torch.randint(1, 127, (batches, rows, cols), generator=g, dtype=torch.uint8)
        scales = raw.view(torch.float8_e4m3fn).permute(1, 2, 0)
        key = f"r{rows}_c{cols}_l{batches}"
        data[key + "_logical"] = raw.numpy()
        data[key + "_blocked"] = q.to_blocked_scales(scales).view(torch.uint8).numpy()
    np.savez_compressed(OUT / "blocked_layout.npz", **data)


def dense_cases():
    workload = get_workload("nvfp4_gemm")(None, device="cpu")
    wanted = {"m128_n128_k128_l1", "m200_n136_k96_l1", "m200_n136_k96_l1_scalesuniform",
              "m300_n264_k384_l3_alpha0.0123", "mm_fp4_m1_n128_k512", "mm_fp4_m31_n256_k256"}
    data = {}
    for case in workload.get_cases():
        if case.name not in wanted:
            continue
        a, b, sfa, sfb, alpha = workload.get_inputs(case)
        (ref,) = workload.get_reference((a, b, sfa, sfb, alpha))
        data[case.name + "/a"] = storage(a)
        data[case.name + "/b"] = storage(b)
        data[case.name + "/sfa"] = blocked_storage(sfa)
        data[case.name + "/sfb"] = blocked_storage(sfb)
        data[case.name + "/alpha"] = alpha.numpy()
        data[case.name + "/d"] = storage(ref)
    assert len(data) == 6 * len(wanted), sorted(data)
    np.savez_compressed(OUT / "nvfp4_gemm_cases.npz", **data)


def dual_cases():
    gemm = get_workload("nvfp4_dual_gemm_gemm")(None, device="cpu")
    pack = get_workload("nvfp4_dual_gemm_pack_scales")(None, device="cpu")
    silu = get_workload("nvfp4_dual_gemm_silu_product")(None, device="cpu")
    wanted = {"m128_n128_k128_l1", "m128_n256_k256_l2", "m200_n136_k96_l1", "m1_n520_k512_l1",
              "m200_n136_k96_l1_valuesfull_scalesint0_3_alpha0.015625"}
    data = {}
    for case in gemm.get_cases():
        if case.name not in wanted:
            continue
        a, b1, b2, sa, s1, s2, alpha = ref_dual.dual_gemm_inputs(gemm, case)
        h1, h2 = silu.get_inputs(case)
        (out,) = silu.get_reference((h1, h2))
        (h1_stage,) = gemm.get_reference(gemm.get_inputs(case))
        assert torch.equal(h1, h1_stage)
        for name, t in (("a", a), ("b1", b1), ("b2", b2), ("sa", sa), ("s1", s1), ("s2", s2),
                        ("h1", h1), ("h2", h2), ("out", out)):
            data[f"{case.name}/{name}"] = storage(t)
        data[f"{case.name}/alpha"] = np.float32(alpha)
        data[f"{case.name}/packed_sa"] = ref_dual.pack_scales_reference(sa).view(torch.uint8).numpy()
        data[f"{case.name}/packed_s1"] = ref_dual.pack_scales_reference(s1).view(torch.uint8).numpy()
    assert pack is not None
    np.savez_compressed(OUT / "nvfp4_dual_gemm_cases.npz", **data)


def group_cases():
    workload = get_workload("nvfp4_group_gemm")(None, device="cpu")
    wanted = {"ragged", "distinct_unit", "ragged_uniform"}
    data = {}
    for case in workload.get_cases():
        if case.name not in wanted:
            continue
        inputs = workload.get_inputs(case)
        outputs = workload.get_reference(inputs)
        for g, ((a, b, sfa, sfb), d) in enumerate(zip(workload.groups_of(inputs), outputs)):
            data[f"{case.name}/{g}/a"] = a.contiguous().numpy()
            data[f"{case.name}/{g}/b"] = b.contiguous().numpy()
            data[f"{case.name}/{g}/sfa"] = sfa.contiguous().view(torch.uint8).numpy()
            data[f"{case.name}/{g}/sfb"] = sfb.contiguous().view(torch.uint8).numpy()
            data[f"{case.name}/{g}/d"] = d.contiguous().numpy()
    np.savez_compressed(OUT / "nvfp4_group_gemm_cases.npz", **data)


def quantiser():
    # The NVFP4 quantiser convention (batched_gemm/formats.py:57-82, trtllm.py:530-547).
    g = torch.Generator().manual_seed(7)
    x = torch.randn(48, 256, generator=g)
    x[0, :16] = 0.0  # a zero block -> zero scale -> zero codes
    x[1, :16] *= 1000.0  # saturating scale
    blocks = x.view(48, 16, 16)
    scale = fmt.e4m3_encode(blocks.abs().amax(-1) / fmt.E2M1_MAX)
    safe = torch.where(scale.float() > 0, scale.float(), torch.ones(()))
    codes = fmt.e2m1_encode(blocks / safe[..., None])
    codes = torch.where((scale.float() > 0)[..., None], codes, torch.zeros_like(codes))
    grid = torch.linspace(-8, 8, 4097)
    np.savez_compressed(
        OUT / "quantiser.npz",
        x=x.numpy(), scale_bits=scale.view(torch.uint8).numpy(),
        packed=fmt.pack_nibbles(codes.view(48, 256)).numpy(),
        grid=grid.numpy(), grid_e2m1=fmt.e2m1_encode(grid).numpy(),
        e4m3_inputs=(grid * 60).numpy(),
        e4m3_bits=fmt.e4m3_encode(grid * 60).view(torch.uint8).numpy(),
    )


def shuffled_weights():
    """The epilogue row shuffle of weights prepared for FlashInfer's trtllm-gen kernels
    (batched_gemm/formats.py:143-161, applied by trtllm.py:257-288: physical row i of the
    data and of the scales holds logical row idx[i])."""
    data = {}
    for rows, tile_m in ((32, 128), (96, 128), (256, 256), (16, 64), (48, 64), (144, 32)):
        data[f"idx_rows{rows}_tile{tile_m}"] = fmt.shuffle_rows(rows, tile_m).numpy()
    np.savez_compressed(OUT / "shuffled_weights.npz", **data)


def case_inventory():
    """Names, seeds and suites of every case of the five reference workloads, so that
    the mirror's case lists can be compared without the reference."""
    lines = []
    for name in ("nvfp4_gemm", "nvfp4_dual_gemm_gemm", "nvfp4_dual_gemm_pack_scales",
                 "nvfp4_dual_gemm_silu_product", "nvfp4_group_gemm"):
        for case in get_workload(name)(None, device="cpu").get_cases():
            lines.append(f"{name}\t{case.name}\t{case.seed}\t{case.suite}\t{sorted(case.params.items())!r}")
    (OUT / "case_inventory.tsv").write_text("\n".join(lines) + "\n")


if __name__ == "__main__":
    torch.manual_seed(0)
    known_answer()
    blocked_layouts()
    dense_cases()
    dual_cases()
    group_cases()
    quantiser()
    shuffled_weights()
    case_inventory()
    for path in sorted(OUT.glob("*.npz")) + sorted(OUT.glob("*.tsv")):
        print(path.name, path.stat().st_size)
