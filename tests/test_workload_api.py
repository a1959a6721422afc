"""The operator API on CPU: registry, case lists (against the reference's inventory),
references against golden fixtures and an FP64 restatement, operand rejection and the
rule that sm_100a code never runs on another device. Follows the reference's
tests/test_nvfp4_gemm.py, test_nvfp4_dual_gemm.py, test_nvfp4_group_gemm.py and
test_workloads.py (RegisteredWorkloads) where they need no generated artifacts."""

from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import GOLDEN, load_golden
from harness import CaseSpec, Workload, enumerate_workloads, get_workload, normalize_arch, register
from harness import native
from harness.registry import REGISTRY, register_variant
from harness.workload import arch_compatible
from harness.workloads.nvfp4_dual_gemm import (
    SILU_BUDGET, dual_gemm_cases, dual_gemm_inputs, pack_scales_reference, silu_bytes,
)
from harness.workloads.nvfp4_gemm import NVFP4GEMM, from_task_scales
from harness.workloads.nvfp4_group_gemm import NVFP4GroupGEMM, example75_groups, from_blocked

REFERENCE_NAMES = ("nvfp4_dual_gemm_gemm", "nvfp4_dual_gemm_pack_scales",
                   "nvfp4_dual_gemm_silu_product", "nvfp4_gemm", "nvfp4_group_gemm")


def test_registry_lists_the_hot_path_workloads():
    names = [cls.name for cls in enumerate_workloads("sm_100a")]
    assert names == sorted(names)
    assert set(REFERENCE_NAMES) <= set(names) and "nvfp4_dual_gemm" in names
    assert enumerate_workloads("sm_86") == []
    for name in names:
        cls = get_workload(name)
        assert cls.name == name and cls.supported_arches == ("sm_100a",)
        assert REGISTRY[name] is cls


def test_register_rejects_duplicates_and_bad_classes():
    with pytest.raises(ValueError):
        register(name="nvfp4_gemm", supported_arches=("sm_100a",))(
            type("Other", (NVFP4GEMM,), {}))
    with pytest.raises(ValueError):
        register(name="empty", supported_arches=())
    with pytest.raises(TypeError):
        register(name="not_a_workload", supported_arches=("sm_100a",))(object)
    variant = register_variant(NVFP4GEMM, name="nvfp4_gemm_test-variant",
                               supported_arches=("100a", "sm_100a"), rtol_hint=1)
    try:
        assert variant.supported_arches == ("sm_100a",) and variant.rtol_hint == 1
        assert variant.__module__ == NVFP4GEMM.__module__
    finally:
        del REGISTRY["nvfp4_gemm_test-variant"]


def test_arch_helpers():
    assert normalize_arch("-arch=sm_100a") == normalize_arch("100a") == "sm_100a"
    assert normalize_arch("compute_86") == "sm_86"
    with pytest.raises(ValueError):
        normalize_arch("sm_1")
    assert arch_compatible("sm_80", "sm_86") and not arch_compatible("sm_100a", "sm_103a")
    assert arch_compatible("sm_100f", "sm_103a") and not arch_compatible("sm_100a", "sm_90")


def test_case_lists_equal_the_reference_inventory():
    """Names, seeds, suites and parameters of every case of the five reference
    workloads equal the inventory recorded from the reference."""
    recorded: dict[str, list[str]] = {}
    for line in (GOLDEN / "case_inventory.tsv").read_text().splitlines():
        name, rest = line.split("\t", 1)
        recorded.setdefault(name, []).append(rest)
    assert set(recorded) == set(REFERENCE_NAMES)
    for name, lines in recorded.items():
        cases = get_workload(name)(None, device="cpu").get_cases()
        mine = [f"{c.name}\t{c.seed}\t{c.suite}\t{sorted(c.params.items())!r}" for c in cases]
        assert mine == lines, name
    fused = get_workload("nvfp4_dual_gemm")(None, device="cpu").get_cases()
    assert [c.name for c in fused] == [c.name for c in dual_gemm_cases()]


def test_case_properties():
    gemm = NVFP4GEMM(None, device="cpu").get_cases()
    shapes = {tuple(c.params[k] for k in "mnkl") for c in gemm}
    assert (128, 7168, 16384, 1) in shapes and (2304, 4608, 7168, 1) in shapes
    assert any(c.params["k"] % 256 for c in gemm) and any(c.params["m"] == 1 for c in gemm)
    group = NVFP4GroupGEMM(None, device="cpu").get_cases()
    by_groups = {tuple(map(tuple, c.params["groups"])): c for c in group}
    example = by_groups[tuple(example75_groups())]
    assert example.source["kind"] == "upstream_test" and len(example.params["groups"]) == 10
    moe = [c for c in group if c.source.get("kind") == "model_shape"]
    assert any(min(m for m, _, _ in c.params["groups"]) == 1 for c in moe)
    assert max(m for c in moe for m, _, _ in c.params["groups"]) >= 1000
    silu = get_workload("nvfp4_dual_gemm_silu_product")(None, device="cpu").get_cases()
    assert all(silu_bytes(c.params) <= SILU_BUDGET for c in silu) and len(silu) < len(dual_gemm_cases())


def test_dense_reference_matches_fp64_restatement():
    workload = NVFP4GEMM(None, device="cpu")
    case = CaseSpec("tiny", {"m": 130, "n": 136, "k": 96, "l": 2, "alpha": 0.37}, 5)
    a, b, sfa, sfb, alpha = workload.get_inputs(case)
    (ref,) = workload.get_reference((a, b, sfa, sfb, alpha))
    lut = torch.tensor([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6],
                       dtype=torch.float64)
    sa = from_task_scales(sfa, 130, 6).double()
    sb = from_task_scales(sfb, 136, 6).double()
    assert (sa == 0).any()

    def dequant(packed, scales):
        values = torch.stack((packed & 15, packed >> 4), dim=-1).flatten(1)
        return lut[values.long()] * scales.repeat_interleave(16, dim=1)

    for batch in range(2):
        expected = (dequant(a[:, :, batch], sa[:, :, batch])
                    @ dequant(b[:, :, batch], sb[:, :, batch]).T) * alpha.double()
        torch.testing.assert_close(ref[:, :, batch], expected.half(), rtol=1e-3, atol=1e-3)
    assert tuple(ref.shape) == (130, 136, 2) and ref.permute(2, 0, 1).is_contiguous()


def test_references_reproduce_golden_outputs():
    """``get_inputs`` regenerates the recorded tensors from the case seeds and
    ``get_reference`` the recorded outputs (same torch CPU generator)."""
    dense = load_golden("nvfp4_gemm_cases.npz")
    workload = NVFP4GEMM(None, device="cpu")
    cases = {c.name: c for c in workload.get_cases()}
    for name in sorted({key.split("/")[0] for key in dense}):
        a, b, sfa, sfb, alpha = workload.get_inputs(cases[name])
        assert np.array_equal(a.permute(2, 0, 1).numpy(), dense[name + "/a"]), name
        assert np.array_equal(
            sfb.permute(5, 2, 4, 0, 1, 3).contiguous().view(torch.uint8).numpy(),
            dense[name + "/sfb"]), name
        (ref,) = workload.get_reference((a, b, sfa, sfb, alpha))
        assert np.array_equal(ref.permute(2, 0, 1).numpy(), dense[name + "/d"]), name

    dual = load_golden("nvfp4_dual_gemm_cases.npz")
    stage = get_workload("nvfp4_dual_gemm_silu_product")(None, device="cpu")
    fused = get_workload("nvfp4_dual_gemm")(None, device="cpu")
    cases = {c.name: c for c in stage.get_cases()}
    for name in sorted({key.split("/")[0] for key in dual}):
        h1, h2 = stage.get_inputs(cases[name])
        assert np.array_equal(h1.permute(2, 0, 1).numpy(), dual[name + "/h1"]), name
        (out,) = stage.get_reference((h1, h2))
        assert np.array_equal(out.permute(2, 0, 1).numpy(), dual[name + "/out"]), name
        (whole,) = fused.get_reference(fused.get_inputs(cases[name]))
        assert torch.equal(whole, out), name
        _, _, _, sa, _, _, _ = dual_gemm_inputs(stage, cases[name])
        assert np.array_equal(pack_scales_reference(sa).view(torch.uint8).numpy(),
                              dual[name + "/packed_sa"]), name

    group = load_golden("nvfp4_group_gemm_cases.npz")
    workload = NVFP4GroupGEMM(None, device="cpu")
    cases = {c.name: c for c in workload.get_cases()}
    for name in ("ragged", "distinct_unit", "ragged_uniform"):
        outputs = workload.get_reference(workload.get_inputs(cases[name]))
        for index, out in enumerate(outputs):
            assert np.array_equal(out.numpy(), group[f"{name}/{index}/d"]), (name, index)


def test_pipeline_stages_share_inputs():
    gemm = get_workload("nvfp4_dual_gemm_gemm")(None, device="cpu")
    silu = get_workload("nvfp4_dual_gemm_silu_product")(None, device="cpu")
    case = next(c for c in gemm.get_cases() if c.name == "m200_n136_k96_l1")
    (h,) = gemm.get_reference(gemm.get_inputs(case))
    h1, _ = silu.get_inputs(case)
    assert torch.equal(h, h1)


def library_workload(cls):
    if not native.LIBRARY_PATH.is_file():
        pytest.skip("native library not built")
    return cls.from_arch("sm_100a", device="cpu")


def test_dense_rejects_bad_operands_before_any_native_work():
    workload = library_workload(NVFP4GEMM)
    assert workload.image_name() == "nvfp4_gemm_launch" and workload.get_image()
    case = workload.get_cases()[1]  # batched
    inputs = workload.get_inputs(case)
    a, b, sfa, sfb, alpha = inputs
    (out,) = workload.allocate_outputs(inputs)
    config = workload.launch_config(inputs, out)
    assert config.problem == (128, 256, 256, 2)
    logical = from_task_scales(sfa, a.shape[0], 2 * a.shape[1] // 16)
    bad = (
        ((a, b, logical, sfb, alpha), out),  # logical instead of blocked scales
        ((a.contiguous(), b, sfa, sfb, alpha), out),  # batch innermost
        (inputs, out.float()),
        ((a, b, sfa, sfb, alpha.double()), out),
        ((a, b, sfa, sfb, torch.ones(2)), out),
    )
    for operands, output in bad:
        with pytest.raises(ValueError):
            workload.launch_config(operands, output)
    with pytest.raises(ValueError):
        workload.build_params(128, 128, 48, 1, 0, 0, 0, 0, 0, 0)
    with pytest.raises(ValueError):
        workload.build_params(128, 132, 64, 1, 0, 0, 0, 0, 0, 0)  # 264-byte D rows
    with pytest.raises(ValueError):
        workload.build_params(128, 128, 64, 1, 8, 0, 0, 0, 0, 0)  # misaligned A
    if not workload.is_supported():
        with pytest.raises(RuntimeError):  # never execute sm_100a code elsewhere
            workload.run(inputs)
        with pytest.raises(RuntimeError):
            workload.prepare(inputs)


def test_group_rejects_bad_operands():
    workload = library_workload(NVFP4GroupGEMM)
    case = workload.get_cases()[1]
    inputs = workload.get_inputs(case)
    outputs = workload.allocate_outputs(inputs)
    config = workload.launch_config(inputs, outputs)
    assert config.problems == ((17, 128, 128), (128, 256, 256), (65, 128, 512))
    assert config.pointers[0] == [g[0].data_ptr() for g in workload.groups_of(inputs)]
    assert config.pointers[4] == [t.data_ptr() for t in outputs]
    logical = from_blocked(inputs[2], 17, 128 // 16)
    with pytest.raises(ValueError):
        workload.launch_config((inputs[0], inputs[1], logical) + inputs[3:], outputs)
    with pytest.raises(ValueError):
        workload.launch_config(inputs, (outputs[0].float(),) + outputs[1:])
    with pytest.raises(ValueError):
        workload.launch_config(inputs[:-1], outputs)
    with pytest.raises(ValueError):
        workload.launch_config(inputs, outputs[:-1])
    if not workload.is_supported():
        with pytest.raises(RuntimeError):
            workload.run(inputs)


def test_reference_only_workload_has_no_image():
    workload = NVFP4GEMM(None, device="cpu")
    assert not workload.is_supported()
    with pytest.raises(RuntimeError):
        workload.get_image()
    with pytest.raises(ValueError):
        NVFP4GEMM.from_arch("sm_86", device="cpu")
    with pytest.raises(ValueError):
        NVFP4GEMM(b"\x7fELF not ours", device="cpu")
    assert isinstance(workload, Workload) and Path(native.LIBRARY_PATH).name.endswith(".so")


def test_fused_dual_gemm_output_alignment_follows_the_store_width():
    """Rows of D are stored in 16-byte pieces unless n % 8 == 4, so only then may D be
    merely 8-byte aligned: a slice of a larger tensor must not reach the kernel otherwise."""
    fused = get_workload("nvfp4_dual_gemm")(None, device="cpu")
    for n, offsets_ok in ((136, {0: True, 4: False}), (132, {0: True, 4: True, 2: False})):
        case = CaseSpec("alignment", {"m": 128, "n": n, "k": 64, "l": 1}, 3)
        inputs = fused.get_inputs(case)
        for offset, ok in offsets_ok.items():
            backing = torch.empty(128 * n + 64, dtype=torch.float16)
            base = (-backing.data_ptr() % 16) // 2  # first 16-byte aligned element
            flat = backing[base + offset: base + offset + 128 * n]
            out = flat.view(1, 128, n).permute(1, 2, 0)
            if ok:
                assert fused.operands(inputs, out) == (128, n, 64, 1)
            else:
                with pytest.raises(ValueError):
                    fused.operands(inputs, out)
