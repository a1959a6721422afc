"""One workload's GPU acceptance loop, run in a process of its own.

    python tests/acceptance_worker.py <workload name>

Every smoke case of the workload against the harness's torch reference (the reference
project's own check, tests/test_workloads.py:98-157 there) and against the numpy oracle;
inputs not mutated; library re-bind; prepared launches allocate nothing and return the same
outputs; the device status word stays zero. The reference runs this loop one workload per
worker process (tests/test_workloads.py:169-324 there) so that a lost CUDA context is
attributed to the workload that lost it and does not fail the tests after it;
``tests/test_gpu_workloads.py`` starts this file the same way. Exit code 0 and a last line
``ok <name> <cases>`` on success."""

import sys
from pathlib import Path

REPO = Path(__file__).resolve().parents[1]
for path in (str(REPO / "flashinfer-cubins_b200"), str(REPO), str(Path(__file__).resolve().parent)):
    if path not in sys.path:
        sys.path.insert(0, path)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from gpu_util import (assert_matches_oracle, blocked_storage, integer_scaled,  # noqa: E402
                      oracle_dense, snapshot, storage, unchanged)
from harness import enumerate_workloads, get_workload  # noqa: E402
from oracle import nvfp4_oracle as o  # noqa: E402


def check_prepared(workload, case, inputs, before, ref):
    tag = f"{workload.name}/{case.name}"
    launch, outputs = workload.prepare(inputs)
    torch.cuda.synchronize()
    for call in range(2):
        allocated = torch.cuda.memory_stats()["allocation.all.allocated"]
        result = launch()
        new = torch.cuda.memory_stats()["allocation.all.allocated"] - allocated
        assert not new, f"{tag}: prepared launch {call} allocated {new} blocks"
        assert result is outputs, f"{tag}: prepared launch must return its outputs"
        torch.cuda.synchronize()
        if call == 0:
            workload.validate(ref, outputs)
    for old, new_input in zip(before, inputs):
        assert unchanged(old, new_input), f"{tag}: prepared launch mutated inputs"


def oracle_check(workload, case, inputs, out):
    name = f"{workload.name}/{case.name}"
    default = {"nvfp4_gemm": "int0_3", "nvfp4_group_gemm": "int1_2"}.get(workload.name)
    exact = integer_scaled(case, default)
    if workload.name == "nvfp4_gemm":
        assert_matches_oracle(out[0], oracle_dense(inputs), name, exact and case.params.get("alpha", 1.0) == 1.0)
    elif workload.name in ("nvfp4_gemm_bf16", "nvfp4_gemm_bf16_shuffled"):
        if workload.name == "nvfp4_gemm_bf16_shuffled":
            # The oracle puts the rows of B and of its scales back in logical order.
            a, b, sfa, sfb, alpha = inputs
            m, half_k, _ = a.shape
            n, k = b.shape[0], 2 * half_k
            product = o.shuffled_gemm(
                storage(a), storage(b), o.from_blocked(blocked_storage(sfa), m, k // 16),
                o.from_blocked(blocked_storage(sfb), n, k // 16), workload.SHUFFLE_BLOCK,
                float(alpha.item()), np.float32)
        else:
            product = oracle_dense(inputs, np.float32)
        want = o.round_to_bf16_bits(product)
        got = out[0].permute(2, 0, 1).contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        if integer_scaled(case, "int0_3") and case.params.get("alpha", 1.0) == 1.0:
            assert np.array_equal(got, want), f"{name}: not bit-identical to the oracle"
        else:
            np.testing.assert_allclose(o.bf16_bits_to_float(got), o.bf16_bits_to_float(want),
                                       rtol=8e-3, atol=1e-3, err_msg=name)
    elif workload.name == "nvfp4_dual_gemm_gemm":
        a, b, sfa, sfb, alpha = inputs
        m, half_k, batches = a.shape
        n, k = b.shape[0], 2 * half_k
        rb_a, rb_n, cb = -(-m // 128), -(-n // 128), -(-(k // 16) // 4)
        sa = o.from_blocked(sfa.view(torch.uint8).cpu().numpy().reshape(batches, rb_a, cb, 32, 4, 4), m, k // 16)
        sb = o.from_blocked(sfb.view(torch.uint8).cpu().numpy().reshape(batches, rb_n, cb, 32, 4, 4), n, k // 16)
        expected = o.gemm(storage(a), storage(b), sa, sb, float(alpha.item()))
        assert_matches_oracle(out[0], expected, name, integer_scaled(case), rtol=1e-4, atol=1e-4)
    elif workload.name == "nvfp4_dual_gemm":
        a, b1, b2, sfa, sfb1, sfb2, alpha = inputs
        m, half_k, _ = a.shape
        n, k = b1.shape[0], 2 * half_k
        sa = o.from_blocked(blocked_storage(sfa), m, k // 16)
        s1 = o.from_blocked(blocked_storage(sfb1), n, k // 16)
        s2 = o.from_blocked(blocked_storage(sfb2), n, k // 16)
        expected = o.dual_gemm(storage(a), storage(b1), storage(b2), sa, s1, s2, float(alpha.item()))
        assert_matches_oracle(out[0], expected, name, False)
    elif workload.name == "nvfp4_group_gemm":
        problems = []
        for a, b, sfa, sfb in workload.groups_of(inputs):
            m, n, k = workload.problem_of((a, b))
            sa = o.from_blocked(sfa.view(torch.uint8).cpu().numpy()[None], m, k // 16)[0]
            sb = o.from_blocked(sfb.view(torch.uint8).cpu().numpy()[None], n, k // 16)[0]
            problems.append((a.cpu().numpy(), b.cpu().numpy(), sa, sb))
        for index, expected in enumerate(o.group_gemm(problems)):
            assert_matches_oracle(out[index], expected, f"{name}/{index}", exact)
    elif workload.name == "nvfp4_dual_gemm_pack_scales":
        expected = o.pack_scales(storage(inputs[0]))
        assert np.array_equal(out[0].view(torch.uint8).cpu().numpy(), expected), name
    else:
        expected = o.silu_product(storage(inputs[0]), storage(inputs[1]))
        assert_matches_oracle(out[0], expected, name, False)


def acceptance(name: str) -> int:
    """Runs the loop for workload ``name``; returns the number of cases checked."""
    torch.backends.cuda.matmul.allow_tf32 = False
    cls = get_workload(name)
    assert cls in enumerate_workloads("sm_100a")
    with cls.from_arch("sm_100a", device="cuda") as workload:
        assert workload.is_supported(), "not a B200"
        cases = [c for c in workload.get_cases() if c.suite == "smoke"]
        assert cases
        for index, case in enumerate(cases):
            inputs = workload.get_inputs(case)
            before = snapshot(inputs)
            ref = workload.get_reference(inputs)
            out = workload.run(inputs)
            torch.cuda.synchronize()
            workload.validate(ref, out)
            oracle_check(workload, case, inputs, out)
            for old, new in zip(before, inputs):
                assert unchanged(old, new), f"{name}/{case.name} mutated inputs"
            if index == 0:
                workload.patch_image(workload.get_image())
                again = workload.run(inputs)
                torch.cuda.synchronize()
                workload.validate(ref, again)
            check_prepared(workload, case, inputs, before, ref)
            workload.check_status()
    return len(cases)


if __name__ == "__main__":
    checked = acceptance(sys.argv[1])
    print(f"ok {sys.argv[1]} {checked}", flush=True)
