"""The reference project's own hot-path test modules, run unchanged against this package
(``tests/run_reference_tests.py``) where ``REFERENCE_ROOT`` names a checkout of the
reference; skipped elsewhere."""

import os
from pathlib import Path

import pytest

import run_reference_tests as runner


def checkout() -> Path | None:
    candidate = os.environ.get("REFERENCE_ROOT")
    if candidate and (Path(candidate) / "tests" / "test_quantization.py").is_file():
        return Path(candidate)
    return None


@pytest.mark.skipif(checkout() is None, reason="no checkout of the reference project")
def test_reference_hot_path_tests_pass_unchanged():
    results = runner.run(checkout())
    failed = [(test, note) for test, outcome, note in results if outcome == "FAIL"]
    assert not failed, failed
    passed = {test for test, outcome, _ in results if outcome == "pass"}
    # The sixteen tests that pass in a bare checkout of the reference.
    assert len(passed) >= 16, sorted(passed)
    assert "test_nvfp4_gemm.py::test_reference_matches_task_definition" in passed
    assert "test_throughput_cases.py::test_nvidia_benchmark_shapes" in passed
    not_applicable = {test for test, outcome, _ in results if outcome == "N/A"}
    assert not_applicable <= set(runner.NOT_APPLICABLE)
