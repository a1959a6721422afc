#!/usr/bin/env python
"""Runs the reference project's own hot-path test modules, unchanged, against this package.

    REFERENCE_ROOT=/path/to/flashinfer-cubins python tests/run_reference_tests.py

The five modules (tests/test_quantization.py, test_nvfp4_gemm.py, test_nvfp4_dual_gemm.py,
test_nvfp4_group_gemm.py, test_throughput_cases.py of the reference) are copied byte for
byte into a temporary directory (run in place they would put the reference's own
``harness`` first on ``sys.path``) and run under pytest with this package's ``harness`` on
the path and ``REFERENCE_ROOT`` telling the package where the reference keeps its data
files (the task definitions and the trace inventories, which are not part of this
repository). One line per test is printed:

* ``pass`` / ``FAIL``;
* ``N/A``: the test pins a mechanism that does not exist here, and it fails in a bare
  reference checkout as well because it needs generated artefacts: byte-for-byte CUTLASS
  ``Params`` and device arrays against fixtures recorded from CUTLASS's host code, the
  ``fake_encode`` tensor-map stand-in, the cubin manifest, or the pinned FlashInfer source
  tree.

Exit code 0 when every test that is not N/A passes. Nothing here needs a GPU.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile
import xml.etree.ElementTree as ET
from pathlib import Path

REPO = Path(__file__).resolve().parents[1]
PACKAGE = REPO / "flashinfer-cubins_b200"
MODULES = ("test_quantization", "test_nvfp4_gemm", "test_nvfp4_dual_gemm",
           "test_nvfp4_group_gemm", "test_throughput_cases")
# Tests of mechanisms this build replaces, with the reason.
NOT_APPLICABLE = {
    "test_nvfp4_gemm.py::test_params_match_cutlass": "pins CUTLASS Params bytes",
    "test_nvfp4_gemm.py::test_fixtures_cover_regimes": "pins CUTLASS Params fixtures",
    "test_nvfp4_gemm.py::test_upstream_parametrizations_are_cases":
        "reads the pinned FlashInfer source tree (absent from the checkout)",
    "test_nvfp4_gemm.py::test_rejects_bad_operands":
        "needs the cubin manifest and the fake tensor-map encoder",
    "test_nvfp4_dual_gemm.py::test_params_match_cutlass": "pins CUTLASS Params bytes",
    "test_nvfp4_dual_gemm.py::test_fixtures_cover_regimes": "pins CUTLASS Params fixtures",
    "test_nvfp4_dual_gemm.py::test_rejects_bad_operands":
        "needs the cubin manifest and the fake tensor-map encoder",
    "test_nvfp4_group_gemm.py::test_params_and_arrays_match_cutlass":
        "pins CUTLASS Params and device-array bytes",
    "test_nvfp4_group_gemm.py::test_fixtures_cover_regimes": "pins CUTLASS Params fixtures",
    "test_nvfp4_group_gemm.py::test_launch_config_wires_tensors":
        "pins CUTLASS device arrays and the fake tensor-map encoder",
    "test_nvfp4_group_gemm.py::test_rejects_bad_operands":
        "needs the cubin manifest and the fake tensor-map encoder",
}


def reference_root() -> Path | None:
    root = os.environ.get("REFERENCE_ROOT")
    if root and (Path(root) / "tests" / "test_quantization.py").is_file():
        return Path(root)
    return None


def run(root: Path) -> list[tuple[str, str, str]]:
    """[(test id, outcome, note)] for every test of the five modules."""
    results = []
    with tempfile.TemporaryDirectory() as tmp:
        tests = Path(tmp) / "tests"
        tests.mkdir()
        for module in MODULES:
            shutil.copyfile(root / "tests" / f"{module}.py", tests / f"{module}.py")
        env = dict(os.environ, REFERENCE_ROOT=str(root),
                   PYTHONPATH=os.pathsep.join([str(PACKAGE), str(REPO)]))
        for module in MODULES:
            report = Path(tmp) / f"{module}.xml"
            subprocess.run(
                [sys.executable, "-m", "pytest", str(tests / f"{module}.py"), "-q",
                 "-p", "no:cacheprovider", f"--junitxml={report}"],
                env=env, cwd=tmp, capture_output=True, text=True)
            if not report.is_file():
                results.append((f"{module}.py", "FAIL", "pytest produced no report"))
                continue
            cases = ET.parse(report).getroot().iter("testcase")
            seen = False
            for case in cases:
                seen = True
                name = case.get("name")
                if not case.get("classname"):  # a collection error, reported as one case
                    text = case.find("error")
                    if text is None:
                        text = case.find("failure")
                    message = text.get("message", "") if text is not None else ""
                    results.append((f"{module}.py", "FAIL",
                                    "could not be imported: " + message[:200]))
                    continue
                test_id = f"{module}.py::{name}"
                failed = case.find("failure") is not None or case.find("error") is not None
                if test_id in NOT_APPLICABLE:
                    results.append((test_id, "N/A", NOT_APPLICABLE[test_id]))
                elif failed:
                    node = case.find("failure") if case.find("failure") is not None \
                        else case.find("error")
                    results.append((test_id, "FAIL", (node.get("message") or "")[:200]))
                else:
                    results.append((test_id, "pass", ""))
            if not seen:
                results.append((f"{module}.py", "FAIL", "no test collected"))
    return results


def main() -> int:
    root = reference_root()
    if root is None:
        print("REFERENCE_ROOT does not name a checkout of the reference; nothing to run")
        return 2
    results = run(root)
    for test_id, outcome, note in results:
        print(f"{outcome:5s} {test_id}" + (f"  ({note})" if note else ""))
    passed = sum(1 for _, outcome, _ in results if outcome == "pass")
    skipped = sum(1 for _, outcome, _ in results if outcome == "N/A")
    failed = sum(1 for _, outcome, _ in results if outcome == "FAIL")
    print(f"{passed} pass, {skipped} N/A, {failed} FAIL")
    return 1 if failed else 0


if __name__ == "__main__":
    raise SystemExit(main())
