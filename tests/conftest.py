"""Shared test setup: import paths, the ``gpu`` marker and fixture loading."""

import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parents[1]
PACKAGE = REPO / "flashinfer-cubins_b200"
GOLDEN = Path(__file__).resolve().parent / "golden"
for path in (str(PACKAGE), str(REPO)):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


def load_golden(name: str) -> dict:
    with np.load(GOLDEN / name) as data:
        return {key: data[key] for key in data.files}


@pytest.fixture(scope="session")
def golden():
    return load_golden
