"""Test configuration: the ``gpu`` marker and the import paths of the package and the oracle."""

import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
for p in (REPO / "emmy-ptx-compiler_b200", REPO):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    import json

    import numpy as np
    here = Path(__file__).resolve().parent / "golden"
    cases = json.loads((here / "oracle_cases.json").read_text())
    arrays = np.load(here / "oracle_cases.npz")
    return {c["name"]: (c, arrays) for c in cases}
