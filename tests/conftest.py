"""pytest configuration: the `gpu` marker and import paths."""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
PACKAGE_DIR = ROOT / "pytorch-approx-topk_b200"
for p in (str(ROOT), str(PACKAGE_DIR)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100); run with -m gpu on a B200")


def pytest_runtest_setup(item):
    # A test marked `gpu` that is run on a machine without a CUDA device fails
    # (it is never skipped): select with -m "not gpu" where there is no GPU.
    if item.get_closest_marker("gpu") is not None:
        import torch

        if not torch.cuda.is_available():
            pytest.fail("this test is marked `gpu` and needs a CUDA device; run the CPU suite with -m \"not gpu\"")


@pytest.fixture(scope="session")
def golden():
    import json

    import numpy as np

    data = np.load(ROOT / "tests" / "golden" / "reference_cpu_vectors.npz")
    meta = json.loads(bytes(data["meta"]).decode())
    return data, meta


@pytest.fixture(scope="session")
def golden_all_dtypes():
    """Reference CPU outputs for float64 and the integer element types."""
    import json

    import numpy as np

    data = np.load(ROOT / "tests" / "golden" / "reference_cpu_vectors_all_dtypes.npz")
    meta = json.loads(bytes(data["meta"]).decode())
    return data, meta
