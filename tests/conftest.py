"""Test configuration.

`-m "not gpu"` : oracle vs. golden vectors, host logic, C-ABI export checks (no GPU needed).
`-m gpu`       : parity tests of the CUDA kernels against the CPU oracle, through the C ABI.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "cutile-python_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture()
def device_ok():
    """Yields, then fails the test if a kernel recorded a device-side timeout."""
    import torch
    import b200k
    yield
    torch.cuda.synchronize()
    code, info = b200k.device_status()
    assert code == 0, f"device status {code}, info {info:#x}"
