import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_sessionstart(session):
    """Build the C-ABI libraries when they are missing or older than their sources (they are build artefacts, not
    tracked files). Without nvcc nothing is built and the tests that need the library fail with its own message."""
    import shutil
    from fastbb_b200 import build
    if shutil.which("nvcc") or os.path.exists("/usr/local/cuda/bin/nvcc"):
        for flash_only in (False, True):
            out = build.FLASH_OUT if flash_only else build.OUT
            if not build.up_to_date(out):
                build.build(flash_only=flash_only)


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def checksum(t):
    return float(t.double().sum()), float(t.double().abs().sum())


def assert_same_inputs(stored, tensor, what):
    """The fixtures hold outputs only; inputs are regenerated from seeds. Fail loudly if the generator drifted."""
    got = checksum(tensor)
    assert np.allclose(np.asarray(stored)[:2], got, rtol=1e-9, atol=1e-9), (
        f"seeded {what} no longer reproduces the tensor the golden fixture was made from "
        f"(stored checksum {np.asarray(stored)[:2]}, now {got}): regenerate tests/golden with make_golden.py")


@pytest.fixture(scope="session")
def oracle():
    from oracle import vit_oracle
    return vit_oracle
