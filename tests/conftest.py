import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(GOLDEN, "reference_cpu.npz"))


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The C-ABI library must exist for every test; build it if the tree is fresh."""
    from fastermoe_b200 import build
    build.build()


@pytest.fixture(autouse=True)
def _seeded(request):
    """Every test draws the same random inputs in every run, whatever ran before it: torch's generators
    (CPU and CUDA) are seeded from the test's id.  A tolerance that holds is then one that holds again."""
    import zlib
    import torch
    torch.manual_seed(zlib.crc32(request.node.nodeid.encode()) & 0x7FFFFFFF)
