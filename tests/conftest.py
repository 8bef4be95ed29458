import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def built_library():
    """Path of libsharpnet_b200.so, compiled on demand (nvcc cross-compiles without a GPU)."""
    from sharpnet_b200.build import build_library
    return build_library()


@pytest.fixture(scope="session")
def wrapper(built_library):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from sharpnet_b200.tensor import GPUWrapper
    return GPUWrapper.FromDeviceId(0)


@pytest.fixture()
def golden():
    import json
    with open(os.path.join(ROOT, "tests", "golden", "reference_vectors.json")) as f:
        return json.load(f)
