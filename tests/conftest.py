import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    here = os.path.join(ROOT, "tests", "golden")
    return {name: np.load(os.path.join(here, name + ".npz"))
            for name in ("preprocess", "misc", "gemv_int4")}


@pytest.fixture(scope="session")
def cuda_lib():
    """The C ABI library on a CUDA device; fails (never skips) when the device is there but the
    library is not."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from mixed_gemv_b200 import _lib
    return _lib.load()
