import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_python.npz"))


@pytest.fixture(scope="session")
def backend():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from speedoza_b200.backend import CudaBackend
    return CudaBackend()


def to_dev(a, dtype=None):
    """numpy -> cuda tensor; uint16 arrays are reinterpreted as bf16."""
    import numpy as np
    import torch
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16).copy()).cuda().view(torch.bfloat16)
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def bf16_host(t):
    """cuda bf16 tensor -> numpy uint16 bit patterns."""
    import numpy as np
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
