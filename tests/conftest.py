import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tallax_b200 import _lib

    _lib.load()  # raises if the in-tree library is missing: GPU tests never fall back
    return torch.device("cuda:0")


def to_np(t):
    import torch

    if t.dtype == torch.bfloat16:
        import ml_dtypes

        return t.detach().cpu().view(torch.int16).numpy().view(ml_dtypes.bfloat16)
    return t.detach().cpu().numpy()


def to_dev(a, device):
    import torch

    a = np.ascontiguousarray(a)
    if a.dtype.name == "bfloat16":
        return torch.from_numpy(a.view(np.int16)).to(device).view(torch.bfloat16)
    return torch.from_numpy(a).to(device)


def exact_match(x, y):
    """array_equal with NaNs equal and -0 == +0: the reference's exact_match (test_utils.py:17-21)."""
    x = np.asarray(x)
    y = np.asarray(y)
    if x.dtype.name == "bfloat16":
        x = x.astype(np.float32)
    if y.dtype.name == "bfloat16":
        y = y.astype(np.float32)
    return x.shape == y.shape and bool(np.array_equal(x, y, equal_nan=x.dtype.kind == "f"))
