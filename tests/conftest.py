"""Shared fixtures and markers.  Tests marked ``gpu`` need a B200; everything else runs on CPU."""
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
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


def load_golden(name: str):
    return np.load(os.path.join(GOLDEN, name))


def from_np(a: np.ndarray, bf16: bool = False) -> torch.Tensor:
    """numpy -> torch; uint16 arrays flagged ``bf16`` are bit patterns of bfloat16."""
    if bf16:
        return torch.from_numpy(a.astype(np.int16)).view(torch.bfloat16)
    return torch.from_numpy(a.copy())


def golden_tensor(z, key: str) -> torch.Tensor:
    a = z[key]
    return from_np(a, bf16=(a.dtype == np.uint16))


@pytest.fixture(scope="session")
def cuda_dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
