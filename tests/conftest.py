"""Shared test configuration: the ``gpu`` marker, repo root on sys.path, fixtures."""
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
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def load_golden(name: str):
    return np.load(os.path.join(GOLDEN, name))


def bf16_from_bits(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def grid_i8_from_codes(codes: torch.Tensor) -> torch.Tensor:
    """4-bit E2M1 codes -> 2 * decoded value as int8 (so that -0 == +0)."""
    lut = torch.tensor([0, 1, 2, 3, 4, 6, 8, 12], dtype=torch.int8)
    mag = lut[(codes & 7).long()]
    return torch.where((codes & 8) != 0, -mag, mag)


@pytest.fixture(scope="session")
def oracle():
    import oracle as orc
    orc.lib()
    return orc
