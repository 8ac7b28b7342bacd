import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def from_bf16_bits(a: np.ndarray) -> torch.Tensor:
    """Inverse of the fixture encoding: raw int16 bit patterns -> bfloat16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(GOLDEN / name)
    return load


@pytest.fixture(scope="session")
def cuda_dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)
