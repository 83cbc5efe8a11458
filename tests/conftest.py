import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def load_golden(name: str) -> dict:
    """Load tests/golden/<name>.npz as torch tensors (``__bf16`` keys are bit patterns)."""
    out = {}
    with np.load(GOLDEN / f"{name}.npz") as data:
        for key in data.files:
            value = torch.from_numpy(data[key].copy())
            if key.endswith("__bf16"):
                out[key[:-6]] = value.view(torch.bfloat16)
            else:
                out[key] = value
    return out


@pytest.fixture(scope="session")
def golden():
    return load_golden


@pytest.fixture(scope="session")
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)


def max_abs_rel(actual: torch.Tensor, reference: torch.Tensor) -> float:
    """max|a - r| / max|r|  - the benchmark's tolerance is 2e-2 on this quantity."""
    reference = reference.double()
    scale = reference.abs().max().item()
    return (actual.double() - reference).abs().max().item() / (scale if scale > 0 else 1.0)
