import os
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
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name):
    """Load a fixture written by tests/golden/make_golden.py; restores bf16/fp16 tensors."""
    out = {}
    with np.load(GOLDEN / f"{name}.npz") as z:
        for k in z.files:
            a = z[k]
            if k.endswith("__bf16"):
                out[k[:-6]] = torch.from_numpy(a.copy()).view(torch.bfloat16)
            elif k.endswith("__fp16"):
                out[k[:-6]] = torch.from_numpy(a.copy()).view(torch.float16)
            elif a.ndim == 0:
                out[k] = a.item()
            else:
                out[k] = torch.from_numpy(a.copy())
    return out


@pytest.fixture
def golden():
    return load_golden


@pytest.fixture
def device():
    return "cuda"
