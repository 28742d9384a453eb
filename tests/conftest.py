"""Shared test plumbing.  GPU tests carry @pytest.mark.gpu; everything else runs on CPU.

The oracle under oracle/ is test infrastructure: tests import it, the package never does.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"
for p in (str(ROOT), str(ROOT / "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def load_golden(name: str) -> dict:
    with np.load(GOLDEN / name, allow_pickle=False) as z:
        return {k: z[k] for k in z.files}


def params_from(blob: dict, prefix: str = "w::") -> dict:
    return {k[len(prefix):]: v for k, v in blob.items() if k.startswith(prefix)}


@pytest.fixture(scope="session")
def engine_lib():
    """The built shared library (compiled on demand where nvcc exists)."""
    from connect6_b200 import build
    if build.is_stale():
        build.build()
    from connect6_b200 import _lib
    return _lib.load()


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)
