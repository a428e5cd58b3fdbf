"""Shared pytest set-up: the ``gpu`` marker, import paths, golden loader."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str):
    return np.load(GOLDEN / name)


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """max|a-b| / (max|b| + 1e-6): the reference's own measure
    (kernels/cuda_fused_sparse_splitk.py:3096, :3102)."""
    a, b = a.double(), b.double()
    return float((a - b).abs().max() / (b.abs().max() + 1e-6))


def corr_diff(a: torch.Tensor, b: torch.Tensor) -> float:
    """1 - 2<a,b>/(|a|^2+|b|^2) (kernels/cuda_fused_sparse_splitk.py:2944-2947)."""
    a, b = a.double(), b.double()
    n = (a * a + b * b).sum()
    return 0.0 if n == 0 else float(1.0 - 2 * (a * b).sum() / n)
