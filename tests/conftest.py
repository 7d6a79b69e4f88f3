"""Shared test configuration: the ``gpu`` marker, import path, seeding and helpers."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(autouse=True)
def _seed():
    """Seed like the reference's autouse fixture (tests/conftest.py:23-33, seed 42)."""
    np.random.seed(42)
    try:
        import torch

        torch.manual_seed(42)
    except Exception:  # pragma: no cover
        pass
    yield


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def seeded_bf16(seed: int, shape, scale: float = 1.0):
    """BF16 tensor from a CPU generator, so CPU oracle and GPU see identical bits
    (tests/quantization/test_bf16_to_fp4_tma.py:326-342)."""
    import torch

    gen = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=gen, dtype=torch.float32) * scale).to(torch.bfloat16)
