"""Shared pytest configuration: the ``gpu`` marker and helpers used by both CPU and GPU tests."""

from __future__ import annotations

import math
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def make_inputs(shape, dtype, seed=0, qk_mul=1.0):
    """Seeded inputs as BASELINE configs describe them: q, k, v, dO iid N(0,1) drawn in fp32 on a
    CPU generator in that order, q and k optionally scaled, then rounded to ``dtype``."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q, k, v, do = (torch.randn(*shape, generator=g) for _ in range(4))
    q, k = q * qk_mul, k * qk_mul
    return tuple(t.to(dtype) for t in (q, k, v, do))


def default_scale(d):
    return 1.0 / math.sqrt(d)
