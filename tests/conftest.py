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
    """Seeded inputs: q, k, v, dO iid N(0,1) drawn in fp32 on a CPU generator in that order,
    q and k optionally scaled (a peaked softmax), then rounded to ``dtype``."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q, k, v, do = (torch.randn(*shape, generator=g) for _ in range(4))
    q, k = q * qk_mul, k * qk_mul
    return tuple(t.to(dtype) for t in (q, k, v, do))


def default_scale(d):
    return 1.0 / math.sqrt(d)


# --------------------------------------------------------------------------- tolerances
#: max-abs bounds against the fp64 oracle on the same 16-bit inputs
BASE_TOL = {torch.float16: 5e-3, torch.bfloat16: 2e-2}
#: explicit mantissa bits of the output formats
MANTISSA_BITS = {torch.float16: 10, torch.bfloat16: 7}


def elementwise_tolerance(dtype, ref):
    """Per-element error bound: the stated max-abs bound (5e-3 for fp16, 2e-2 for bf16), or one
    unit in the last place of the element's OWN oracle value where that is larger (an output
    rounded to 16 bits cannot be closer than half an ulp to the exact value, so a flat bound is
    unattainable for |x| >= 8 in fp16 and |x| >= 4 in bf16)."""
    mag = ref.detach().double().abs().clamp_min(2.0**-60)
    ulp = torch.exp2(torch.floor(torch.log2(mag)) - MANTISSA_BITS[dtype])
    return ulp.clamp_min(BASE_TOL[dtype])


def error_stats(got, ref):
    """max-abs and rms error of ``got`` against ``ref`` (both taken to fp64 on ref's device)."""
    d = got.detach().to(ref.device, torch.float64) - ref.detach().double()
    return d.abs().max().item(), d.pow(2).mean().sqrt().item()


#: "never worse than the reference's own error", as a factor on the rms error of the reference's
#: arithmetic (oracle.reference_tiled) on the same inputs.  fp16: the same arithmetic, so the same
#: error level (25 % covers sampling noise).  bf16: the reference computes bf16 problems in fp16
#: (flash_attention_2.py:316), so its P and dS carry 11 significant bits against the 8 of the
#: bf16 P and dS here; next to the rounding of the bf16 output that makes the rms error 1.25x
#: (O) to 1.45x (dq, dk) the reference's at N = 8192 .. 32768 with the default scale, and 1.75x
#: (dq) on a short, peaked problem (N = 257, scale 0.3).  An fp16 P / dS beside bf16 operands
#: would close the gap, but the tensor core refuses that operand mix.
RMS_FACTOR_VS_REFERENCE = {torch.float16: 1.25, torch.bfloat16: 2.0}
#: The same for the maximum error, which is a tail value over 1e5 .. 1e7 elements quantised in
#: ulps of the output: within 2x of the reference's for fp16, and 1.6x that for bf16.
MAX_FACTOR_VS_REFERENCE = {torch.float16: 2.0, torch.bfloat16: 3.2}
