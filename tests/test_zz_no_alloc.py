"""fa2_bwd_static_scratch: the backward for callers that cannot allocate device memory.

Some users of this library sit inside code that must not call cudaMalloc at all: a replayed
inference / training loop whose memory plan is frozen, a plugin living under somebody else's
allocator, a latency-critical server where a device-wide synchronising allocation is not
acceptable.  For them the library carries its own 4 MiB scratch array (the row statistics of
the backward) and this entry point uses it instead of a caller workspace.

The test calls the entry point through the C ABI, twice in a row on the same stream (the
second call reuses the array with the first call's contents still in it), and compares with
the ordinary path (fa2_bwd_preprocess + fa2_bwd, deterministic) — same kernels, same order of
operations, so the results must be bit-identical (tolerance 0).  It also checks that a problem
larger than the built-in scratch is refused cleanly.
"""

from __future__ import annotations

import math

import pytest
import torch

from conftest import make_inputs
from flash_attention_triton_b200 import _lib

pytestmark = pytest.mark.gpu


def _forward(lib, q, k, v, scale, code):
    b, h, n, d = q.shape
    o = torch.empty_like(q)
    lse = torch.empty(b, h, n, device=q.device, dtype=torch.float32)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.fa2_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                       b, h, n, d, code, scale, st) == 0
    return o, lse


def _backward_with_workspace(lib, q, k, v, o, do, lse, scale, code):
    b, h, n, d = q.shape
    st = torch.cuda.current_stream().cuda_stream
    rs = torch.empty(lib.fa2_rowstats_bytes(b, h, n) // 4, device=q.device, dtype=torch.float32)
    assert lib.fa2_bwd_preprocess(o.data_ptr(), do.data_ptr(), lse.data_ptr(), rs.data_ptr(),
                                  b, h, n, d, code, st) == 0
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    assert lib.fa2_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr(), rs.data_ptr(),
                       dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), None, 0,
                       b, h, n, d, code, scale, 1, st) == 0
    return dq, dk, dv


def _backward_static(lib, q, k, v, o, do, lse, scale, code):
    b, h, n, d = q.shape
    st = torch.cuda.current_stream().cuda_stream
    dq, dk, dv = (torch.full_like(q, float("nan")) for _ in range(3))
    rc = lib.fa2_bwd_static_scratch(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                    do.data_ptr(), lse.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                                    dv.data_ptr(), b, h, n, d, code, scale, st)
    assert rc == 0, lib.fa2_strerror(rc)
    return dq, dk, dv


def test_static_scratch_backward_matches_workspace_backward_twice():
    lib = _lib.lib()
    # two different problems back to back: the second finds the first one's row statistics
    # (other N, other tile count) still in the built-in array
    for shape, dtype in (((2, 3, 777, 64), torch.bfloat16), ((1, 4, 300, 128), torch.float16)):
        code = 0 if dtype == torch.float16 else 1
        scale = 1.0 / math.sqrt(shape[-1])
        q, k, v, do = (t.cuda() for t in make_inputs(shape, dtype, seed=5))
        o, lse = _forward(lib, q, k, v, scale, code)
        want = _backward_with_workspace(lib, q, k, v, o, do, lse, scale, code)
        for _ in range(2):
            got = _backward_static(lib, q, k, v, o, do, lse, scale, code)
            assert _lib.device_status() == 0
            for name, g, w in zip(("dq", "dk", "dv"), got, want):
                assert not torch.isnan(g).any(), name
                assert torch.equal(g, w), name  # tolerance 0: identical kernels and order


def test_static_scratch_rejects_oversized_problem_without_launching():
    lib = _lib.lib()
    # B*H*ceil(N/128) = 65 * 64 = 4160 > 4096 tiles; pointers are never dereferenced
    rc = lib.fa2_bwd_static_scratch(*([0x1000] * 9), 1, 65, 8192, 128, 1, 0.1, None)
    assert rc == -11
    assert b"4096" in lib.fa2_strerror(rc)
