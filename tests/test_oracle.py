"""The oracle pinned against the reference: golden vectors produced by the reference's own
Triton kernels (CPU interpreter, see tests/golden/make_golden.py)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR
from oracle.attention_oracle import naive_attention, naive_attention_per_head, reference_tiled

GOLDEN = sorted(GOLDEN_DIR.glob("*.npz"))


def test_golden_files_present():
    assert len(GOLDEN) >= 6


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_restatement_matches_reference_kernels(path):
    """The numpy restatement reproduces the reference kernels: bit-exact for four of the six
    cases (square and more-keys-than-queries).  In the d=128 case BLAS blocking reorders a
    128-long fp32 sum, and in the fewer-keys case ten lse values differ in the last fp32 bit
    (numpy's exp/log against the interpreter's); either can move a result across an fp16
    rounding boundary, so the bound there is one fp16 ulp (2^-10 relative, 5e-4 absolute near
    zero)."""
    z = np.load(path)
    r = reference_tiled(
        z["q"], z["k"], z["v"], z["dout"], float(z["softmax_scale"]),
        int(z["fwd_block"]), int(z["fwd_block"]), int(z["bwd_block"]),
    )
    exact = "d128" not in path.stem and "fewer_keys" not in path.stem
    for key in ("o", "dq", "dk", "dv"):
        if exact:
            assert np.array_equal(r[key], z[key]), key
        else:
            np.testing.assert_allclose(
                r[key].astype(np.float32), z[key].astype(np.float32), rtol=2**-10, atol=5e-4
            )
    np.testing.assert_allclose(r["lse"], z["lse"], rtol=0, atol=0 if exact else 2e-6)


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_naive_oracle_agrees_with_reference_kernels(path):
    """The closed-form fp64 oracle and the reference agree to fp16 rounding of the outputs:
    max-abs 5e-3 where |x| stays O(1), and 2 fp16 ulps of the largest value otherwise."""
    z = np.load(path)
    nv = naive_attention(
        *(torch.from_numpy(z[x]) for x in ("q", "k", "v", "dout")),
        softmax_scale=float(z["softmax_scale"]),
    )
    for key in ("o", "dq", "dk", "dv"):
        want = nv[key].numpy()
        tol = max(5e-3, 2 * float(np.spacing(np.float16(np.abs(want).max()))))
        assert np.abs(z[key].astype(np.float64) - want).max() <= tol, key
    assert np.abs(z["lse"].astype(np.float64) - nv["lse"].numpy()).max() <= 1e-4


def test_naive_gradients_match_autograd():
    g = torch.Generator().manual_seed(1)
    q, k, v, do = (torch.randn(1, 2, 37, 16, generator=g, dtype=torch.float64) for _ in range(4))
    r = naive_attention(q, k, v, do, 0.3)
    qa, ka, va = (t.clone().requires_grad_() for t in (q, k, v))
    s = (qa @ ka.transpose(-1, -2)) * 0.3
    s = s.masked_fill(~torch.ones(37, 37, dtype=torch.bool).tril(), float("-inf"))
    (torch.softmax(s, -1) @ va).backward(do)
    for key, t in (("dq", qa), ("dk", ka), ("dv", va)):
        torch.testing.assert_close(r[key], t.grad, rtol=1e-10, atol=1e-10)


def test_per_head_loop_equals_batched():
    g = torch.Generator().manual_seed(2)
    q, k, v, do = (torch.randn(2, 3, 40, 8, generator=g) for _ in range(4))
    a = naive_attention(q, k, v, do, None, torch.float32)
    b = naive_attention_per_head(q, k, v, do, None, torch.float32)
    for key in a:
        torch.testing.assert_close(a[key], b[key], rtol=1e-6, atol=1e-6)


def test_zero_scale_means_default():
    """softmax_scale=0.0 is treated as unset, as `softmax_scale or ...` does in the reference
    (flash_attention_2.py:94)."""
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(1, 1, 16, 32, generator=g) for _ in range(3))
    a = naive_attention(q, k, v, None, 0.0)
    b = naive_attention(q, k, v, None, None)
    torch.testing.assert_close(a["o"], b["o"])
