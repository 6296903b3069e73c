"""The reference's own test plan, restated against this package.

flash-attention-triton checks its operator (tests/test_flash_attention_2.py) on five shapes with
fp32 CUDA inputs drawn by torch.randn: output shape / dtype / NaN (lines 232-273), agreement with
attention written out by its definition (275-297) and with torch's scaled_dot_product_attention
(300-318) at atol=1e-2, rtol=1e-3, bitwise repeatability in the deterministic mode (321-342) and
equality of the custom and the default entry point (345-411).  The same plan runs here through the
same public names, plus what the reference leaves out: the gradients are compared too.
"""

from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

from conftest import elementwise_tolerance

from flash_attention_triton_b200 import (KernelsConfigV2, _lib, flash_attention_v2,
                                         flash_attention_v2_custom, init_to_zero_v2)

pytestmark = pytest.mark.gpu

# (batch, heads, seqlen, headdim): the reference's "small" .. "large+" (lines 22-29)
SHAPES = {
    "small": (8, 12, 512, 32),
    "medium": (16, 16, 1024, 48),
    "medium+": (32, 20, 1024, 64),
    "large": (32, 20, 1024, 96),
    "large+": (64, 32, 2048, 128),
}
ATOL, RTOL = 1e-2, 1e-3  # the reference's output tolerance


def draw(shape, seed=42):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v, do = (torch.randn(*shape, device="cuda", dtype=torch.float32, generator=g) for _ in range(4))
    return q, k, v, do, 1.0 / shape[-1] ** 0.5


def forward_backward(fn, q, k, v, do, *args, **kwargs):
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    out = fn(q, k, v, *args, **kwargs)
    out.backward(do)
    return out.detach(), q.grad, k.grad, v.grad


@pytest.mark.parametrize("name", list(SHAPES))
def test_output_shape_dtype_and_finiteness(name):
    q, k, v, _, scale = draw(SHAPES[name])
    out = flash_attention_v2(q, k, v, scale)
    assert out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous()
    assert torch.isfinite(out).all()
    assert _lib.device_status() == 0


@pytest.mark.parametrize("name", list(SHAPES))
def test_agrees_with_attention_by_definition(name):
    """softmax(mask(q k^T * scale)) v with an explicit upper-triangular mask, in fp32, a few batch
    entries at a time so that the score tensor stays small."""
    q, k, v, _, scale = draw(SHAPES[name])
    out = flash_attention_v2(q, k, v, scale)
    n = q.shape[2]
    mask = torch.ones(n, n, dtype=torch.bool, device="cuda").triu(1)
    for b0 in range(0, q.shape[0], 4):
        sl = slice(b0, b0 + 4)
        scores = (q[sl] @ k[sl].transpose(-2, -1)) * scale
        want = torch.softmax(scores.masked_fill(mask, float("-inf")), dim=-1) @ v[sl]
        assert torch.allclose(out[sl], want, atol=ATOL, rtol=RTOL), (name, b0)


@pytest.mark.parametrize("name", list(SHAPES))
def test_agrees_with_torch_sdpa_including_gradients(name):
    q, k, v, do, scale = draw(SHAPES[name])
    ours = forward_backward(flash_attention_v2, q, k, v, do, scale)
    theirs = forward_backward(
        lambda a, b, c: F.scaled_dot_product_attention(a, b, c, is_causal=True, scale=scale), q, k, v, do)
    assert torch.allclose(ours[0], theirs[0], atol=ATOL, rtol=RTOL), "output"
    # Gradients: the kernels compute in fp16 (the reference's dtype policy for fp32 inputs,
    # flash_attention_2.py:316), so the comparison that isolates kernel error is against torch's
    # fp32 attention on the SAME fp16-rounded inputs, element by element within
    # max(5e-3, one fp16 ulp of the element's own value).
    q16, k16, v16, do16 = (t.half().float() for t in (q, k, v, do))
    exact = forward_backward(
        lambda a, b, c: F.scaled_dot_product_attention(a, b, c, is_causal=True, scale=scale), q16, k16, v16, do16)
    for label, a, b in zip(("dq", "dk", "dv"), ours[1:], exact[1:]):
        over = ((a - b).abs().double() - elementwise_tolerance(torch.float16, b)).max().item()
        assert over <= 0, (label, (a - b).abs().max().item(), over)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("name", list(SHAPES))
def test_deterministic_mode_repeats_bit_for_bit(name):
    q, k, v, do, scale = draw(SHAPES[name])
    first = forward_backward(flash_attention_v2, q, k, v, do, scale, deterministic=True)
    for _ in range(5):
        again = forward_backward(flash_attention_v2, q, k, v, do, scale, deterministic=True)
        for a, b in zip(first, again):
            assert torch.equal(a, b)


@pytest.mark.parametrize("name", ["small", "large"])
def test_custom_entry_point_equals_default(name):
    """The custom entry point with a configuration for this GPU equals the default one bit for bit
    (reference lines 345-411); tile and warp knobs are accepted and ignored here."""

    class FakeTritonConfig:  # carries what triton.Config carries for the reference
        def __init__(self, kwargs, num_warps, num_stages, pre_hook):
            self.kwargs, self.num_warps, self.num_stages, self.pre_hook = kwargs, num_warps, num_stages, pre_hook

    q, k, v, do, scale = draw(SHAPES[name])
    cc = torch.cuda.get_device_capability()
    for seq_parallel in (False, True):
        cfg = KernelsConfigV2(128, 128, 32, 256, 32, 8, 16, 1, [
            FakeTritonConfig({"BLOCK_Q_ROWS_SIZE": 128, "BLOCK_KV_COLS_SIZE": 128,
                              "SEQUENCE_PARALLEL": seq_parallel}, 8, 1, init_to_zero_v2("DQ"))])
        custom = forward_backward(flash_attention_v2_custom, q, k, v, do, scale, {cc: cfg})
        default = forward_backward(flash_attention_v2, q, k, v, do, scale, deterministic=not seq_parallel)
        assert torch.equal(custom[0], default[0])
        if not seq_parallel:  # atomics are not repeatable; the deterministic pair must be identical
            for a, b in zip(custom[1:], default[1:]):
                assert torch.equal(a, b)
