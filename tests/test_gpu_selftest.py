"""Single-tile tensor-core self-test through the C ABI: each operand form the attention
kernels rely on (K-major shared memory, tensor-memory A operand, MN-major shared memory)
against a plain fp64 matrix product."""

from __future__ import annotations

import pytest
import torch

from flash_attention_triton_b200 import _lib

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["fp16", "bf16"])
@pytest.mark.parametrize("d", [32, 64, 128])
@pytest.mark.parametrize("form", [0, 1, 2])
def test_mma_operand_forms(form, d, dtype):
    g = torch.Generator().manual_seed(100 * form + d)
    a = torch.randn(128, d if form == 0 else 128, generator=g).to(dtype)
    b = torch.randn(128, d, generator=g).to(dtype)
    ad64, bd64 = a.double(), b.double()
    ref = ad64 @ bd64.T if form == 0 else (ad64 @ bd64 if form == 1 else ad64.T @ bd64)
    ad, bd = a.cuda(), b.cuda()
    c = torch.full(ref.shape, float("nan"), device="cuda", dtype=torch.float32)
    rc = _lib.lib().fa2_selftest_mma(form, ad.data_ptr(), bd.data_ptr(), c.data_ptr(), d,
                                     0 if dtype == torch.float16 else 1,
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert _lib.device_status() == 0
    # fp32 accumulation of exact 16-bit products: error is a few fp32 ulps of the result
    assert (c.cpu().double() - ref).abs().max().item() < 1e-3


def test_a_lost_signal_ends_in_a_status_word_not_in_a_hang():
    """Two warps wait for a barrier nobody arrives at; the bounded wait gives up after about two
    seconds, the kernel ends by itself, fa2_device_status reports where, and the next kernel runs
    as if nothing had happened."""
    lib = _lib.lib()
    assert _lib.device_status() == 0
    assert lib.fa2_selftest_wait_timeout(torch.cuda.current_stream().cuda_stream) == 0
    assert _lib.device_status() == (0x10000 | 120)
    assert _lib.device_status() == 0  # reading clears it
    q = torch.randn(1, 1, 128, 64, device="cuda", dtype=torch.float16)
    from flash_attention_triton_b200 import flash_attention_v2

    out = flash_attention_v2(q, q, q)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all() and _lib.device_status() == 0
