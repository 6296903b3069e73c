"""GPU parity: the sm_100a kernels against the CPU oracle, the reference-generated golden
vectors, and size-independent properties.  Everything here calls the C ABI (directly through
ctypes, or through the Python surface that wraps it).

Tolerances, measured on the FINAL tensors against the fp64 closed-form oracle evaluated on the
same 16-bit inputs:
    fp16 outputs: max-abs <= 5e-3          bf16 outputs: max-abs <= 2e-2
applied element by element, with one escape: an element whose own oracle value is so large that
one unit in its last place exceeds the bound may be off by that one ulp (|x| >= 8 in fp16,
|x| >= 4 in bf16; conftest.elementwise_tolerance).  The third criterion, "never worse than the
reference's own error", is what binds where not even the reference's arithmetic meets the flat
bound (peaked softmax, gradients of tens accumulated from 16-bit dS tiles): there the error is
compared with that of the restatement of the reference's kernels (oracle.reference_tiled,
pinned to their outputs by tests/test_oracle.py) on the same inputs.
"""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from conftest import (BASE_TOL, GOLDEN_DIR, MAX_FACTOR_VS_REFERENCE, RMS_FACTOR_VS_REFERENCE, elementwise_tolerance, error_stats,
                      make_inputs)
from flash_attention_triton_b200 import (
    KernelsConfigV2,
    _lib,
    flash_attention_v2,
    flash_attention_v2_custom,
    shard_slab,
)
from oracle.attention_oracle import naive_attention, naive_attention_per_head, reference_tiled

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_api(q, k, v, do, scale, det, dev=DEV):
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    out = flash_attention_v2(qd, kd, vd, scale, deterministic=det)
    out.backward(do.to(dev))
    with torch.cuda.device(dev):
        assert _lib.device_status() == 0
    return {"o": out.detach(), "dq": qd.grad, "dk": kd.grad, "dv": vd.grad}


def run_api_no_sync(q, k, v, do, scale, det, dev=DEV):
    """Like run_api on the current stream, without reading the status word (which synchronises)."""
    qd, kd, vd = (t.to(dev, non_blocking=True).requires_grad_(True) for t in (q, k, v))
    out = flash_attention_v2(qd, kd, vd, scale, deterministic=det)
    out.backward(do.to(dev, non_blocking=True))
    return {"o": out.detach(), "dq": qd.grad, "dk": kd.grad, "dv": vd.grad}


def check_against(ref, got, dtype, keys=("o", "dq", "dk", "dv")):
    """Every element within max(5e-3 | 2e-2, one ulp of its own oracle value)."""
    problems = []
    for key in keys:
        want = ref[key].double()
        g = got[key].detach().to(want.device, torch.float64)
        assert not torch.isnan(g).any(), key
        err = (g - want).abs()
        excess = (err - elementwise_tolerance(dtype, want)).max().item()
        if excess > 0:
            problems.append(f"{key}: max-abs error {err.max().item():.3e}, {excess:.3e} over the bound")
    assert not problems, "; ".join(problems)


def check_not_worse_than_reference(q, k, v, do, scale, got, ref, dtype, keys=("dq", "dk", "dv"),
                                   block=128):
    """"Never worse than the reference's own error": the reference computes in fp16 whatever the
    input dtype (flash_attention_2.py:316,339,379) and returns the input dtype, so its side is
    reference_tiled on the inputs cast to fp16 with the outputs rounded to ``dtype``.  Ours
    must have the same error level (rms within conftest.RMS_FACTOR_VS_REFERENCE) and a maximum
    within conftest.MAX_FACTOR_VS_REFERENCE of the reference's, or meet the flat bound."""
    d = q.shape[-1]
    theirs = reference_tiled(q.half().numpy(), k.half().numpy(), v.half().numpy(), do.half().numpy(),
                             scale or 1.0 / math.sqrt(d), block, block, block)
    report = {}
    for key in keys:
        want = ref[key].double().cpu()
        t = torch.from_numpy(theirs[key].astype(np.float32)).to(dtype).double()
        e_ref, rms_ref = error_stats(t, want)
        e_ours, rms_ours = error_stats(got[key].cpu(), want)
        report[key] = {"max_ours": e_ours, "max_ref": e_ref, "rms_ours": rms_ours, "rms_ref": rms_ref}
        assert rms_ours <= RMS_FACTOR_VS_REFERENCE[dtype] * rms_ref + 1e-5, \
            f"{key}: rms ours {rms_ours:.3e}, reference {rms_ref:.3e}"
        assert e_ours <= max(BASE_TOL[dtype], MAX_FACTOR_VS_REFERENCE[dtype] * e_ref), \
            f"{key}: ours {e_ours:.3e}, reference {e_ref:.3e}"
    return report


# --------------------------------------------------------------------------- oracle parity
CASES = [
    # (shape, dtype, scale, qk_mul) — C1 and reduced C2/C3/C5 shapes, ragged tails, odd tile counts
    ((2, 4, 256, 64), torch.float16, None, 1.0),
    ((1, 4, 2048, 64), torch.float16, None, 1.0),
    ((1, 2, 1024, 128), torch.bfloat16, None, 1.0),
    ((1, 2, 2048, 128), torch.float16, None, 1.0),
    ((2, 3, 1023, 32), torch.float16, 0.5, 3.0),
    # head dims between the instantiated 32 / 64 / 128 (the reference's own test shapes use 48
    # and 96, tests/test_flash_attention_2.py:23-29) and one that is not a multiple of 8
    ((2, 2, 1024, 48), torch.float16, None, 1.0),
    ((1, 3, 1000, 96), torch.bfloat16, None, 1.0),
    ((1, 2, 300, 8), torch.float16, None, 1.0),
    ((1, 2, 333, 72), torch.float16, None, 1.0),
    ((1, 2, 200, 20), torch.float16, None, 1.0),
    ((1, 2, 1, 64), torch.float16, None, 1.0),
    ((1, 2, 7, 32), torch.bfloat16, None, 1.0),
    ((1, 1, 127, 128), torch.bfloat16, None, 1.0),
    ((1, 1, 129, 128), torch.float16, None, 1.0),
    ((1, 2, 257, 64), torch.bfloat16, 0.3, 1.0),
    ((1, 2, 640, 32), torch.bfloat16, None, 1.0),
    ((3, 1, 385, 128), torch.bfloat16, None, 1.0),
]


@pytest.mark.parametrize("mode", ["spill", "recompute", "atomic"])
@pytest.mark.parametrize("shape,dtype,scale,qk_mul", CASES,
                         ids=[f"{'x'.join(map(str, c[0]))}-{str(c[1])[6:]}" for c in CASES])
def test_forward_backward_match_oracle(shape, dtype, scale, qk_mul, mode, monkeypatch):
    """Every dQ strategy of the backward (the API picks one per shape; here each is forced).
    Where the softmax is peaked (a scale above 1/sqrt(d), or q, k of variance 9) gradients reach
    tens and not even the reference's arithmetic meets the flat bound on them; there O and dv
    keep the flat bound and dq, dk must not be worse than the reference's arithmetic."""
    monkeypatch.setenv("FA2_B200_BWD_MODE", mode)
    q, k, v, do = make_inputs(shape, dtype, seed=0, qk_mul=qk_mul)
    ref = naive_attention(q, k, v, do, scale)
    got = run_api(q, k, v, do, scale, mode != "atomic")
    if scale is not None or qk_mul != 1.0:
        check_against(ref, got, dtype, keys=("o", "dv"))
        check_not_worse_than_reference(q, k, v, do, scale, got, ref, dtype, keys=("dq", "dk"))
    else:
        check_against(ref, got, dtype)


def test_spill_mode_chunks_change_no_bit(monkeypatch):
    """With a scratch bound of 3 MiB the spill mode works through [3, 5, 700, 64] (0.7 MiB per
    head) in chunks of 3 + 2 heads per batch entry; with 8 MiB in chunks of 2 + 1 batch
    entries; unbounded in one piece.  Same bits every time, and dK, dV equal the recompute
    mode's."""
    monkeypatch.setenv("FA2_B200_BWD_MODE", "spill")
    q, k, v, do = make_inputs((3, 5, 700, 64), torch.float16, seed=4)
    lib = _lib.lib()
    previous = lib.fa2_set_spill_budget(1 << 40)
    try:
        whole = run_api(q, k, v, do, None, True)
        for budget in (3 << 20, 8 << 20, 1):
            lib.fa2_set_spill_budget(budget)
            assert lib.fa2_bwd_workspace_bytes(3, 5, 700, 64, 2) <= max(budget, 21 * 32768)
            chunked = run_api(q, k, v, do, None, True)
            for key in whole:
                assert torch.equal(chunked[key], whole[key]), (key, budget)
    finally:
        lib.fa2_set_spill_budget(previous)
    monkeypatch.setenv("FA2_B200_BWD_MODE", "recompute")
    recompute = run_api(q, k, v, do, None, True)
    assert torch.equal(recompute["dk"], whole["dk"]) and torch.equal(recompute["dv"], whole["dv"])
    assert (recompute["dq"].float() - whole["dq"].float()).abs().max() <= 2e-3


@pytest.mark.parametrize("d", [64, 256])
def test_spill_chunks_with_strided_tensors(d, monkeypatch):
    """The chunks of the spill mode are sub-ranges of the caller's tensors addressed through the
    caller's strides: [B, N, H, D] storage, fewer keys than queries, head dim 64 (one scratch) and
    256 (two scratches), chunked by a small budget; same bits as in one piece, parity with the oracle."""
    monkeypatch.setenv("FA2_B200_BWD_MODE", "spill")
    g = torch.Generator().manual_seed(11)
    q, do = (torch.randn(3, 500, 4, d, generator=g).to(torch.bfloat16).transpose(1, 2) for _ in range(2))
    k, v = (torch.randn(3, 300, 4, d, generator=g).to(torch.bfloat16).transpose(1, 2) for _ in range(2))
    ref = naive_attention(q, k, v, do)
    lib = _lib.lib()
    previous = lib.fa2_set_spill_budget(1 << 40)
    try:
        whole = run_api(q, k, v, do, None, True)
        check_against(ref, whole, torch.bfloat16)
        per_head = 10 * 32768 * (2 if d > 128 else 1)  # T = 4 Q tiles: 10 pairs
        for budget in (3 * per_head, 9 * per_head):     # 2 + 2 heads per batch entry; 2 + 1 batch entries
            lib.fa2_set_spill_budget(budget)
            chunked = run_api(q, k, v, do, None, True)
            for key in whole:
                assert torch.equal(chunked[key], whole[key]), (key, budget)
    finally:
        lib.fa2_set_spill_budget(previous)


def test_random_shapes_against_the_oracle(monkeypatch):
    """A seeded sweep over shapes the fixed cases do not name: sequence lengths 1..700 for queries
    and keys, head dims 8..256 in steps of 8, both dtypes, every dQ strategy, dense and
    [B, N, H, D]-strided storage."""
    import random

    rng = random.Random(1234)
    for case in range(36):
        nq = rng.choice([1, 2, 63, 64, 65, 127, 128, 129, 255, 256, 257]) if case % 3 == 0 else rng.randint(1, 700)
        nk = nq if case % 2 == 0 else rng.randint(1, 700)
        d = 8 * rng.randint(1, 32)
        b, h = rng.randint(1, 3), rng.randint(1, 3)
        dtype = rng.choice([torch.float16, torch.bfloat16])
        mode = rng.choice(["spill", "recompute", "atomic"])
        strided = rng.random() < 0.4
        monkeypatch.setenv("FA2_B200_BWD_MODE", mode)
        g = torch.Generator().manual_seed(case)
        if strided:
            q, do = (torch.randn(b, nq, h, d, generator=g).to(dtype).transpose(1, 2) for _ in range(2))
            k, v = (torch.randn(b, nk, h, d, generator=g).to(dtype).transpose(1, 2) for _ in range(2))
        else:
            q, do = (torch.randn(b, h, nq, d, generator=g).to(dtype) for _ in range(2))
            k, v = (torch.randn(b, h, nk, d, generator=g).to(dtype) for _ in range(2))
        ref = naive_attention(q, k, v, do)
        got = run_api(q, k, v, do, None, mode != "atomic")
        try:
            check_against(ref, got, dtype)
        except AssertionError as exc:
            raise AssertionError(f"case {case}: nq={nq} nk={nk} d={d} b={b} h={h} {dtype} {mode} "
                                 f"strided={strided}: {exc}") from exc


def test_calls_on_two_streams_do_not_disturb_each_other():
    """Forward and backward of two different problems issued alternately on two CUDA streams (the
    forward kernels draw work from per-call counters) give the bits of the serial runs."""
    a = make_inputs((2, 4, 1500, 128), torch.bfloat16, seed=21)
    b = make_inputs((3, 2, 900, 64), torch.float16, seed=22)
    want_a = run_api(*a, None, True)
    want_b = run_api(*b, None, True)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    for _ in range(3):
        outs = []
        for stream, inputs in ((s1, a), (s2, b), (s1, b), (s2, a)):
            with torch.cuda.stream(stream):
                outs.append(run_api_no_sync(*inputs, None, True))
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        for got, want in zip(outs, (want_a, want_b, want_b, want_a)):
            for key in want:
                assert torch.equal(got[key], want[key]), key


def test_lse_and_rowstats_through_the_c_abi():
    """fa2_fwd's LSE and fa2_bwd_preprocess's tile-blocked (-lse*log2e, -delta) array, ragged N."""
    b, h, n, d = 2, 3, 300, 64
    q, k, v, do = make_inputs((b, h, n, d), torch.bfloat16)
    ref = naive_attention(q, k, v, do)
    lib = _lib.lib()
    qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, do))
    o = torch.empty_like(qd)
    lse = torch.empty(b, h, n, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.fa2_fwd(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(),
                       b, h, n, d, 1, 1 / math.sqrt(d), st) == 0
    assert (lse.cpu().double() - ref["lse"]).abs().max() < 1e-4
    rs = torch.empty(lib.fa2_rowstats_bytes(b, h, n) // 4, device=DEV)
    assert lib.fa2_bwd_preprocess(o.data_ptr(), dod.data_ptr(), lse.data_ptr(), rs.data_ptr(),
                                  b, h, n, d, 1, st) == 0
    assert _lib.device_status() == 0
    t = 3
    tile_amax = rs[b * h * t * 256:].cpu().view(torch.int32).view(b * h, t)  # one word per tile
    rs = rs[: b * h * t * 256].view(b * h, t, 2, 128).cpu()
    lse2 = -rs[:, :, 0].reshape(b * h, t * 128)  # both vectors are stored negated
    delta = -rs[:, :, 1].reshape(b * h, t * 128)
    want_delta = (o.cpu().double() * do.double()).sum(-1).reshape(b * h, n)
    assert (delta[:, :n].double() - want_delta).abs().max() < 1e-5 * max(1.0, want_delta.abs().max())
    assert (lse2[:, :n].double() - lse.cpu().double().reshape(b * h, n) * math.log2(math.e)).abs().max() < 1e-5
    assert torch.isinf(lse2[:, n:]).all() and (lse2[:, n:] > 0).all()
    assert (delta[:, n:] == 0).all()
    # largest |dout| per 128-row tile, as the bf16 pattern with the sign cleared
    want_amax = torch.nn.functional.pad(do.abs().reshape(b * h, n, d), (0, 0, 0, t * 128 - n))
    want_amax = want_amax.reshape(b * h, t, 128 * d).amax(-1).view(torch.int16).to(torch.int32)
    assert torch.equal(tile_amax, want_amax)


@pytest.mark.parametrize("d, strided", [(32, False), (48, True), (64, True), (128, False), (128, True), (256, False)])
def test_preprocess_over_many_tiles_per_sm(d, strided):
    """fa2_bwd_preprocess on more tiles than one pass of the persistent CTAs covers (every CTA
    walks several tiles and its ring of stages wraps), ragged N, head dims below their padded
    width, rows contiguous (one bulk copy per tile) and strided (`[B, N, H, d]`: one per row)."""
    b, h, n = 3, 8, 128 * 39 + 77  # 3 * 8 * 40 = 960 tiles on 148 SMs
    g = torch.Generator().manual_seed(11)
    o = torch.randn(b, h, n, d, generator=g).to(torch.float16)
    do = (torch.randn(b, h, n, d, generator=g) * 3e-3).to(torch.float16)
    lse = torch.randn(b, h, n, generator=g).to(DEV)
    if strided:
        od, dod = (t.transpose(1, 2).contiguous().to(DEV).transpose(1, 2) for t in (o, do))
    else:
        od, dod = o.to(DEV), do.to(DEV)
    lib = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    rs = torch.full((lib.fa2_rowstats_bytes(b, h, n) // 4,), float("nan"), device=DEV)
    assert lib.fa2_bwd_preprocess_strided(od.data_ptr(), dod.data_ptr(), lse.data_ptr(), rs.data_ptr(),
                                          b, h, n, d, 0, _lib.stride_array(od, dod), st) == 0
    assert _lib.device_status() == 0
    t = 40
    tile_amax = rs[b * h * t * 256:].cpu().view(torch.int32).view(b * h, t)
    rs = rs[: b * h * t * 256].view(b * h, t, 2, 128).cpu()
    lse2 = -rs[:, :, 0].reshape(b * h, t * 128)
    delta = -rs[:, :, 1].reshape(b * h, t * 128)
    want_delta = (o.double() * do.double()).sum(-1).reshape(b * h, n)
    assert (delta[:, :n].double() - want_delta).abs().max() < 1e-5 * max(1.0, want_delta.abs().max().item())
    assert (lse2[:, :n].double() - lse.cpu().double().reshape(b * h, n) * math.log2(math.e)).abs().max() < 1e-5
    assert torch.isinf(lse2[:, n:]).all() and (delta[:, n:] == 0).all()
    want_amax = torch.nn.functional.pad(do.abs().reshape(b * h, n, d), (0, 0, 0, t * 128 - n))
    want_amax = want_amax.reshape(b * h, t, 128 * d).amax(-1).view(torch.int16).to(torch.int32)
    assert torch.equal(tile_amax, want_amax)


def test_fp32_inputs_follow_the_reference_dtype_policy():
    """fp32 in -> computed in fp16, output and grads returned as fp32 (flash_attention_2.py:316,339);
    the reference's own tests use fp32 inputs with atol 1e-2 on O (tests/test_flash_attention_2.py:297)."""
    q, k, v, do = make_inputs((2, 2, 512, 64), torch.float32)
    got = run_api(q, k, v, do, None, True)
    assert got["o"].dtype == torch.float32 and got["dq"].dtype == torch.float32
    ref = naive_attention(q.half(), k.half(), v.half(), do.half())
    check_against(ref, got, torch.float16)
    sdpa = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    torch.testing.assert_close(got["o"].cpu(), sdpa, atol=1e-2, rtol=1e-3)


def test_non_contiguous_inputs_are_accepted():
    q, k, v, do = make_inputs((1, 256, 2, 64), torch.float16)  # [B, N, H, D] storage
    qt, kt, vt, dot = (t.transpose(1, 2) for t in (q, k, v, do))
    got = run_api(qt, kt, vt, dot, None, True)
    ref = naive_attention(qt, kt, vt, dot)
    check_against(ref, got, torch.float16)


def test_transposed_inputs_are_read_in_place():
    """A [B, N, H, D] buffer viewed as [B, H, N, D] (what `x.view(B, N, H, D).transpose(1, 2)` of
    a projection gives) goes to the kernels as it is; the reference copies it
    (flash_attention_2.py:316)."""
    from flash_attention_triton_b200.api import _as_kernel_input

    q, k, v, do = make_inputs((2, 300, 3, 64), torch.bfloat16)  # [B, N, H, D] storage
    qt, kt, vt, dot = (t.transpose(1, 2) for t in (q, k, v, do))
    for t in (qt, kt, vt, dot):
        on_device = t.to(DEV)  # keeps the strides
        assert not on_device.is_contiguous() and _as_kernel_input(on_device) is on_device
    ref = naive_attention(qt, kt, vt, dot)
    for det in (True, False):
        got = run_api(qt, kt, vt, dot, None, det)
        check_against(ref, got, torch.bfloat16)
        assert got["o"].is_contiguous()


@pytest.mark.parametrize("det", [1, 0], ids=["det", "atomic"])
def test_packed_qkv_through_the_strided_c_abi(det):
    """q, k, v are slices of one [B, N, 3, H, D] buffer and dq, dk, dv are written straight into
    the matching slices of a gradient buffer of the same layout: no copy on either side."""
    b, h, n, d = 2, 3, 200, 96
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(b, n, 3, h, d, generator=g).to(torch.float16).to(DEV)
    do = torch.randn(b, n, h, d, generator=g).to(torch.float16).to(DEV).transpose(1, 2)
    q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
    dqkv = torch.full_like(qkv, float("nan"))
    dq, dk, dv = (dqkv[:, :, i].transpose(1, 2) for i in range(3))
    lib = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    scale = 1.0 / math.sqrt(d)
    o = torch.empty(b, h, n, d, device=DEV, dtype=torch.float16)
    lse = torch.empty(b, h, n, device=DEV, dtype=torch.float32)
    assert lib.fa2_fwd_strided(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                               lse.data_ptr(), b, h, n, n, d, 0, scale,
                               _lib.stride_array(q, k, v, o), st) == 0
    rs = torch.empty(lib.fa2_rowstats_bytes(b, h, n) // 4, device=DEV, dtype=torch.float32)
    assert lib.fa2_bwd_preprocess_strided(o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                                          rs.data_ptr(), b, h, n, d, 0,
                                          _lib.stride_array(o, do), st) == 0
    wsb = lib.fa2_bwd_workspace_bytes(b, h, n, d, det)
    ws = torch.empty(max(wsb, 256), device=DEV, dtype=torch.uint8)
    assert lib.fa2_bwd_strided(q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr(),
                               rs.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                               ws.data_ptr(), wsb, b, h, n, n, d, 0, scale, det,
                               _lib.stride_array(q, k, v, do, dq, dk, dv), st) == 0
    assert _lib.device_status() == 0
    ref = naive_attention(q.cpu(), k.cpu(), v.cpu(), do.cpu())
    check_against(ref, {"o": o, "dq": dq, "dk": dk, "dv": dv}, torch.float16)
    assert not torch.isnan(dqkv).any()  # every element of the packed gradient was written


def test_unsupported_head_dim_raises():
    q = torch.randn(1, 1, 64, 264, device=DEV, dtype=torch.float16)
    with pytest.raises(ValueError, match="head dimension"):
        flash_attention_v2(q, q, q)


@pytest.mark.parametrize(
    "shape,dtype",
    [
        ((2, 2, 1000, 256), torch.bfloat16),  # the reference's max_headdim
        ((1, 3, 300, 160), torch.float16),
        ((1, 2, 129, 192), torch.bfloat16),
        ((1, 2, 640, 136), torch.float16),
    ],
    ids=lambda v: "x".join(map(str, v)) if isinstance(v, tuple) else str(v)[6:],
)
def test_forward_backward_with_head_dims_up_to_256(shape, dtype):
    """Head dims in (128, 256] run the forward on the 128-wide plan with one Q tile per CTA and
    the head dim split in two halves (zero-padded to 256 by TMA like every other in-between
    size); O and LSE against the fp64 definition."""
    q, k, v, _ = make_inputs(shape, dtype)
    ref = naive_attention(q, k, v)
    with torch.no_grad():
        out = flash_attention_v2(q.to(DEV), k.to(DEV), v.to(DEV))
    assert _lib.device_status() == 0
    check_against(ref, {"o": out}, dtype, keys=("o",))
    # LSE through the C ABI
    b, h, n, d = shape
    lib = _lib.lib()
    qd, kd, vd = (t.to(DEV) for t in (q, k, v))
    o = torch.empty_like(qd)
    lse = torch.empty(b, h, n, device=DEV, dtype=torch.float32)
    assert lib.fa2_fwd(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), o.data_ptr(), lse.data_ptr(),
                       b, h, n, d, 0 if dtype == torch.float16 else 1, 1.0 / math.sqrt(d),
                       torch.cuda.current_stream().cuda_stream) == 0
    assert _lib.device_status() == 0
    assert torch.equal(o, out)
    assert (lse.cpu().double() - ref["lse"]).abs().max() <= 2e-3
    # backward: scores kernel + dV, dK, dQ consumer kernels; deterministic
    _, _, _, do = make_inputs(shape, dtype)
    ref = naive_attention(q, k, v, do)
    got = run_api(q, k, v, do, None, False)
    check_against(ref, got, dtype)
    again = run_api(q, k, v, do, None, True)
    for key in got:
        assert torch.equal(got[key], again[key]), key


@pytest.mark.parametrize("mode", ["spill", "recompute", "atomic"])
@pytest.mark.parametrize(
    "nq,nk,d,dtype",
    [
        (300, 100, 64, torch.float16),    # keys end inside the first tile: every later row sees all
        (1000, 257, 128, torch.bfloat16),  # ragged last KV tile seen by many Q tiles
        (640, 384, 32, torch.float16),    # tile-aligned key count
        (200, 520, 64, torch.bfloat16),   # more keys than queries: the tail gets zero gradients
        (129, 1, 64, torch.float16),      # a single key
        (700, 300, 256, torch.bfloat16),  # head dim above 128: scores + consumer kernels
    ],
)
def test_seqlen_q_differs_from_seqlen_k(nq, nk, d, dtype, mode, monkeypatch):
    """Top-left aligned causal mask as in the reference (_triton_kernels_v2.py:139-147):
    query row i sees keys 0 .. min(i, seqlen_k - 1)."""
    monkeypatch.setenv("FA2_B200_BWD_MODE", mode)
    det = mode != "atomic"
    g = torch.Generator().manual_seed(nq + nk)
    q, do = (torch.randn(2, 2, nq, d, generator=g).to(dtype) for _ in range(2))
    k, v = (torch.randn(2, 2, nk, d, generator=g).to(dtype) for _ in range(2))
    ref = naive_attention(q, k, v, do)
    got = run_api(q, k, v, do, None, det)
    check_against(ref, got, dtype)


# --------------------------------------------------------------------------- golden vectors
@pytest.mark.parametrize("path", sorted(GOLDEN_DIR.glob("*.npz")), ids=lambda p: p.stem)
def test_matches_reference_kernel_outputs(path):
    """Same fp16 inputs as the reference's kernels saw: our error against the fp64 oracle is no
    worse than the reference's own outputs' (maximum within 1.5x + 1e-3, rms within 25 %)."""
    z = np.load(path)
    q, k, v, do = (torch.from_numpy(z[x]) for x in ("q", "k", "v", "dout"))
    scale = float(z["softmax_scale"])
    det = not bool(z["sequence_parallel"])
    got = run_api(q, k, v, do, scale, det)
    ref = naive_attention(q, k, v, do, scale)
    for key in ("o", "dq", "dk", "dv"):
        ours = got[key].cpu().double()
        theirs = torch.from_numpy(z[key].astype(np.float64))
        e_ours, rms_ours = error_stats(ours, ref[key])
        e_ref, rms_ref = error_stats(theirs, ref[key])
        assert e_ours <= 1.5 * e_ref + 1e-3, f"{key}: ours {e_ours:.3e} vs reference {e_ref:.3e}"
        assert rms_ours <= 1.25 * rms_ref + 1e-5, f"{key}: rms ours {rms_ours:.3e} vs reference {rms_ref:.3e}"


# --------------------------------------------------------------------------- determinism
def test_deterministic_mode_is_bit_identical_across_runs():
    """Mirrors tests/test_flash_attention_2.py:322-342 (ragged, peaked-softmax inputs)."""
    q, k, v, do = make_inputs((2, 3, 1535, 32), torch.float16, qk_mul=3.0)
    first = run_api(q, k, v, do, 0.5, True)
    for _ in range(5):
        again = run_api(q, k, v, do, 0.5, True)
        for key in first:
            assert torch.equal(first[key], again[key]), key


def test_deterministic_mode_is_bit_identical_across_partitionings():
    """Splitting the (batch, head) axis 1/2/4/8 ways (as the multi-GPU run does) changes no bit."""
    q, k, v, do = make_inputs((2, 4, 640, 128), torch.bfloat16)
    full = run_api(q, k, v, do, None, True)
    for world in (2, 4, 8):
        parts = {key: [] for key in full}
        for rank in range(world):
            sl = [shard_slab(t, world, rank) for t in (q, k, v, do)]
            r = run_api(*sl, None, True)
            for key in full:
                parts[key].append(r[key])
        for key in full:
            assert torch.equal(torch.cat(parts[key], dim=1).view_as(full[key]), full[key]), (key, world)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_deterministic_mode_is_bit_identical_across_gpus():
    """Each GPU of the node computes its slab of (batch, head) problems; gathered, the results
    equal the single-GPU results bit for bit (no collective on the data path)."""
    world = min(torch.cuda.device_count(), 8)
    q, k, v, do = make_inputs((2, 8, 1100, 128), torch.bfloat16)
    full = run_api(q, k, v, do, None, True)
    parts = {key: [] for key in full}
    for rank in range(world):
        dev = torch.device("cuda", rank)
        sl = [shard_slab(t, world, rank) for t in (q, k, v, do)]
        with torch.cuda.device(dev):
            r = run_api(*sl, None, True, dev=dev)
        for key in full:
            parts[key].append(r[key].to(DEV))
    for key in full:
        assert torch.equal(torch.cat(parts[key], dim=1).view_as(full[key]), full[key]), key


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_data_parallel_matches_single_gpu():
    """The operator under nn.DataParallel (one host thread per GPU, batch split) against one GPU,
    like tests/test_flash_attention_2.py:415-480 of the reference, with the deterministic mode
    so that the comparison is exact instead of allclose."""

    class AttentionModel(torch.nn.Module):
        def forward(self, q, k, v):
            return flash_attention_v2(q, k, v, None, deterministic=True)

    ngpu = min(torch.cuda.device_count(), 4)
    q, k, v, do = (t.to(DEV) for t in make_inputs((2 * ngpu, 3, 700, 64), torch.float16))
    model = torch.nn.DataParallel(AttentionModel(), device_ids=list(range(ngpu))).to(DEV)
    qp, kp, vp = (t.clone().requires_grad_(True) for t in (q, k, v))
    out_p = model(qp, kp, vp)
    out_p.backward(do)
    single = run_api(q, k, v, do, None, True)
    for dev in range(ngpu):
        with torch.cuda.device(dev):
            assert _lib.device_status() == 0
    assert torch.equal(out_p, single["o"])
    for key, t in (("dq", qp), ("dk", kp), ("dv", vp)):
        assert torch.equal(t.grad, single[key]), key


def test_atomic_mode_matches_deterministic_mode_closely():
    """dK, dV and O do not depend on the dQ strategy (bit-equal); dQ differs only by fp32
    summation order before the single rounding."""
    q, k, v, do = make_inputs((1, 4, 1024, 64), torch.float16)
    a = run_api(q, k, v, do, None, True)
    b = run_api(q, k, v, do, None, False)
    for key in ("o", "dk", "dv"):
        assert torch.equal(a[key], b[key]), key
    assert (a["dq"].float() - b["dq"].float()).abs().max() <= 2e-3


def test_custom_entry_point_equals_default():
    """Mirrors tests/test_flash_attention_2.py:389-411: custom config == default deterministic."""

    class Cfg:
        kwargs = {"BLOCK_Q_ROWS_SIZE": 64, "BLOCK_KV_COLS_SIZE": 64, "SEQUENCE_PARALLEL": False}

    cfg = KernelsConfigV2(128, 128, 32, 256, 32, 8, 16, 1, [Cfg()])
    q, k, v, do = make_inputs((1, 2, 512, 64), torch.float16)
    a = run_api(q, k, v, do, None, True)
    qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    out = flash_attention_v2_custom(qd, kd, vd, None, {torch.cuda.get_device_capability(): cfg})
    out.backward(do.to(DEV))
    assert torch.equal(out, a["o"]) and torch.equal(qd.grad, a["dq"])
    assert torch.equal(kd.grad, a["dk"]) and torch.equal(vd.grad, a["dv"])
    with pytest.raises(ValueError, match="Missing kernel configuration"):
        flash_attention_v2_custom(qd, kd, vd, None, {(7, 5): cfg})


# --------------------------------------------------------------------------- properties at full size
def test_full_size_properties_c3_shape():
    """bf16 [2,32,8192,128] is too large for the fp64 oracle; check it through properties:
    (1) sampled (batch, head) problems against the per-head fp32 oracle,
    (2) linearity of the backward in dO: grads(2*dO) == 2*grads(dO) exactly in the
        deterministic mode (a power-of-two scale commutes with every rounding),
    (3) rows are convex combinations of V: |O| <= max |V| (1% slack: P is rounded to 16 bits
        after the row sum is taken in fp32)."""
    shape = (2, 32, 8192, 128)
    q, k, v, do = make_inputs(shape, torch.bfloat16)
    got = run_api(q, k, v, do, None, True)
    for (bi, hi) in ((0, 0), (1, 31)):
        sl = lambda t: t[bi:bi + 1, hi:hi + 1]
        ref = naive_attention_per_head(sl(q), sl(k), sl(v), sl(do), None, torch.float32)
        check_against(ref, {key: sl(val) for key, val in got.items()}, torch.bfloat16)
    twice = run_api(q, k, v, do * 2, None, True)
    for key in ("dq", "dk", "dv"):
        assert torch.equal(twice[key], got[key] * 2), key
    assert got["o"].abs().max().item() <= 1.01 * v.abs().max().item()
    atomic = run_api(q, k, v, do, None, False)
    assert torch.equal(atomic["dk"], got["dk"]) and torch.equal(atomic["dv"], got["dv"])
    assert (atomic["dq"].float() - got["dq"].float()).abs().max() <= 2e-2


def test_long_sequence_c4_slab():
    """One GPU's share of the 8-GPU long-context configuration: bf16 [1,2,32768,128] (2 of the 16
    heads), atomic dQ as that configuration asks.  256 tiles per head; checked through
    (1) rows of the last tile and of the first tile of one head against the fp64 definition
        (a row only needs its own q and the k, v before it, so single rows are cheap),
    (2) |O| <= max |V|, no NaN anywhere,
    (3) dK, dV bit-equal between the atomic and the deterministic mode, dQ close."""
    n, d = 32768, 128
    q, k, v, do = make_inputs((1, 2, n, d), torch.bfloat16)
    got = run_api(q, k, v, do, None, False)
    for key in got:
        assert not torch.isnan(got[key]).any(), key
    assert got["o"].abs().max().item() <= 1.01 * v.abs().max().item()
    scale = 1.0 / math.sqrt(d)
    for row in (0, 127, 128, 20000, n - 129, n - 1):
        qr = q[0, 1, row].double()
        s = (k[0, 1, : row + 1].double() @ qr) * scale
        p = torch.softmax(s, dim=0)
        want = p @ v[0, 1, : row + 1].double()
        err = (got["o"][0, 1, row].cpu().double() - want).abs().max().item()
        assert err <= 2e-2, (row, err)
    det = run_api(q, k, v, do, None, True)
    assert torch.equal(det["o"], got["o"])
    assert torch.equal(det["dk"], got["dk"]) and torch.equal(det["dv"], got["dv"])
    assert (det["dq"].float() - got["dq"].float()).abs().max() <= 2e-2
    # dV of the last key row: only the last query sees it, with probability p_last
    p_last = torch.softmax((k[0, 1].double() @ q[0, 1, n - 1].double()) * scale, dim=0)[n - 1]
    want_dv = p_last * do[0, 1, n - 1].double()
    assert (got["dv"][0, 1, n - 1].cpu().double() - want_dv).abs().max() <= 2e-2


def test_ragged_peaked_c5_shape_is_repeatable():
    """fp16 [8,12,4095,32], q,k ~ N(0,3), scale 0.5, deterministic: bit-exact repeat, no NaN,
    and one sampled head against the oracle.  Gradients reach |x| ~ 30 here, where one fp16
    ulp is 1.6e-2 and 32 tiles of fp16-rounded dS accumulate, so the 5e-3 bound cannot hold
    for any fp16 kernel; the binding criterion is "never worse than the reference": our error
    must stay at the level of the reference's own arithmetic (the tiled restatement
    that is pinned to the reference kernels) on the same head: equal rms error (within 25 %)
    and a maximum within 2x (the maximum over 131k elements is a tail value quantised in ulps)."""
    from oracle.attention_oracle import reference_tiled

    shape = (8, 12, 4095, 32)
    q, k, v, do = make_inputs(shape, torch.float16, qk_mul=3.0)
    a = run_api(q, k, v, do, 0.5, True)
    b = run_api(q, k, v, do, 0.5, True)
    for key in a:
        assert torch.equal(a[key], b[key]), key
        assert not torch.isnan(a[key]).any()
    sl = lambda t: t[7:8, 11:12]
    ref = naive_attention_per_head(sl(q), sl(k), sl(v), sl(do), 0.5, torch.float64)
    theirs = reference_tiled(sl(q).numpy(), sl(k).numpy(), sl(v).numpy(), sl(do).numpy(), 0.5, 128, 128, 128)
    for key in ("o", "dq", "dk", "dv"):
        d_ours = sl(a[key]).cpu().double() - ref[key]
        d_ref = torch.from_numpy(theirs[key].astype(np.float64)) - ref[key]
        e_ours, e_ref = d_ours.abs().max().item(), d_ref.abs().max().item()
        rms_ours, rms_ref = d_ours.pow(2).mean().sqrt().item(), d_ref.pow(2).mean().sqrt().item()
        print(f"{key}: max-abs ours {e_ours:.3e} ref {e_ref:.3e}; rms ours {rms_ours:.3e} ref {rms_ref:.3e}")
        # the error level (rms) must match the reference arithmetic's; the maximum over 131k
        # elements is a tail value quantised in fp16 ulps, so it gets a factor of two
        assert rms_ours <= 1.25 * rms_ref + 1e-5, f"{key}: rms ours {rms_ours:.3e}, reference {rms_ref:.3e}"
        assert e_ours <= max(5e-3, 2.0 * e_ref), f"{key}: ours {e_ours:.3e}, reference {e_ref:.3e}"
