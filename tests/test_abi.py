"""The C-ABI shared library: loads without a GPU, exports every symbol the header declares,
and rejects bad arguments with the documented codes before touching the device."""

from __future__ import annotations

import ctypes
import re

import pytest

from conftest import ROOT
from flash_attention_triton_b200 import _lib

HEADER = ROOT / "include" / "fa2_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(fa2_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_hot_path_entry_points():
    names = declared_functions()
    for need in ("fa2_fwd", "fa2_bwd_preprocess", "fa2_bwd", "fa2_bwd_workspace_bytes",
                 "fa2_rowstats_bytes", "fa2_strerror", "fa2_abi_version", "fa2_device_status"):
        assert need in names


def test_library_exports_every_declared_symbol():
    handle = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"


def test_binding_table_covers_header():
    assert sorted(n for n, _, _ in _lib.SYMBOLS) == declared_functions()


def test_abi_version_and_error_text():
    lib = _lib.lib()
    assert lib.fa2_abi_version() == 3
    assert lib.fa2_strerror(0) == b"success"
    assert b"multiple of 8" in lib.fa2_strerror(-2)
    assert lib.fa2_strerror(-12345) == b"unknown fa2 error code"


def test_size_queries():
    lib = _lib.lib()
    # rowstats: [B*H][ceil(N/128)][2][128] fp32, then one word per tile (its largest |dout|)
    assert lib.fa2_rowstats_bytes(2, 3, 4095) == 2 * 3 * 32 * (256 + 1) * 4
    assert lib.fa2_rowstats_bytes(0, 3, 128) == 0
    # dq workspace: fp32 [B*H][ceil(N/128)*128][D], none in deterministic mode
    assert lib.fa2_bwd_workspace_bytes(2, 3, 4095, 32, 0) == 2 * 3 * 4096 * 32 * 4
    assert lib.fa2_bwd_workspace_bytes(2, 3, 4095, 32, 1) == 0
    # head dims between the instantiated sizes accumulate in the next size up
    assert lib.fa2_bwd_workspace_bytes(1, 1, 128, 48, 0) == 128 * 64 * 4
    assert lib.fa2_bwd_workspace_bytes(1, 1, 128, 96, 0) == 128 * 128 * 4


@pytest.mark.parametrize(
    "kwargs, code",
    [
        (dict(q=0), -1),                      # NULL pointer
        (dict(D=44), -2),                     # head dim not a multiple of 8
        (dict(D=264), -2),                    # head dim above 256
        (dict(dtype=7), -3),                  # unsupported dtype
        (dict(q=0x1008), -4),                 # misaligned pointer
        (dict(N=0), -5),                      # empty sequence
        (dict(B=70000), -5),                  # B*H > 65535
        (dict(scale=float("nan")), -9),
        (dict(scale=-1.0), -9),
    ],
)
def test_forward_argument_errors_need_no_gpu(kwargs, code):
    a = dict(q=0x1000, k=0x2000, v=0x3000, o=0x4000, lse=0x5000, B=1, H=1, N=128, D=64, dtype=0,
             scale=0.125)
    a.update(kwargs)
    rc = _lib.lib().fa2_fwd(a["q"], a["k"], a["v"], a["o"], a["lse"], a["B"], a["H"], a["N"],
                            a["D"], a["dtype"], a["scale"], None)
    assert rc == code


def test_backward_argument_errors_need_no_gpu():
    lib = _lib.lib()
    p = [0x1000 * (i + 1) for i in range(8)]
    # non-deterministic mode without a workspace
    rc = lib.fa2_bwd(*p[:5], p[5], p[6], p[7], None, 0, 1, 1, 128, 64, 0, 0.125, 0, None)
    assert rc == -10
    # a workspace below the mode's minimum is refused before anything is launched: the atomic
    # accumulator of [1, 1, 128, 64] is 32 KiB, one head's tile of the spill mode 32 KiB
    rc = lib.fa2_bwd(*p[:5], p[5], p[6], p[7], 0x10000, 1024, 1, 1, 128, 64, 0, 0.125, 0, None)
    assert rc == -10
    rc = lib.fa2_bwd(*p[:5], p[5], p[6], p[7], 0x10000, 32767, 1, 1, 128, 64, 0, 0.125, 2, None)
    assert rc == -10
    rc = lib.fa2_bwd(*p[:5], p[5], p[6], p[7], 0x10000, 100, 1, 1, 128, 256, 0, 0.125, 1, None)
    assert rc == -10
    rc = lib.fa2_bwd(*p[:5], p[5], p[6], p[7], 0x10010, 1 << 20, 1, 1, 128, 64, 0, 0.125, 2, None)
    assert rc == -4  # workspace not 256-byte aligned
    rc = lib.fa2_bwd(*p[:5], p[5], p[6], None, None, 0, 1, 1, 128, 64, 0, 0.125, 1, None)
    assert rc == -1
    rc = lib.fa2_bwd_preprocess(p[0], p[1], p[2], None, 1, 1, 128, 64, 0, None)
    assert rc == -1
    rc = lib.fa2_bwd_preprocess(p[0], p[1], p[2], p[3], 1, 1, 128, 264, 0, None)
    assert rc == -2


def test_check_raises_with_text():
    with pytest.raises(_lib.Fa2Error, match="head dimension"):
        _lib.check("fa2_fwd", -2)


@pytest.mark.parametrize(
    "triple, code",
    [
        ((4, 64, 8192), -12),       # batch stride not a multiple of 8 elements
        ((1 << 20, -64, 8192), -12),  # negative head stride
        ((1 << 20, 64, 32), -12),   # row stride smaller than the head dim
        ((1 << 20, 64, 0), -12),    # a zero stride inside a non-zero triple
    ],
)
def test_stride_errors_need_no_gpu(triple, code):
    """fa2_fwd_strided checks the (batch, head, row) element strides before touching the device."""
    import ctypes

    strides = (ctypes.c_longlong * 12)(*(list(triple) + [0] * 9))  # q strided, k, v, o dense
    rc = _lib.lib().fa2_fwd_strided(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, 2, 4, 128, 128, 64, 0,
                                    0.125, strides, None)
    assert rc == code
    assert b"stride" in _lib.lib().fa2_strerror(code)


def test_stride_array_packs_batch_head_row_strides():
    import torch

    a = torch.empty(2, 5, 3, 16).transpose(1, 2)  # [B, H=3, N=5, D] view of [B, N, H, D] storage
    arr = _lib.stride_array(a, a.contiguous())
    assert list(arr) == [240, 16, 48, 240, 80, 16]


def test_key_count_must_not_exceed_query_count():
    """Keys beyond the last query row are never attended under the top-left aligned mask; the C
    entry points refuse them (the Python API slices them off and zeroes their gradients)."""
    lib = _lib.lib()
    assert lib.fa2_fwd_strided(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, 1, 1, 128, 129, 64, 0,
                               0.125, None, None) == -5
    assert lib.fa2_fwd_strided(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, 1, 1, 128, 0, 64, 0,
                               0.125, None, None) == -5


def test_spill_scratch_size_follows_the_budget():
    """32 KiB per (KV tile, Q tile) pair; chunks of whole heads of about 2048 tiles, so the
    recommendation is linear in N and independent of B*H; bounded by fa2_set_spill_budget."""
    lib = _lib.lib()
    pairs = 64 * 65 // 2  # N = 8192: 64 tiles
    previous = lib.fa2_set_spill_budget(1 << 40)
    try:
        # 2048 tiles = 32 heads of 64 tiles, whatever the number of heads beyond that
        assert lib.fa2_bwd_workspace_bytes(2, 32, 8192, 128, 2) == 32 * pairs * 32768
        assert lib.fa2_bwd_workspace_bytes(8, 32, 8192, 128, 2) == 32 * pairs * 32768
        assert lib.fa2_bwd_workspace_bytes(1, 8, 8192, 128, 2) == 8 * pairs * 32768  # all there is
        # four times the rows: a quarter of the heads, 4x the bytes (not 16x)
        pairs4 = 256 * 257 // 2
        assert lib.fa2_bwd_workspace_bytes(2, 32, 32768, 128, 2) == 8 * pairs4 * 32768
        lib.fa2_set_spill_budget(20 * pairs * 32768)      # 20 heads fit: two chunks of 16
        assert lib.fa2_bwd_workspace_bytes(2, 32, 8192, 128, 2) == 16 * pairs * 32768
        assert lib.fa2_bwd_workspace_bytes(2, 16, 8192, 256, 0) == 8 * 2 * pairs * 32768  # 64 KiB per pair: 10 heads fit, two chunks of 8
        lib.fa2_set_spill_budget(1)                       # never below one head
        assert lib.fa2_bwd_workspace_bytes(2, 32, 8192, 128, 2) == pairs * 32768
        assert lib.fa2_set_spill_budget(previous) == 1
    finally:
        lib.fa2_set_spill_budget(previous)
    assert lib.fa2_bwd_workspace_bytes(2, 32, 8192, 128, 1) == 0


def test_backward_mode_choice_depends_on_the_sequence_length_only(monkeypatch):
    from flash_attention_triton_b200 import api

    monkeypatch.delenv("FA2_B200_BWD_MODE", raising=False)
    assert api._backward_mode(True, 128, 8192) == api._MODE_SPILL
    assert api._backward_mode(True, 32, 4095) == api._MODE_RECOMPUTE     # no scratch at d <= 64: same speed
    assert api._backward_mode(True, 64, 8192) == api._MODE_RECOMPUTE
    assert api._backward_mode(True, 96, 8192) == api._MODE_SPILL
    assert api._backward_mode(True, 128, 32768) == api._MODE_SPILL       # 1 GiB of dS per head
    assert api._backward_mode(True, 128, 65536) == api._MODE_RECOMPUTE   # 4 GiB per head
    assert api._backward_mode(False, 128, 8192) == api._MODE_SPILL       # fastest at d = 128
    assert api._backward_mode(False, 128, 65536) == api._MODE_RECOMPUTE  # ahead of the atomic kernel there
    assert api._backward_mode(False, 64, 8192) == api._MODE_ATOMIC
    assert api._backward_mode(False, 256, 8192) == api._MODE_SPILL       # the one backward there
    monkeypatch.setenv("FA2_B200_BWD_MODE", "recompute")
    assert api._backward_mode(False, 64, 8192) == api._MODE_RECOMPUTE


def test_workspace_allocation_falls_back_when_memory_is_short(monkeypatch):
    """The recommended scratch, an eighth of it, one head's worth, then the scratch-free
    recompute backward."""
    import torch

    from flash_attention_triton_b200 import api

    lib = _lib.lib()
    head = 2080 * 32768
    want = lib.fa2_bwd_workspace_bytes(2, 32, 8192, 128, 2)
    assert want == 32 * head  # chunks of 2048 tiles
    calls, limit = [], [1 << 62]

    def fake_empty(nbytes, device=None, dtype=None):
        calls.append(nbytes)
        if nbytes > limit[0]:
            raise torch.cuda.OutOfMemoryError("no memory")
        return torch.zeros(1, dtype=torch.uint8)

    monkeypatch.setattr(api.torch, "empty", fake_empty)
    assert api._allocate_workspace(lib, "cpu", 2, 32, 8192, 128, api._MODE_SPILL)[1:] == (want, api._MODE_SPILL)
    limit[0] = 1 << 29  # 7 heads fit
    calls.clear()
    assert api._allocate_workspace(lib, "cpu", 2, 32, 8192, 128, api._MODE_SPILL)[1:] == (4 * head, api._MODE_SPILL)
    limit[0] = 100 << 20  # one head (68 MB) fits
    calls.clear()
    assert api._allocate_workspace(lib, "cpu", 2, 32, 8192, 128, api._MODE_SPILL)[1:] == (head, api._MODE_SPILL)
    assert calls == [want, 4 * head, head]
    # exactly what fa2_bwd accepts as the minimum: refused with one byte less
    assert lib.fa2_bwd(*([0x1000] * 8), 0x10000, head - 1, 1, 1, 8192, 128, 1, 0.1, 2, None) == -10
    limit[0] = 1 << 20
    assert api._allocate_workspace(lib, "cpu", 2, 32, 8192, 128, api._MODE_SPILL) == (None, 0, api._MODE_RECOMPUTE)
    with pytest.raises(torch.cuda.OutOfMemoryError):  # head dim 256 has no scratch-free backward
        api._allocate_workspace(lib, "cpu", 2, 16, 8192, 256, api._MODE_SPILL)
    assert api._allocate_workspace(lib, "cpu", 2, 32, 8192, 128, api._MODE_RECOMPUTE) == (None, 0, 1)


def test_static_scratch_refuses_bad_arguments_before_launching():
    """Everything fa2_bwd would refuse is refused before the preprocess kernel could overwrite the
    shared array: head dims above 128, a bad scale, misaligned pointers."""
    lib = _lib.lib()
    p = [0x1000] * 9
    assert lib.fa2_bwd_static_scratch(*p, 1, 2, 256, 256, 1, 0.1, None) == -10
    assert lib.fa2_bwd_static_scratch(*p, 1, 2, 256, 64, 1, 0.0, None) == -9
    assert lib.fa2_bwd_static_scratch(*p, 1, 2, 256, 64, 1, float("nan"), None) == -9
    assert lib.fa2_bwd_static_scratch(*([0x1000] * 6 + [0x1008] + [0x1000] * 2), 1, 2, 256, 64, 1, 0.1, None) == -4
    assert lib.fa2_bwd_static_scratch(*p, 1, 65, 8192, 128, 1, 0.1, None) == -11
