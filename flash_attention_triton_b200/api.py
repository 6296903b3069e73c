"""Drop-in Python surface of the reference's causal FlashAttention-2 operator.

Mirrors ``src/flash_attention_triton/flash_attention_2.py`` of flash-attention-triton:

* :func:`flash_attention_v2` (reference lines 646-697) — same name, arguments and defaults;
* :func:`flash_attention_v2_custom` (700-790) — same signature; the tile/warp knobs of the
  config are ignored (there is no Triton here), only its ``SEQUENCE_PARALLEL`` flag survives
  as the deterministic switch;
* :class:`FlashAttentionV2Function` (280-384) — ``apply(q, k, v, softmax_scale, deterministic)``
  returning five gradients ``(dq, dk, dv, None, None)``;
* :class:`KernelsConfigV2`, :func:`init_to_zero_v2` (``_configurators_v2.py:9-93``).

Differences, all deliberate: fp16 and bf16 inputs run natively (the reference casts
everything to fp16, lines 316/379); other float dtypes are cast to fp16 exactly as the
reference does.  Multiples of 8 run natively as head dimension (the kernels run them
zero-padded to 32 / 64 / 128 / 256 through TMA out-of-bounds fill; other sizes are
zero-padded to a multiple of 8 on the host first); head dimensions up to 256 are supported.
``seqlen_q != seqlen_k`` follows the reference's top-left aligned causal mask: query row i sees keys ``0 .. min(i, seqlen_k - 1)``;
keys beyond ``seqlen_q`` are seen by nobody and get zero gradients.
Everything runs through the C library on the tensors' CUDA device; there is no fallback.
"""

from __future__ import annotations

import math
import os
from collections.abc import Callable
from dataclasses import dataclass
from typing import Any

import torch

from . import _lib

_MAX_HEAD_DIM = 256  # the reference's max_headdim on B200 (line 533)


# ------------------------------------------------------------------ host launch wrappers
def _dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float16:
        return _lib.FA2_DTYPE_FP16
    if dtype == torch.bfloat16:
        return _lib.FA2_DTYPE_BF16
    raise AssertionError("Supports only fp16 and bf16 compute dtypes")


def _check_status_if_asked(fn: str) -> None:
    """Kernels that give up on a bounded wait leave their outputs unwritten and only set the
    device status word; reading it synchronises the device, so it is not read by default.
    ``FA2_B200_CHECK_STATUS=1`` makes every forward / backward call read it and raise
    ``Fa2Error`` (``FA2_ERR_DEVICE_STATUS``) when it is non-zero."""
    if os.environ.get("FA2_B200_CHECK_STATUS") == "1":
        word = _lib.device_status()
        if word:
            raise _lib.Fa2Error(fn, -7, f"{_lib.lib().fa2_strerror(-7).decode()} (status {word:#x})")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _readable_in_place(t: torch.Tensor) -> bool:
    """Whether the kernels can read a ``[B, H, N, D]`` tensor through its own strides: unit
    last stride, 16-byte aligned base, batch / head / row strides that are positive multiples
    of 8 elements (strides of size-1 dimensions do not matter)."""
    if t.stride(-1) != 1 or t.data_ptr() % 16:
        return False
    for size, stride in zip(t.shape[:3], t.stride()[:3]):
        if size > 1 and (stride <= 0 or stride % 8):
            return False
    return t.shape[2] == 1 or t.stride(2) >= t.shape[3]


def _as_kernel_input(t: torch.Tensor) -> torch.Tensor:
    """The tensor itself when it can be read in place (e.g. a transposed ``[B, N, H, D]``
    buffer), else a contiguous copy (what the reference always makes, line 316)."""
    return t if _readable_in_place(t) else t.contiguous()


def _flash_attention_forward(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float | None
) -> tuple[torch.Tensor, torch.Tensor, float]:
    """Validate, allocate O and LSE, launch ``fa2_fwd``.

    Counterpart of ``_flash_attention_forward`` (reference lines 61-144): the same asserts on
    shapes / device / dtype, ``softmax_scale or 1/sqrt(d)`` (so 0.0 means "default"), but
    LSE is an unpadded ``[B, H, N]`` fp32 tensor and no scratch buffer exists.
    """
    batch, nheads, seqlen_q, headdim = q.shape
    seqlen_k = k.shape[2]
    assert k.shape == (batch, nheads, seqlen_k, headdim)
    assert v.shape == (batch, nheads, seqlen_k, headdim)
    assert q.is_cuda and k.is_cuda and v.is_cuda, "All tensors must reside on CUDA device"
    assert q.dtype == k.dtype == v.dtype, "All tensors must be the same type"
    if headdim > _MAX_HEAD_DIM or headdim % 8:
        raise ValueError(f"head dimension {headdim} is not supported (multiples of 8 up to {_MAX_HEAD_DIM})")
    if seqlen_k > seqlen_q:  # no query sees the keys beyond seqlen_q - 1 (top-left aligned mask)
        k, v, seqlen_k = k[:, :, :seqlen_q], v[:, :, :seqlen_q], seqlen_q
    softmax_scale = softmax_scale or 1.0 / math.sqrt(headdim)
    q, k, v = [_as_kernel_input(t) for t in (q, k, v)]
    output = torch.empty(q.shape, device=q.device, dtype=q.dtype)  # dense, like the reference's O
    lse = torch.empty((batch, nheads, seqlen_q), device=q.device, dtype=torch.float32)
    with torch.cuda.device(q.device):
        _lib.check(
            "fa2_fwd_strided",
            _lib.lib().fa2_fwd_strided(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), output.data_ptr(), lse.data_ptr(),
                batch, nheads, seqlen_q, seqlen_k, headdim, _dtype_code(q.dtype),
                float(softmax_scale), _lib.stride_array(q, k, v, output), _stream(q),
            ),
        )
        _check_status_if_asked("fa2_fwd_strided")
    return output, lse, softmax_scale


#: dQ strategies of the C library (the ``deterministic`` argument of ``fa2_bwd``)
_MODE_ATOMIC, _MODE_RECOMPUTE, _MODE_SPILL = 0, 1, 2
_MODE_NAMES = {"atomic": _MODE_ATOMIC, "recompute": _MODE_RECOMPUTE, "spill": _MODE_SPILL}
#: the spill mode keeps 32 KiB per tile pair of a head in scratch; when one head's tiles exceed
#: this much (N above ~45 k) the recompute mode, which needs no scratch, takes over
_SCRATCH_MAX_BYTES_PER_HEAD = 2 << 30


def _scratch_bytes_per_head(seqlen_q: int, headdim: int) -> int:
    tiles = (seqlen_q + 127) // 128
    return tiles * (tiles + 1) // 2 * 32768 * (2 if headdim > 128 else 1)


def _backward_mode(deterministic: bool, headdim: int, seqlen_q: int) -> int:
    """Which dQ strategy serves ``deterministic``.

    ``True`` must give the same bits whatever the batch / head partitioning, so the choice
    depends on the head dim and the sequence length only.  Head dims above 64: the spill mode
    (fastest there, 12-15 % ahead of the recompute mode) unless one head's scratch is too
    large, then the recompute mode.  Head dims up to 64: the recompute mode, which measures
    within 4 % of the spill mode either way there (the 32 KiB dS tile does not shrink with the
    head dim, the tensor work does) and needs no scratch, like the reference's O(N) backward.
    ``False`` (the reference's default, atomics there) means "fastest": the atomic kernel at
    head dims up to 64 (15-25 % ahead), the deterministic choice above.  ``FA2_B200_BWD_MODE`` =
    ``atomic`` / ``recompute`` / ``spill`` overrides both (for experiments).
    """
    if headdim > 128:  # one (deterministic) backward exists there: scores + three consumers
        return _MODE_SPILL
    forced = os.environ.get("FA2_B200_BWD_MODE")
    if forced:
        return _MODE_NAMES[forced]
    if headdim <= 64:
        return _MODE_RECOMPUTE if deterministic else _MODE_ATOMIC
    scratch_ok = _scratch_bytes_per_head(seqlen_q, headdim) <= _SCRATCH_MAX_BYTES_PER_HEAD
    return _MODE_SPILL if scratch_ok else _MODE_RECOMPUTE


def _allocate_workspace(lib, device, batch, nheads, seqlen_q, headdim, mode):
    """The workspace of a backward mode, and the mode that will run.

    The scratch of the spill mode is a convenience, not a need (the reference's backward is
    O(N) in memory, ``flash_attention_2.py:195-196``): when the recommended size cannot be had,
    an eighth of it is tried (more chunks, a few per cent slower), then one head's worth, and
    when even that fails the recompute backward, which needs no scratch and gives the same dK,
    dV and a dQ that differs in the last bit at most, runs instead.  Head dims above 128 have no
    scratch-free backward: there the out-of-memory error propagates.
    """
    want = lib.fa2_bwd_workspace_bytes(batch, nheads, seqlen_q, headdim, mode)
    if not want:
        return None, 0, mode
    sizes = [want]
    if mode == _MODE_SPILL:
        one_head = _scratch_bytes_per_head(seqlen_q, headdim)
        sizes += [n for n in (want // 8 // one_head * one_head, one_head) if one_head <= n < sizes[-1]]
    for nbytes in sizes:
        try:
            return torch.empty(nbytes, device=device, dtype=torch.uint8), nbytes, mode
        except torch.cuda.OutOfMemoryError:
            continue
    if mode == _MODE_SPILL and headdim <= 128:
        return None, 0, _MODE_RECOMPUTE
    raise torch.cuda.OutOfMemoryError(
        f"no memory for the backward workspace ({sizes[-1]} bytes at least)")


def _flash_attention_backward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    output: torch.Tensor,
    lse: torch.Tensor,
    dq: torch.Tensor,
    dk: torch.Tensor,
    dv: torch.Tensor,
    d_output: torch.Tensor,
    softmax_scale: float,
    deterministic: bool,
) -> None:
    """Launch ``fa2_bwd_preprocess`` and ``fa2_bwd``.

    Counterpart of ``_flash_attention_backward`` (reference lines 147-277).  The workspace
    depends on the dQ strategy (:func:`_backward_mode`): an fp32 accumulator for the atomic
    kernel, the dS scratch for the spill mode, nothing for the recompute mode; the
    deterministic modes write dQ once, already rounded.
    """
    batch, nheads, seqlen_q, headdim = q.shape
    seqlen_k = k.shape[2]
    if seqlen_k > seqlen_q:  # keys nobody sees: zero gradients, and the kernels skip them
        dk[:, :, seqlen_q:].zero_()
        dv[:, :, seqlen_q:].zero_()
        k, v, dk, dv = (t[:, :, :seqlen_q] for t in (k, v, dk, dv))
        seqlen_k = seqlen_q
    # The reference requires everything contiguous here (lines 183-192) and copies dO when it
    # is not (170-171); the inputs may keep their strides, only our own buffers are dense.
    q, k, v, d_output = [_as_kernel_input(t) for t in (q, k, v, d_output)]
    assert lse.shape == (batch, nheads, seqlen_q)
    assert output.is_contiguous() and dq.is_contiguous()
    assert _readable_in_place(dk) and _readable_in_place(dv)
    lib = _lib.lib()
    code = _dtype_code(q.dtype)
    with torch.cuda.device(q.device):
        stats_bytes = lib.fa2_rowstats_bytes(batch, nheads, seqlen_q)
        rowstats = torch.empty(stats_bytes // 4, device=q.device, dtype=torch.float32)
        _lib.check(
            "fa2_bwd_preprocess_strided",
            lib.fa2_bwd_preprocess_strided(
                output.data_ptr(), d_output.data_ptr(), lse.data_ptr(), rowstats.data_ptr(),
                batch, nheads, seqlen_q, headdim, code, _lib.stride_array(output, d_output),
                _stream(q),
            ),
        )
        mode = _backward_mode(bool(deterministic), headdim, seqlen_q)
        workspace, ws_bytes, mode = _allocate_workspace(
            lib, q.device, batch, nheads, seqlen_q, headdim, mode)
        _lib.check(
            "fa2_bwd_strided",
            lib.fa2_bwd_strided(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), d_output.data_ptr(), rowstats.data_ptr(),
                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                workspace.data_ptr() if workspace is not None else None, ws_bytes,
                batch, nheads, seqlen_q, seqlen_k, headdim, code, float(softmax_scale),
                mode, _lib.stride_array(q, k, v, d_output, dq, dk, dv), _stream(q),
            ),
        )
        _check_status_if_asked("fa2_bwd_strided")


# ------------------------------------------------------------------ autograd integration
def _compute_dtype(dtype: torch.dtype) -> torch.dtype:
    # fp16 / bf16 run natively; everything else takes the reference's route (cast to fp16,
    # reference line 316).
    return dtype if dtype in (torch.float16, torch.bfloat16) else torch.float16


class FlashAttentionV2Function(torch.autograd.Function):
    """Autograd function for causal FlashAttention-2 (reference lines 280-384)."""

    @staticmethod
    def forward(ctx: Any, q, k, v, softmax_scale, deterministic):  # noqa: ANN001
        initial_dtype = q.dtype
        cdtype = _compute_dtype(q.dtype)
        headdim = q.shape[-1]
        if headdim > _MAX_HEAD_DIM:
            raise ValueError(f"head dimension {headdim} is not supported (at most {_MAX_HEAD_DIM})")
        softmax_scale = softmax_scale or 1.0 / math.sqrt(headdim)  # reference line 94: 0.0 -> default
        q, k, v = [_as_kernel_input(t.to(cdtype)) for t in (q, k, v)]
        pad = -headdim % 8  # zero columns change neither the scores nor the real output columns
        if pad:
            q, k, v = [torch.nn.functional.pad(t, (0, pad)) for t in (q, k, v)]
        output, lse, ctx.softmax_scale = _flash_attention_forward(q, k, v, softmax_scale)
        ctx.save_for_backward(q, k, v, output, lse)
        ctx.deterministic = bool(deterministic)
        ctx.headdim = headdim
        return output[..., :headdim].contiguous().to(initial_dtype)

    @staticmethod
    def backward(ctx: Any, d_output):  # noqa: ANN001
        q, k, v, output, lse = ctx.saved_tensors
        dq, dk, dv = (torch.empty(t.shape, device=t.device, dtype=t.dtype) for t in (q, k, v))
        d_output = d_output.to(q.dtype)
        pad = q.shape[-1] - ctx.headdim
        if pad:
            d_output = torch.nn.functional.pad(d_output, (0, pad))
        _flash_attention_backward(
            q, k, v, output, lse, dq, dk, dv, d_output, ctx.softmax_scale, ctx.deterministic,
        )
        if pad:
            dq, dk, dv = [t[..., : ctx.headdim].contiguous() for t in (dq, dk, dv)]
        return dq, dk, dv, None, None


# ------------------------------------------------------------------ configuration shim
@dataclass(frozen=True)
class KernelsConfigV2:
    """Name-compatible stand-in for the reference's kernel configuration container.

    Same fields as ``_configurators_v2.py:9-38``.  Tile sizes, warp counts and stages have
    no meaning for the hand-written sm_100a kernels and are ignored; the only information
    used is whether the first backward config asks for ``SEQUENCE_PARALLEL`` (atomic dQ,
    non-deterministic) or not (deterministic), as in the reference's tables (lines 570-589).
    """

    block_rows_size: int
    block_cols_size: int
    min_block_headdim: int
    max_headdim: int
    seqlen_cache_divisor: int
    min_warps: int
    max_warps: int
    num_stages: int
    backward_autotune_configs: list

    def is_deterministic(self) -> bool:
        if not self.backward_autotune_configs:
            return True
        first = self.backward_autotune_configs[0]
        kwargs = getattr(first, "kwargs", first if isinstance(first, dict) else {})
        return not bool(kwargs.get("SEQUENCE_PARALLEL", False))


def init_to_zero_v2(name: str) -> Callable[[dict[str, torch.Tensor]], torch.Tensor]:
    """Pre-hook factory kept for source compatibility (``_configurators_v2.py:81-93``)."""
    return lambda nargs: nargs[name].zero_()


# ------------------------------------------------------------------ public API
def _check_device(q: torch.Tensor) -> None:
    assert q.is_cuda, "All tensors must reside on CUDA device"
    cc = torch.cuda.get_device_capability(q.device)
    if cc[0] != 10:
        raise RuntimeError(
            f"compute capability {cc} is not supported: this library targets B200 (sm_100a) only"
        )


def flash_attention_v2(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    softmax_scale: float | None = None,
    deterministic: bool = False,
) -> torch.Tensor:
    """Causal FlashAttention-2 on B200; same contract as the reference (lines 646-697).

    Args:
        q, k, v: ``(batch, nheads, seqlen, headdim)`` CUDA tensors of one float dtype.
        softmax_scale: scaling factor (default and 0.0: ``1/sqrt(headdim)``).
        deterministic: use the backward whose dQ has a fixed summation order (bit-identical
            across runs and across batch x head partitionings) instead of fp32 atomics.

    Returns:
        Attention output, same shape and dtype as ``q``.
    """
    _check_device(q)
    return FlashAttentionV2Function.apply(q, k, v, softmax_scale, deterministic)


def flash_attention_v2_custom(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    softmax_scale: float | None,
    kernels_configs: dict[tuple[int, int], KernelsConfigV2],
) -> torch.Tensor:
    """Same signature as the reference (lines 700-790): config looked up by compute capability.

    Raises ``ValueError`` when the current device's capability has no entry, as the
    reference does (lines 775-779).
    """
    _check_device(q)
    cc = torch.cuda.get_device_capability(q.device)
    if cc not in kernels_configs:
        raise ValueError(
            f"Missing kernel configuration for compute capability {cc}. "
            "KernelsConfig must be provided for the current GPU architecture"
        )
    deterministic = kernels_configs[cc].is_deterministic()
    return FlashAttentionV2Function.apply(q, k, v, softmax_scale, deterministic)
