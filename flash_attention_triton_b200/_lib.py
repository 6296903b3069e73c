"""ctypes binding of ``libfa2_b200.so`` (the C ABI declared in ``include/fa2_b200.h``).

The library is the only execution path of this package: if the shared object is missing or
cannot be loaded, :func:`lib` raises; nothing falls back to PyTorch or to the CPU.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libfa2_b200.so"

FA2_DTYPE_FP16 = 0
FA2_DTYPE_BF16 = 1

#: every symbol ``include/fa2_b200.h`` declares: (name, restype, argtypes)
SYMBOLS = [
    ("fa2_abi_version", c_int, []),
    ("fa2_strerror", c_char_p, [c_int]),
    ("fa2_fwd", c_int, [c_void_p] * 5 + [c_int] * 5 + [c_float, c_void_p]),
    ("fa2_bwd_preprocess", c_int, [c_void_p] * 4 + [c_int] * 5 + [c_void_p]),
    ("fa2_rowstats_bytes", c_size_t, [c_int] * 3),
    ("fa2_bwd", c_int, [c_void_p] * 9 + [c_size_t] + [c_int] * 5 + [c_float, c_int, c_void_p]),
    ("fa2_bwd_workspace_bytes", c_size_t, [c_int] * 5),
    ("fa2_set_spill_budget", c_size_t, [c_size_t]),
    ("fa2_bwd_mark_between", c_int, [c_void_p]),
    ("fa2_device_status", c_int, [ctypes.POINTER(c_int)]),
    ("fa2_selftest_mma", c_int, [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]),
    ("fa2_selftest_wait_timeout", c_int, [c_void_p]),
    ("fa2_bwd_static_scratch", c_int, [c_void_p] * 9 + [c_int] * 5 + [c_float, c_void_p]),
    ("fa2_fwd_strided", c_int, [c_void_p] * 5 + [c_int] * 6 + [c_float, c_void_p, c_void_p]),
    ("fa2_bwd_preprocess_strided", c_int, [c_void_p] * 4 + [c_int] * 5 + [c_void_p, c_void_p]),
    ("fa2_bwd_strided", c_int,
     [c_void_p] * 9 + [c_size_t] + [c_int] * 6 + [c_float, c_int, c_void_p, c_void_p]),
]


def stride_array(*tensors):
    """ctypes array of (batch, head, row) element strides, one triple per ``[B, H, N, D]`` tensor."""
    flat = [st for t in tensors for st in t.stride()[:3]]
    return (ctypes.c_longlong * len(flat))(*flat)

_lib = None


class Fa2Error(RuntimeError):
    """A non-zero return code of the C library."""

    def __init__(self, fn: str, code: int, text: str):
        super().__init__(f"{fn} failed with code {code}: {text}")
        self.code = code


def lib() -> ctypes.CDLL:
    """Load (once) and return the shared library with typed signatures."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing. Build it with `python -m flash_attention_triton_b200.build` "
            "(needs nvcc with sm_100a support). There is no fallback path."
        )
    handle = ctypes.CDLL(str(LIB_PATH))
    for name, restype, argtypes in SYMBOLS:
        fn = getattr(handle, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = handle
    return _lib


def check(fn: str, code: int) -> None:
    """Raise :class:`Fa2Error` (ValueError-like for argument errors) on a non-zero code."""
    if code != 0:
        text = lib().fa2_strerror(code).decode()
        raise Fa2Error(fn, code, text)


def device_status() -> int:
    """Synchronise the current device and return (and clear) its kernel status word."""
    out = c_int(0)
    check("fa2_device_status", lib().fa2_device_status(ctypes.byref(out)))
    return out.value
