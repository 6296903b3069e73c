"""Generate golden vectors from the reference's own kernels (run once, where the reference is mounted).

The reference has no golden files and needs a CUDA device through its public API, but its
three Triton kernels run unmodified on CPU tensors under Triton's interpreter
(``TRITON_INTERPRET=1``).  This script imports flash-attention-triton from ``--reference``
(a checkout of the project, its ``src`` directory), runs ``_forward_kernel`` and ``_flash_attention_backward`` on
seeded inputs and stores inputs + outputs as compressed ``.npz`` next to this file.  The
tests only read the ``.npz`` files; they never need the reference.

Usage:  python tests/golden/make_golden.py --reference /path/to/flash-attention-triton/src [--only NAME]
"""

from __future__ import annotations

import argparse
import math
import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"  # must precede the triton import

HERE = Path(__file__).resolve().parent

# name, (B, H, N, D), softmax_scale (None = default), q/k multiplier, fwd tile, bwd tile,
# seq-parallel, key rows (None = N; otherwise k and v have that many rows)
CASES = [
    ("c1_fp16_2x4x256x64_det", (2, 4, 256, 64), None, 1.0, 64, 64, False, None),
    ("ragged_fp16_1x2x191x32_det", (1, 2, 191, 32), 0.5, 3.0, 64, 64, False, None),
    ("ragged_fp16_1x2x191x32_seqpar", (1, 2, 191, 32), 0.5, 3.0, 64, 64, True, None),
    ("d128_fp16_1x2x160x128_det", (1, 2, 160, 128), None, 1.0, 32, 32, False, None),
    ("fewer_keys_fp16_1x2_q200_k70_d32_det", (1, 2, 200, 32), None, 1.0, 64, 64, False, 70),
    ("more_keys_fp16_1x2_q100_k170_d64_det", (1, 2, 100, 64), None, 1.0, 64, 64, False, 170),
]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path to flash-attention-triton/src")
    ap.add_argument("--only", default="", help="substring of the case names to (re)generate")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)

    import numpy as np
    import torch
    import triton

    # The reference asks the CUDA driver for the compute capability when it builds its kernel
    # cache key (_configurators_v2.py:48); there is no GPU where this script runs.
    torch.cuda.get_device_capability = lambda *a, **k: (10, 0)
    import flash_attention_triton.flash_attention_2 as fa
    from flash_attention_triton import KernelsConfigV2, init_to_zero_v2
    from flash_attention_triton._triton_kernels_v2 import _forward_kernel

    for name, (b, h, n, d), scale, qk_mul, fwd_blk, bwd_blk, seqpar, nk in CASES:
        if args.only not in name:
            continue
        nk = nk or n
        g = torch.Generator(device="cpu").manual_seed(0)
        q, k, v, do = (torch.randn(b, h, rows, d, generator=g) for rows in (n, nk, nk, n))
        q, k = q * qk_mul, k * qk_mul
        q, k, v, do = (t.half() for t in (q, k, v, do))
        sc = scale or 1.0 / math.sqrt(d)
        cfg = KernelsConfigV2(
            fwd_blk, fwd_blk, 16, 128, 32, 4, 8, 1,
            [triton.Config(
                {"BLOCK_Q_ROWS_SIZE": bwd_blk, "BLOCK_KV_COLS_SIZE": bwd_blk, "SEQUENCE_PARALLEL": seqpar},
                num_warps=4, num_stages=1, pre_hook=init_to_zero_v2("DQ"),
            )],
        )
        nr = math.ceil(n / cfg.max_headdim) * cfg.max_headdim
        out = torch.empty_like(q)
        lse = torch.empty(b, h, nr, dtype=torch.float32)
        spd = torch.empty_like(lse)
        bhd = max(triton.next_power_of_2(d), cfg.min_block_headdim)
        grid = (triton.cdiv(n, fwd_blk), b * h)
        _forward_kernel[grid](
            q, k, v, out, lse, spd, sc,
            q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
            v.stride(0), v.stride(1), v.stride(2), out.stride(0), out.stride(1), out.stride(2),
            h, n, nk, nr, d, n // 32, nk // 32, bhd,
            BLOCK_Q_ROWS_SIZE=fwd_blk, BLOCK_KV_COLS_SIZE=fwd_blk,
        )
        dq, dk, dv = (torch.empty_like(t) for t in (q, k, v))
        fa._flash_attention_backward(q, k, v, out, lse, dq, dk, dv, do, sc, cfg)
        np.savez_compressed(
            HERE / f"{name}.npz",
            q=q.numpy(), k=k.numpy(), v=v.numpy(), dout=do.numpy(),
            o=out.numpy(), lse=lse[:, :, :n].numpy(), dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy(),
            softmax_scale=np.float32(sc), fwd_block=np.int32(fwd_blk), bwd_block=np.int32(bwd_blk),
            sequence_parallel=np.bool_(seqpar),
        )
        print(f"wrote {name}.npz")


if __name__ == "__main__":
    main()
