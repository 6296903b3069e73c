"""The five benchmark configurations at FULL size: achieved error of O, dq, dk, dv against the
fp64 definition, next to the error of the reference's own arithmetic on the same inputs.

For each configuration the operator runs once at full size through the public API; then at least
four (batch, head) problems are compared

* with the fp64 closed-form oracle (oracle.naive_attention; its N x N matrices are evaluated with
  the same torch operations on the GPU, where a head of 32768 rows takes seconds instead of
  minutes): every element within max(5e-3 fp16 | 2e-2 bf16, one ulp of its own oracle value);
* with the restatement of the reference's kernels (oracle.reference_tiled, pinned to the
  reference's outputs by tests/test_oracle.py) fed the same inputs the way the reference would see
  them: cast to fp16 whatever the input dtype, results rounded to the input dtype
  (flash_attention_2.py:316,339,379).  "Never worse than the reference": rms error within
  conftest.RMS_FACTOR_VS_REFERENCE of the reference's (1.25 for fp16; 2.0 for bf16, see there),
  maximum within conftest.MAX_FACTOR_VS_REFERENCE (or inside the flat bound).

The numbers are printed and, when the environment variable ``FA2_B200_REPORT_DIR`` names a
directory, written to ``parity_<config>.json`` there.
"""

from __future__ import annotations

import json
import math
import os
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import (BASE_TOL, MAX_FACTOR_VS_REFERENCE, RMS_FACTOR_VS_REFERENCE, elementwise_tolerance, error_stats,
                      make_inputs)
from flash_attention_triton_b200 import _lib, flash_attention_v2
from oracle.attention_oracle import naive_attention, reference_tiled

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# name: (shape [B, H, N, d], dtype, scale, q/k multiplier, deterministic, sampled (b, h), tile of
# the reference restatement).  c4 runs one GPU's share of the 8-GPU split (2 of the 16 heads).
CONFIGS = {
    "c1": ((2, 4, 256, 64), torch.float16, 1.0 / 8.0, 1.0, True, [(0, 0), (0, 3), (1, 1), (1, 3)], 64),
    "c2": ((4, 16, 2048, 64), torch.float16, None, 1.0, True, [(0, 0), (1, 5), (2, 10), (3, 15)], 128),
    "c2-atomic": ((4, 16, 2048, 64), torch.float16, None, 1.0, False, [(0, 0), (1, 5), (2, 10), (3, 15)], 128),
    "c3": ((2, 32, 8192, 128), torch.bfloat16, None, 1.0, False, [(0, 0), (0, 17), (1, 8), (1, 31)], 128),
    "c4": ((1, 2, 32768, 128), torch.bfloat16, None, 1.0, False, [(0, 0), (0, 1)], 1024),
    "c5": ((8, 12, 4095, 32), torch.float16, 0.5, 3.0, True, [(0, 0), (3, 4), (5, 9), (7, 11)], 128),
}


@pytest.mark.parametrize("name", list(CONFIGS))
def test_error_at_full_size_against_oracle_and_reference_arithmetic(name):
    shape, dtype, scale, qk_mul, det, samples, block = CONFIGS[name]
    q, k, v, do = make_inputs(shape, dtype, seed=0, qk_mul=qk_mul)
    qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    out = flash_attention_v2(qd, kd, vd, scale, deterministic=det)
    out.backward(do.to(DEV))
    assert _lib.device_status() == 0
    got = {"o": out.detach(), "dq": qd.grad, "dk": kd.grad, "dv": vd.grad}
    rows = []
    worst = {key: {"max_ours": 0.0, "rms_ours": 0.0, "max_ref": 0.0, "rms_ref": 0.0} for key in got}
    n_ref = 0
    for (bi, hi) in samples:
        sl = lambda t: t[bi:bi + 1, hi:hi + 1]
        ref = naive_attention(sl(q), sl(k), sl(v), sl(do), scale, torch.float64, device=DEV)
        # the reference's arithmetic on the same problem; the long configuration affords one head
        theirs = None
        if n_ref < (1 if shape[2] > 8192 else len(samples)):
            n_ref += 1
            theirs = reference_tiled(sl(q).half().numpy(), sl(k).half().numpy(), sl(v).half().numpy(),
                                     sl(do).half().numpy(), scale or 1.0 / math.sqrt(shape[3]),
                                     block, block, block)
        for key in ("o", "dq", "dk", "dv"):
            mine = sl(got[key])
            e_ours, rms_ours = error_stats(mine, ref[key])
            over = ((mine.double() - ref[key]).abs() - elementwise_tolerance(dtype, ref[key])).max().item()
            row = {"config": name, "b": bi, "h": hi, "tensor": key, "max_ours": e_ours,
                   "rms_ours": rms_ours, "over_flat_bound": max(over, 0.0),
                   "max_abs_value": ref[key].abs().max().item()}
            if theirs is not None:
                t = torch.from_numpy(theirs[key].astype(np.float32)).to(dtype).to(DEV)
                row["max_ref"], row["rms_ref"] = error_stats(t, ref[key])
            rows.append(row)
            for stat in worst[key]:
                if stat in row:
                    worst[key][stat] = max(worst[key][stat], row[stat])
        del ref
    print(f"\n{name}: worst over {len(samples)} sampled (batch, head) problems")
    for key, w in worst.items():
        print(f"  {key}: max-abs ours {w['max_ours']:.3e} ref {w['max_ref']:.3e} | "
              f"rms ours {w['rms_ours']:.3e} ref {w['rms_ref']:.3e}")
    out_dir = os.environ.get("FA2_B200_REPORT_DIR")
    if out_dir and os.path.isdir(out_dir):
        (Path(out_dir) / f"parity_{name}.json").write_text(json.dumps({"worst": worst, "rows": rows}, indent=1))
    problems = []
    for row in rows:
        tag = f"{row['tensor']}[{row['b']},{row['h']}]"
        inside_flat = row["over_flat_bound"] <= 0.0
        if row["tensor"] == "o" and not inside_flat:
            problems.append(f"{tag}: max-abs {row['max_ours']:.3e} is over the flat bound")
        if "max_ref" in row:
            if row["rms_ours"] > RMS_FACTOR_VS_REFERENCE[dtype] * row["rms_ref"] + 1e-5:
                problems.append(f"{tag}: rms ours {row['rms_ours']:.3e} vs reference {row['rms_ref']:.3e}")
            if row["max_ours"] > max(BASE_TOL[dtype], MAX_FACTOR_VS_REFERENCE[dtype] * row["max_ref"]) and not inside_flat:
                problems.append(f"{tag}: max-abs ours {row['max_ours']:.3e} vs reference {row['max_ref']:.3e}")
        elif not inside_flat:
            problems.append(f"{tag}: max-abs {row['max_ours']:.3e} is over the flat bound")
    assert not problems, "; ".join(problems)
