"""CPU oracle for causal FlashAttention-2 forward + backward.  TEST INFRASTRUCTURE ONLY.

Nothing in the product path imports this module: it is the checker used by ``tests/``, by
``__graft_entry__.smoke()`` and by the CPU-baseline leg of ``bench.py``.

Two restatements of the reference (paths inside flash-attention-triton):

``naive_attention``
    The closed-form definition the reference's own tests compare against
    (``tests/test_flash_attention_2.py:289-294``: ``softmax(mask(Q K^T * s)) V`` with a
    lower-triangular mask) plus its analytic backward, evaluated in fp64 or fp32.  This is the
    arbiter for the tolerances (fp16 max-abs 5e-3, bf16 2e-2).

``reference_tiled``
    A numpy restatement of the arithmetic of the reference's three Triton kernels, keeping
    its rounding points: fp16 operands, fp32 accumulation, online softmax with the
    ``max(rowmax, lse_prev)`` update, fp16 cast of P before P V
    (``src/flash_attention_triton/_triton_kernels_v2.py:111-171``); backward with P recomputed
    from LSE, the scale folded into dS before its fp16 cast, fp16 P for dV
    (``_triton_kernels_v2.py:312-343``); delta in fp32 (``:607``); one fp32->fp16 rounding of
    dQ (``flash_attention_2.py:277``).  Pinned against the reference itself: the fixtures in
    ``tests/golden/`` are outputs of the reference's kernels executed by Triton's CPU
    interpreter (``tests/golden/make_golden.py``), and ``tests/test_oracle.py`` checks this
    restatement against them.
"""

from __future__ import annotations

import math

import numpy as np
import torch


def naive_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    dout: torch.Tensor | None = None,
    softmax_scale: float | None = None,
    dtype: torch.dtype = torch.float64,
    device: str | torch.device = "cpu",
) -> dict[str, torch.Tensor]:
    """Causal attention by its definition, with analytic gradients.

    Inputs ``[B, H, N, D]`` (any float dtype; they are up-cast to ``dtype`` as they are, so
    pass tensors already rounded to the kernel's 16-bit dtype to isolate kernel error).  ``k``
    and ``v`` may have a different number of rows than ``q``; the mask ``row >= col`` is then
    aligned at the top left, as in the reference's kernels (``_triton_kernels_v2.py:139-147``).
    Returns ``o, lse`` and, when ``dout`` is given, ``dq, dk, dv, delta``.  ``device`` is where
    the plain torch arithmetic of this definition runs (the CPU unless a test asks for the
    full-size configurations, whose N x N fp64 matrices per head are evaluated with the same
    torch operations on the GPU; results are returned on that device).
    Formula: ``tests/test_flash_attention_2.py:289-294`` of the reference; backward is the
    chain rule the reference's kernel implements (``_triton_kernels_v2.py:312-343``).
    """
    qf, kf, vf = (t.detach().to(device, dtype) for t in (q, k, v))
    n, d = qf.shape[-2], qf.shape[-1]
    scale = softmax_scale or 1.0 / math.sqrt(d)
    mask = torch.ones(n, kf.shape[-2], dtype=torch.bool, device=device).tril()
    s = (qf @ kf.transpose(-1, -2)) * scale
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    o = p @ vf
    out = {"o": o, "lse": lse}
    if dout is not None:
        dof = dout.detach().to(device, dtype)
        delta = (o * dof).sum(-1)
        dv = p.transpose(-1, -2) @ dof
        dp = dof @ vf.transpose(-1, -2)
        ds = p * (dp - delta[..., None]) * scale
        out.update({"dq": ds @ kf, "dk": ds.transpose(-1, -2) @ qf, "dv": dv, "delta": delta})
    return out


def naive_attention_per_head(q, k, v, dout, softmax_scale=None, dtype=torch.float32, device="cpu"):
    """Same as :func:`naive_attention` but looping over (batch, head) to bound memory
    (the score matrix is N^2 per head).  Returns tensors in ``dtype``."""
    b, h = q.shape[:2]
    keys = ["o", "lse", "dq", "dk", "dv", "delta"]
    acc: dict[str, list] = {key: [] for key in keys}
    for bi in range(b):
        for hi in range(h):
            r = naive_attention(
                q[bi : bi + 1, hi : hi + 1], k[bi : bi + 1, hi : hi + 1], v[bi : bi + 1, hi : hi + 1],
                dout[bi : bi + 1, hi : hi + 1], softmax_scale, dtype, device,
            )
            for key in keys:
                acc[key].append(r[key])
    return {
        key: torch.cat(vals, dim=1).reshape(b, h, *vals[0].shape[2:]) for key, vals in acc.items()
    }


def _f16(x: np.ndarray) -> np.ndarray:
    return x.astype(np.float16).astype(np.float32)


def reference_tiled(
    q: np.ndarray,
    k: np.ndarray,
    v: np.ndarray,
    dout: np.ndarray,
    softmax_scale: float,
    block_q: int = 64,
    block_kv: int = 64,
    bwd_block: int = 64,
) -> dict[str, np.ndarray]:
    """Restates the reference kernels' arithmetic for one problem ``[B, H, N, D]`` (fp16 data).

    ``block_q`` x ``block_kv`` are the forward tile sizes (``BLOCK_Q_ROWS_SIZE`` /
    ``BLOCK_KV_COLS_SIZE``); ``bwd_block`` is the (square) backward tile.  dQ is accumulated in
    ascending KV-tile order like the reference's sequential mode
    (``_triton_kernels_v2.py:495-525``).  Returns fp16 ``o, dq, dk, dv`` and fp32 ``lse, delta``.
    """
    q, k, v, dout = (np.asarray(t, dtype=np.float16).astype(np.float32) for t in (q, k, v, dout))
    b, h, n, d = q.shape
    nk = k.shape[2]  # key rows; the causal mask is aligned at the top left (:139-147)
    s32 = np.float32(softmax_scale)
    o = np.zeros((b, h, n, d), np.float32)
    lse_out = np.zeros((b, h, n), np.float32)
    neg_inf = np.float32(-np.inf)
    with np.errstate(invalid="ignore", divide="ignore", over="ignore"):
        # ---------------------------------------------------------------- forward, :111-171
        for bi in range(b):
            for hi in range(h):
                for q0 in range(0, n, block_q):
                    rows = np.arange(q0, min(q0 + block_q, n))
                    qb = q[bi, hi, rows]
                    lse = np.full(len(rows), neg_inf, np.float32)
                    m = np.full(len(rows), neg_inf, np.float32)
                    acc = np.zeros((len(rows), d), np.float32)
                    end = min(q0 + block_q, nk)  # (:76)
                    for k0 in range(0, end, block_kv):
                        cols = np.arange(k0, min(k0 + block_kv, nk))
                        sc = qb @ k[bi, hi, cols].T  # fp32 accumulate (:137-138)
                        sc = np.where(rows[:, None] >= cols[None, :], sc, neg_inf)  # (:142-147)
                        m_new = np.maximum((sc * s32).max(axis=1), lse)  # (:150) max with lse
                        p = np.exp(sc * s32 - m_new[:, None])  # (:151)
                        l = p.sum(axis=1, dtype=np.float32)  # (:152)
                        acc = acc * np.exp(m - m_new)[:, None] + _f16(p) @ v[bi, hi, cols]  # (:156-160)
                        m = m_new
                        lse = m_new + np.log(np.exp(lse - m_new) + l)  # (:163-165)
                    o[bi, hi, rows] = acc * np.exp(m - lse)[:, None]  # (:168-171)
                    lse_out[bi, hi, rows] = lse
        o16 = o.astype(np.float16)
        o = o16.astype(np.float32)
        # ---------------------------------------------------------------- preprocess, :607
        delta = (o * dout).sum(axis=-1, dtype=np.float32)
        # ---------------------------------------------------------------- backward, :312-343
        dq_acc = np.zeros((b, h, n, d), np.float32)
        dk = np.zeros((b, h, nk, d), np.float32)
        dv = np.zeros((b, h, nk, d), np.float32)
        for bi in range(b):
            for hi in range(h):
                for k0 in range(0, nk, bwd_block):
                    cols = np.arange(k0, min(k0 + bwd_block, nk))
                    kb, vb = k[bi, hi, cols], v[bi, hi, cols]
                    dk_acc = np.zeros((len(cols), d), np.float32)
                    dv_acc = np.zeros((len(cols), d), np.float32)
                    q_start = (k0 // bwd_block) * bwd_block
                    for q0 in range(q_start, n, bwd_block):
                        rows = np.arange(q0, min(q0 + bwd_block, n))
                        qb, dob = q[bi, hi, rows], dout[bi, hi, rows]
                        sc = qb @ kb.T
                        sc = np.where(rows[:, None] >= cols[None, :], sc, neg_inf)
                        p = np.exp(sc * s32 - lse_out[bi, hi, rows][:, None])  # (:321-322)
                        dp = dob @ vb.T  # (:329)
                        ds = _f16(p * (dp - delta[bi, hi, rows][:, None]) * s32)  # (:330-332)
                        dk_acc += ds.T @ qb  # (:333)
                        dv_acc += _f16(p).T @ dob  # (:334)
                        dq_acc[bi, hi, rows] += ds @ kb  # (:338-343)
                    dk[bi, hi, cols] = dk_acc
                    dv[bi, hi, cols] = dv_acc
    return {
        "o": o16,
        "lse": lse_out,
        "delta": delta,
        "dq": dq_acc.astype(np.float16),  # flash_attention_2.py:277
        "dk": dk.astype(np.float16),
        "dv": dv.astype(np.float16),
    }
