"""Benchmark of the causal attention forward + backward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c3|c2|c5|c4|d256] [--deterministic] [--scaling weak|strong]

A "step" is one forward + backward (forward, preprocess, backward main, plus memset/convert
in the atomic mode) over one batch of seeded synthetic inputs of the workload's shape.
Default workload: bf16, q,k,v,dO [B=2, H=32, N=8192, d=128], iid N(0,1), scale 1/sqrt(128).

Printed JSON (one line, rank 0):
  value        whole-job causal fwd+bwd TFLOP/s with inputs resident in HBM, all kernels launched
               through the C ABI on preallocated buffers, timed with CUDA events, max over ranks.
               FLOPs = 3.5 * 4*B*H*N^2*d/2 (FlashAttention convention, causal-halved; the extra
               recompute of the deterministic two-kernel backward is not counted).
  e2e          same metric through flash_attention_v2(...).backward() starting from pinned HOST
               tensors: host->device copies of q,k,v,dO and device->host copies of o,dq,dk,dv are
               inside the timed region, every step; copy-in, compute and copy-out of
               neighbouring steps overlap on three streams.
  roofline     the dominant kernel of the step, bwd_dkdv_kernel (half of the step: 4 of the
               backward's 5 tile products), against the tensor roofline (achieved = its
               algorithmic FLOPs / its average duration, peak = MEASURED_PEAKS.json bf16_tflops),
               then backward_call (both kernels of fa2_bwd together) and one entry per other
               kernel: fwd, preprocess (HBM), and bwd_consume_kernel (HBM: it reads the spilled
               dS tiles) or bwd_dq_kernel.  In the atomic mode and at head dim 256, where no
               event separates the kernels of the call, the top level is the call.  Every
               duration comes from CUDA events recorded between the calls of the timed steps
               themselves (the one between the two backward kernels through fa2_bwd_mark_between),
               so sum_of_parts_ms = ms_per_step up to the event overhead.  traffic = DRAM bytes of
               the kernel per launch from an ncu capture (see NCU_DKDV_DRAM_MB_PER_24).
               At head dims 32 and 64 the entries carry softmax_ceiling (see softmax_ceiling).
  sustained    the same device-resident step run back to back for about a second under the
               clock sampler (the timed region is too short for NVML's clock averaging):
               steps, ms_per_step, value, its fraction of the sustained GEMM peak, the clocks /
               throttle reasons seen, and mcycles_per_step = ms x median SM MHz (comparable
               between GPUs and power states).
  strong       strong-scaling legs (default workload only): the c4 shape [1,16,32768,128] and, at
               N > 1, the c3 shape, split over the ranks by (batch, head) with shard_slab;
               value = whole-job FLOPs / slowest rank's time.  --no-strong leaves them out.
  triton_reference  the reference's own Triton kernels timed on this GPU in a child process, when
               the reference is installed under baseline/_ref (N=1 only; --no-triton-reference).
  cpu_baseline naive fp32 PyTorch causal attention fwd+bwd on the host cores over a bounded
               sample of the same workload's heads (rank 0, N=1 only).
  clocks, gpu_launches  SM clock / throttle reasons sampled during the timed region; kernels of
               this library launched inside it.

Multi-GPU: one process per GPU (torchrun); every (batch, head) problem is independent, so
ranks share nothing on the data path.  --scaling weak (default): every rank runs the whole
workload shape on its own data; --scaling strong: the workload's B*H problems are split
across ranks (shard_slab).  --impl reference times the CPU oracle (the reference has no CPU
implementation of its own; the oracle restates its test-suite formula) on rank 0.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (B, H, N, D, dtype, qk_mul, scale)
    "c2": (4, 16, 2048, 64, torch.float16, 1.0, None),
    "c3": (2, 32, 8192, 128, torch.bfloat16, 1.0, None),
    "c4": (1, 16, 32768, 128, torch.bfloat16, 1.0, None),
    "c5": (8, 12, 4095, 32, torch.float16, 3.0, 0.5),
    # head dim 256 (the reference's max_headdim): forward on the split plan, backward through the
    # scores + consumer kernels; d256small for profiler captures
    "d256": (2, 16, 8192, 256, torch.bfloat16, 1.0, None),
    "d256small": (1, 16, 8192, 256, torch.bfloat16, 1.0, None),
    # reduced C3 (same N, d, dtype; 24 instead of 64 batch*heads) for profiler captures
    "c3small": (1, 24, 8192, 128, torch.bfloat16, 1.0, None),
}
METRIC = "causal attn fwd+bwd TFLOP/s, bf16 N=8192 d=128"


# DRAM bytes (read + write) of the backward-main kernels measured by ncu on the reduced C3
# workload (24 batch*head problems, N=8192, d=128): fused kernel 381.8 + 209.7 MB and the convert
# 100.7 + 20.1 MB; the recompute pair 208.6 + 74.7 MB (dK/dV) plus 204.3 + 36.8 MB (dQ); the spill
# pair 329.6 + 1679.5 MB (dK/dV, writes the dS tiles) plus 1744.1 + 46.2 MB (dQ, reads them back).
NCU_BWD_DRAM_MB_PER_24 = {0: 381.8 + 209.7 + 100.7 + 20.1, 1: 208.6 + 74.7 + 204.3 + 36.8,
                          2: 329.6 + 1679.5 + 1744.1 + 46.2}
NCU_DKDV_DRAM_MB_PER_24 = {1: 208.6 + 74.7, 2: 329.6 + 1679.5}  # the dK/dV kernel alone

# Polynomial share of the exponentials (of every 8 column pairs) the kernels are built with
# (FA2_FWD_POLY_PAIRS_PER_8 in csrc/fwd.cu, FA2_BWD_POLY_PAIRS_PER_8 in csrc/bwd_roles.cuh).
POLY_SHARE = {"fwd": 3 / 8, "bwd": 2 / 8}  # at the head dims the ceiling is reported for (<= 64)


def softmax_ceiling(d, which):
    """Upper bound on the tensor-pipe fraction of a 128 x 128 score tile set by the softmax work.

    Per SM and tile: the tensor pipe needs 8 d cycles in the forward (2 tile products) and 20 d in
    the dK/dV kernel (5 products counted at 8192 dense 16-bit FLOP / clk / SM); the 16384
    exponentials need 1024 (1 - p) cycles of the MUFU (16 / clk / SM) for a polynomial share p;
    all the per-element instructions (scale, max, sum, pack; in the backward also dP - delta and
    the product with P) plus the MUFU issues and about 5.5 instructions per polynomial
    exponential share 128 issue slots / clk / SM.  The slower of the two is the floor under the
    tile time; at d = 128 it is below the tensor time, at d <= 64 above it.
    """
    p = POLY_SHARE[which]
    base = 2.5 if which == "fwd" else 6.0
    mufu = 1024.0 * (1.0 - p)
    issue = 16384.0 * (base + (1.0 - p) + 5.5 * p) / 128.0
    tensor_cycles = (8.0 if which == "fwd" else 20.0) * d
    floor = max(mufu, issue)
    return {"tensor_cycles": tensor_cycles, "mufu_cycles": mufu, "issue_cycles": issue,
            "frac_of_tensor_peak": min(1.0, tensor_cycles / floor)}


def traffic_bytes(d, mode, batch_heads, n=8192):
    if d != 128 or n != 8192 or NCU_BWD_DRAM_MB_PER_24[mode] is None:
        return None
    return NCU_BWD_DRAM_MB_PER_24[mode] * 1e6 * batch_heads / 24.0


def fwd_flops(b, h, n, d):
    return 4.0 * b * h * n * n * d / 2.0


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        j = json.loads(p.read_text())
        return {"bf16": float(j["bf16_tflops"]), "bf16_sustained": float(j["bf16_tflops_sustained"]),
                "hbm": float(j["hbm_gbs"]), "source": "measured"}
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: clocks are reported as null
            self.nvml = None

    def _run(self):
        n = self.nvml
        names = {
            "hw_slowdown": getattr(n, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(n, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(n, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(n, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self.nvml:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def make_inputs(shape, dtype, seed, qk_mul):
    g = torch.Generator(device="cpu").manual_seed(seed)
    q, k, v, do = (torch.randn(*shape, generator=g) for _ in range(4))
    return tuple((t * m).to(dtype) for t, m in ((q, qk_mul), (k, qk_mul), (v, 1.0), (do, 1.0)))


def cpu_baseline(b, h, n, d, dtype, qk_mul, scale, budget_s=12.0, max_heads=32):
    """Naive fp32 causal attention fwd+bwd (the oracle), one head at a time, on all host threads."""
    from oracle.attention_oracle import naive_attention

    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, do = make_inputs((1, 1, n, d), dtype, 123, qk_mul)
    naive_attention(q, k, v, do, scale, torch.float32)  # warm-up
    heads, t0 = 0, time.perf_counter()
    while heads < max_heads and (heads == 0 or time.perf_counter() - t0 < budget_s):
        naive_attention(q, k, v, do, scale, torch.float32)
        heads += 1
    el = time.perf_counter() - t0
    tf = 3.5 * fwd_flops(1, 1, n, d) * heads / el / 1e12
    return {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{heads} of {b * h} (batch,head) problems of the workload, fp32 naive "
                      f"attention + analytic backward, {el:.1f} s"}


def triton_reference(workload, our_ms):
    """The reference's own Triton kernels on this GPU (informational: the unmodified package from
    baseline/_ref through its public API, in a child process, after every timed region)."""
    import subprocess

    cmd = [sys.executable, str(ROOT / "baseline" / "reference_triton_bench.py"), "--workload", workload,
           "--steps", "3"]
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=420)
    except Exception as exc:  # noqa: BLE001
        return {"unavailable": repr(exc)[:200]}
    recs = []
    for ln in out.stdout.splitlines():
        try:
            recs.append(json.loads(ln))
        except ValueError:
            pass
    if not recs or "unavailable" in recs[0]:
        return {"unavailable": (recs[0]["unavailable"] if recs else (out.stderr or "no output")[-200:])}
    res = {"config": WORKLOADS[workload][:4], "note": recs[0].get("note"), "triton": recs[0].get("triton")}
    for r in recs:
        key = "deterministic" if r.get("deterministic") else "default"
        default_err = r.get("tried", {}).get("default", {}).get("error")
        res[key] = {"fwd_bwd_ms": r.get("fwd_bwd_ms"), "tflops": r.get("fwd_bwd_tflops"),
                    "fwd_ms": r.get("fwd_ms"), "best_config": r.get("config"),
                    "default_config_error": default_err,
                    "ours_over_triton": (r["fwd_bwd_ms"] / our_ms) if r.get("fwd_bwd_ms") else None}
    return res


def run_reference_arm(args, rank, world):
    wl = WORKLOADS[args.workload]
    b, h, n, d, dtype, qk_mul, scale = wl
    if rank != 0:
        return
    from oracle.attention_oracle import naive_attention

    torch.set_num_threads(os.cpu_count() or 1)
    heads_per_step = 1 if n >= 8192 else max(1, min(b * h, (8192 // n) ** 2))
    q, k, v, do = make_inputs((1, heads_per_step, n, d), dtype, 123, qk_mul)
    for _ in range(args.warmup):
        naive_attention(q[:, :1], k[:, :1], v[:, :1], do[:, :1], scale, torch.float32)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for hh in range(heads_per_step):
            naive_attention(q[:, hh:hh + 1], k[:, hh:hh + 1], v[:, hh:hh + 1], do[:, hh:hh + 1],
                            scale, torch.float32)
    el = time.perf_counter() - t0
    tf = 3.5 * fwd_flops(1, heads_per_step, n, d) * args.steps / el / 1e12
    sample = (f"each step = {heads_per_step} of the workload's {b * h} (batch,head) problems, "
              "fp32 naive attention + analytic backward on host cores")
    line = {
        "impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(args, wl, world),
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, wl, world):
    from flash_attention_triton_b200 import api

    b, h, n, d, dtype, qk_mul, scale = wl
    return {
        "workload": f"{args.workload}: causal self-attention fwd+bwd, q,k,v,dO [B={b},H={h},N={n},d={d}] "
                    f"{str(dtype)[6:]}, iid N(0,{qk_mul:g}) q,k / N(0,1) v,dO, scale "
                    f"{scale if scale else '1/sqrt(d)'}",
        "deterministic": bool(args.deterministic),
        "bwd_mode": args.bwd_mode or ("atomic", "recompute", "spill")[
            api._backward_mode(bool(args.deterministic), d, n)],
        "batch_heads_per_gpu": b * h if args.scaling == "weak" else f"{b * h}/{world}",
        "l2": "inputs (4 x %.0f MB per step) exceed the 126 MB L2; no explicit flush" % (b * h * n * d * 2 / 1e6),
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--deterministic", action="store_true")
    ap.add_argument("--bwd-mode", default="", choices=["", "atomic", "recompute", "spill"],
                    help="force a dQ strategy instead of the one the API picks")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-strong", action="store_true", help="skip the strong-scaling legs (c3, c4 split over the GPUs)")
    ap.add_argument("--no-triton-reference", action="store_true")
    ap.add_argument("--sustain-seconds", type=float, default=1.0,
                    help="extra untimed-for-the-metric run of the same step under the clock sampler")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch.distributed as dist

    from flash_attention_triton_b200 import _lib, api, flash_attention_v2, shard_slab

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    wl = WORKLOADS[args.workload]
    b, h, n, d, dtype, qk_mul, scale_opt = wl
    scale = scale_opt or 1.0 / math.sqrt(d)
    code = 0 if dtype == torch.float16 else 1
    det = int(args.deterministic)
    # dQ strategy: what flash_attention_v2(..., deterministic=args.deterministic) would pick
    # (0 atomic, 1 recompute, 2 spill), unless --bwd-mode names one.
    mode = ({"atomic": 0, "recompute": 1, "spill": 2}[args.bwd_mode] if args.bwd_mode
            else api._backward_mode(bool(det), d, n))

    # Inputs: seeded on the CPU, then moved.  weak: each rank its own seed, whole shape.
    # strong: one global tensor (seed 0), each rank takes its contiguous (batch, head) slab.
    if args.scaling == "weak":
        host = make_inputs((b, h, n, d), dtype, rank, qk_mul)
    else:
        host = tuple(shard_slab(t, world, rank).contiguous() for t in make_inputs((b, h, n, d), dtype, 0, qk_mul))
    host = tuple(t.pin_memory() for t in host)
    lb, lh = host[0].shape[0], host[0].shape[1]
    my_fwd_flops = fwd_flops(lb, lh, n, d)

    lib = _lib.lib()
    peaks = load_peaks()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_over_ranks(x, op):
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=op)
        return float(t.item())

    def max_over_ranks(x):
        return reduce_over_ranks(x, dist.ReduceOp.MAX if world > 1 else None)

    def sum_over_ranks(x):
        return reduce_over_ranks(x, dist.ReduceOp.SUM if world > 1 else None)

    class Problem:
        """Device-resident buffers of one problem and the three C-ABI calls of a step on them."""

        def __init__(self, tensors, n, d, code, scale, mode):
            self.q, self.k, self.v, self.do = (t.to(dev) for t in tensors)
            self.lb, self.lh = self.q.shape[0], self.q.shape[1]
            self.n, self.d, self.code, self.scale, self.mode = n, d, code, scale, mode
            self.o, self.dq, self.dk, self.dv = (torch.empty_like(self.q) for _ in range(4))
            self.lse = torch.empty(self.lb, self.lh, n, device=dev, dtype=torch.float32)
            self.rowstats = torch.empty(lib.fa2_rowstats_bytes(self.lb, self.lh, n) // 4, device=dev,
                                        dtype=torch.float32)
            # Workspace: what fa2_bwd_workspace_bytes recommends, except that the spill modes get
            # the tiles of ALL heads when that stays under 24 GiB, so that the backward is one
            # chunk and the event between its two kernels splits the whole call (the recommended
            # size, chunks of 2048 tiles, costs 0.6 % more on the default workload; the e2e leg
            # goes through the Python API and runs with it).
            self.wsb = lib.fa2_bwd_workspace_bytes(self.lb, self.lh, n, d, mode)
            if mode == 2 or d > 128:
                everything = lib.fa2_bwd_workspace_bytes(1, 1, n, d, mode) * self.lb * self.lh
                if everything <= 24 << 30:
                    self.wsb = everything
            self.ws = torch.empty(max(self.wsb, 256), device=dev, dtype=torch.uint8)
            self.stream = torch.cuda.current_stream().cuda_stream
            self.fwd_flops = fwd_flops(self.lb, self.lh, n, d)

        def fwd(self):
            _lib.check("fa2_fwd", lib.fa2_fwd(
                self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.o.data_ptr(),
                self.lse.data_ptr(), self.lb, self.lh, self.n, self.d, self.code, self.scale, self.stream))

        def pre(self):
            _lib.check("fa2_bwd_preprocess", lib.fa2_bwd_preprocess(
                self.o.data_ptr(), self.do.data_ptr(), self.lse.data_ptr(), self.rowstats.data_ptr(),
                self.lb, self.lh, self.n, self.d, self.code, self.stream))

        def bwd(self):
            _lib.check("fa2_bwd", lib.fa2_bwd(
                self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.do.data_ptr(),
                self.rowstats.data_ptr(), self.dq.data_ptr(), self.dk.data_ptr(), self.dv.data_ptr(),
                self.ws.data_ptr() if self.wsb else None, self.wsb, self.lb, self.lh, self.n, self.d,
                self.code, self.scale, self.mode, self.stream))

        def step(self):
            self.fwd()
            self.pre()
            self.bwd()

        def launches_per_step(self):
            """Kernels of this library per step: forward, preprocess and the backward-main kernels
            of the mode (atomic: memset + fused kernel + convert; recompute: dK/dV + dQ; spill:
            dK/dV + dQ per chunk of the workspace; head dims above 128: scores + three consumers
            per chunk)."""
            if self.mode == 2 or self.d > 128:
                tiles = (self.n + 127) // 128
                per_head = tiles * (tiles + 1) // 2 * 32768 * (2 if self.d > 128 else 1)
                chunks = -(-self.lb * self.lh * per_head // max(self.wsb, 1))
                return 2 + chunks * (4 if self.d > 128 else 2)
            return 4

        def timed(self, steps, warmup, split=False):
            """ms per step over `steps` steps after `warmup`, max over ranks, barrier on both sides.
            With split, every step also records events between its calls (and between the two
            kernels of the backward call where it has two), and the per-call means are returned:
            they are parts of the very steps that give the headline."""
            for _ in range(warmup):
                self.step()
            st = _lib.device_status()
            if st != 0:
                raise RuntimeError(f"kernel status word {st:#x} after warm-up")
            two_kernels = self.mode in (1, 2) and self.d <= 128
            marks = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(steps if split else 0)]
            for evs in marks:  # an event has no handle before its first record
                for e in evs:
                    e.record()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            ev0.record()
            for i in range(steps):
                if split:
                    m = marks[i]
                    m[0].record()
                    self.fwd()
                    m[1].record()
                    self.pre()
                    m[2].record()
                    if two_kernels:
                        lib.fa2_bwd_mark_between(m[3].cuda_event)
                    self.bwd()
                    m[4].record()
                else:
                    self.step()
            ev1.record()
            torch.cuda.synchronize()
            barrier()
            ms = max_over_ranks(ev0.elapsed_time(ev1)) / steps
            parts = None
            if split:
                mean = lambda i, j: sum(m[i].elapsed_time(m[j]) for m in marks) / steps
                parts = {"fwd": mean(0, 1), "pre": mean(1, 2), "bwd": mean(2, 4)}
                if two_kernels:
                    parts["bwd_first"], parts["bwd_second"] = mean(2, 3), mean(3, 4)
                parts = {key: max_over_ranks(val) for key, val in parts.items()}
            return ms, parts

    prob = Problem(host, n, d, code, scale, mode)
    lb, lh = prob.lb, prob.lh
    prob_wsb = prob.wsb
    q = prob.q
    my_fwd_flops = prob.fwd_flops
    total_fwd_flops = sum_over_ranks(my_fwd_flops)

    # ------------------------------------------------------------ timed region (device-resident)
    with ClockSampler(local_rank) as clocks:
        ms_per_step, parts = prob.timed(args.steps, args.warmup, split=True)
    value = 3.5 * total_fwd_flops / (ms_per_step * 1e-3) / 1e12
    launches_per_step = prob.launches_per_step()

    # ------------------------------------------------------------ rooflines, from the same steps
    ms_fwd, ms_pre, ms_bwd = parts["fwd"], parts["pre"], parts["bwd"]
    bwd_tf = 2.5 * my_fwd_flops / (ms_bwd * 1e-3) / 1e12
    fwd_tf = my_fwd_flops / (ms_fwd * 1e-3) / 1e12
    pre_bytes = 2.0 * lb * lh * n * d * 2 + lb * lh * n * 4 * 3
    tensor = lambda tf: {"achieved": tf, "frac": tf / peaks["bf16"], "frac_of_sustained": tf / peaks["bf16_sustained"]}
    hbm = lambda nbytes, ms: {"bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": peaks["hbm"],
                              "unit": "GB/s", "frac": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm"], "ms": ms}
    def ceiling(which, tf):
        # head dims 32 and 64: the softmax work, not the tensor pipe, bounds a tile
        c = softmax_ceiling(d, which)
        if c["frac_of_tensor_peak"] >= 1.0:
            return {}
        top = c["frac_of_tensor_peak"] * peaks["bf16"]
        return {"bound": "exp", "softmax_ceiling": {**c, "tflops": top, "frac": tf / top}}

    call_names = ("bwd_dkdv_kernel (fused dQ atomics) + memset + dq_convert",
                  "bwd_dkdv_kernel + bwd_dq_kernel (S, dP recomputed)",
                  "bwd_dkdv_kernel (dS tiles spilled) + bwd_consume_kernel (dQ)")
    backward_call = {
        "kernels": "bwd_scores_wide_kernel + bwd_consume_kernel x3 (dV, dK, dQ)" if d > 128 else call_names[mode],
        **tensor(bwd_tf), "ms": ms_bwd, "algorithmic_flops": 2.5 * my_fwd_flops,
        "traffic": traffic_bytes(d, mode, lb * lh, n),
    }
    # The top level is the DOMINANT kernel of the step.  Where the backward call is two kernels
    # and the event between them exists, that is bwd_dkdv_kernel (4 of the backward's 5 tile
    # products; about half of the step), else the backward call as a whole.
    split_bwd = "bwd_first" in parts and d <= 128
    pad_d = 32 if d <= 32 else 64 if d <= 64 else 128
    if split_bwd:
        t1, t2 = parts["bwd_first"], parts["bwd_second"]
        dkdv_flops = 0.8 * 2.5 * my_fwd_flops
        dkdv_tf = dkdv_flops / (t1 * 1e-3) / 1e12
        top = {"kernel": "bwd_dkdv_kernel<%d, %s, %s>" % (pad_d, "bf16" if code else "fp16", ("", "plain", "spill")[mode]),
               **tensor(dkdv_tf), "ms": t1, "algorithmic_flops": dkdv_flops,
               "share_of_step": t1 / ms_per_step,
               "traffic": NCU_DKDV_DRAM_MB_PER_24.get(mode) and (
                   NCU_DKDV_DRAM_MB_PER_24[mode] * 1e6 * lb * lh / 24.0 if (d, n) == (128, 8192) else None),
               **ceiling("bwd", dkdv_tf)}
    else:
        top = {"kernel": backward_call["kernels"], **tensor(bwd_tf), "ms": ms_bwd,
               "algorithmic_flops": 2.5 * my_fwd_flops, "share_of_step": ms_bwd / ms_per_step,
               "traffic": backward_call["traffic"]}
    roofline = {
        "bound": "tensor", "peak": peaks["bf16"], "unit": "TFLOP/s", **top,
        "peak_source": f"{peaks['source']} burst bf16 GEMM; frac_of_sustained uses the sustained one",
        "timing": "CUDA events between the calls of the timed steps themselves (and between the two kernels of the "
                  "backward call): fwd + pre + bwd = ms_per_step",
        "traffic_note": "dram__bytes_read+write of this kernel per launch, from an ncu capture of 24 batch*head "
                        "problems (d=128, N=8192) scaled by batch*head; null for other shapes",
        "backward_call": backward_call,
        "fwd": {**tensor(fwd_tf), "ms": ms_fwd, **ceiling("fwd", fwd_tf)},
        "bwd_ms": ms_bwd,
        "preprocess": hbm(pre_bytes, ms_pre),
        "sum_of_parts_ms": ms_fwd + ms_pre + ms_bwd,
    }
    if split_bwd:
        # second kernel: the fifth tile product (spill: bound by reading the 32 KiB dS tile and
        # the K tile per product) or, recomputing, 3 products and the exponentials
        tiles = (n + 127) // 128
        if mode == 2:
            scratch = lb * lh * tiles * (tiles + 1) // 2 * 32768
            roofline["bwd_consume_kernel"] = {
                **hbm(scratch + 2.0 * lb * lh * n * d * 2, t2),
                "bytes": "the dS scratch read once + K read and dQ written once (K tiles are re-read from L2)",
                "tensor_frac": 0.2 * 2.5 * my_fwd_flops / (t2 * 1e-3) / 1e12 / peaks["bf16"]}
        else:
            roofline["bwd_dq_kernel"] = {**tensor(0.2 * 2.5 * my_fwd_flops / (t2 * 1e-3) / 1e12), "ms": t2,
                                         "note": "3 tile products and the exponentials run for 1 counted"}

    # ------------------------------------------------------------ end to end (host buffers)
    e2e = None
    if not args.no_e2e:
        # Every step copies its q, k, v, dO from pinned host memory, runs the public API and
        # copies O, dq, dk, dv back.  The three stages run on three streams over two sets of
        # device input buffers, so step i's copy-out, step i+1's compute and step i+2's copy-in
        # overlap (PCIe is full duplex); all copies of all timed steps are inside the events.
        outs_host = [torch.empty(q.shape, dtype=dtype).pin_memory() for _ in range(4)]
        main = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        dev_in = [[torch.empty(q.shape, dtype=dtype, device=dev) for _ in range(4)] for _ in range(2)]
        in_ready = [torch.cuda.Event() for _ in range(2)]
        in_free = [torch.cuda.Event() for _ in range(2)]
        out_ready = torch.cuda.Event()
        step_no = [0]

        def e2e_step():
            b = step_no[0] % 2
            step_no[0] += 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(in_free[b])  # the step that last read this buffer set is done
                for dst, src in zip(dev_in[b], host):
                    dst.copy_(src, non_blocking=True)
                in_ready[b].record(s_in)
            main.wait_event(in_ready[b])
            qd, kd, vd = (t.detach().requires_grad_(True) for t in dev_in[b][:3])
            out = flash_attention_v2(qd, kd, vd, scale_opt, bool(det))
            out.backward(dev_in[b][3])
            in_free[b].record(main)
            out_ready.record(main)
            results = (out.detach(), qd.grad, kd.grad, vd.grad)
            with torch.cuda.stream(s_out):
                s_out.wait_event(out_ready)
                for dst, src in zip(outs_host, results):
                    src.record_stream(s_out)
                    dst.copy_(src, non_blocking=True)

        for _ in range(3):
            e2e_step()
        torch.cuda.synchronize()
        e_steps = max(3, args.steps)  # the same K steps; fill and drain of the copy pipeline are inside
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        for _ in range(e_steps):
            e2e_step()
        main.wait_stream(s_out)  # the last step's results have reached the host
        main.wait_stream(s_in)
        ev1.record()
        torch.cuda.synchronize()
        barrier()
        e_ms = max_over_ranks(ev0.elapsed_time(ev1)) / e_steps
        nbytes = q.numel() * q.element_size()
        e2e = {"value": 3.5 * total_fwd_flops / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "ms_per_step": e_ms, "h2d_bytes_per_step": 4 * nbytes, "d2h_bytes_per_step": 4 * nbytes}

    # ------------------------------------------------------------ the same step, sustained
    # The timed region lasts tens of milliseconds, shorter than NVML's clock averaging, so its
    # clock samples mostly show the idle clock.  Run the same step back to back for about a
    # second under the sampler: this is where the power cap and the clock it settles at show.
    sustained = None
    if args.sustain_seconds > 0:
        n_sus = max(args.steps, int(args.sustain_seconds * 1e3 / ms_per_step))
        with ClockSampler(local_rank) as sus_clocks:
            sus_ms, _ = prob.timed(n_sus, 0)
        sus_value = 3.5 * total_fwd_flops / (sus_ms * 1e-3) / 1e12
        sus_clock = sus_clocks.summary()
        sustained = {"steps": n_sus, "ms_per_step": sus_ms, "value": sus_value, "unit": "TFLOP/s",
                     "frac_of_sustained_peak": sus_value / world / peaks["bf16_sustained"],
                     "clocks": sus_clock,
                     # time x clock: what the step costs in SM cycles, comparable between GPUs of the
                     # pool and between runs whose power state differs
                     "mcycles_per_step": sus_ms * sus_clock["sm_mhz"] / 1e3 if sus_clock["sm_mhz"] else None}

    # ------------------------------------------------------------ strong scaling of the two split
    # configurations: one seeded global problem, each rank its contiguous (batch, head) slab
    # (shard_slab), no collective on the data path; value = whole-job FLOPs / slowest rank's time.
    def strong_leg(name, steps, warmup):
        lb_, lh_, n_, d_, dtype_, qk_, sc_ = WORKLOADS[name]
        if lb_ * lh_ % world:
            return {"skipped": f"{lb_ * lh_} problems do not split evenly over {world} GPUs"}
        tensors = tuple(shard_slab(t, world, rank).contiguous()
                        for t in make_inputs((lb_, lh_, n_, d_), dtype_, 0, qk_))
        p_ = Problem(tensors, n_, d_, 0 if dtype_ == torch.float16 else 1, sc_ or 1.0 / math.sqrt(d_),
                     api._backward_mode(bool(det), d_, n_))
        ms_, _ = p_.timed(steps, warmup)
        flops = 3.5 * fwd_flops(lb_, lh_, n_, d_)
        return {"workload": name, "shape": [lb_, lh_, n_, d_], "batch_heads_per_gpu": lb_ * lh_ // world,
                "steps": steps, "ms_per_step": ms_, "value": flops / (ms_ * 1e-3) / 1e12, "unit": "TFLOP/s",
                "per_gpu_tflops": flops / (ms_ * 1e-3) / 1e12 / world,
                "frac_of_burst_peak": flops / (ms_ * 1e-3) / 1e12 / world / peaks["bf16"]}

    strong = None
    if args.workload == "c3" and args.scaling == "weak" and not args.no_strong:
        del prob.ws  # the legs bring their own scratch
        torch.cuda.empty_cache()
        strong = {"c4": strong_leg("c4", max(3, args.steps // 4), 3)}
        if world > 1:
            strong["c3"] = strong_leg("c3", args.steps, args.warmup)

    st = _lib.device_status()
    if st != 0:
        raise RuntimeError(f"kernel status word {st:#x} after the timed region")

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": str(dtype)[6:].replace("bfloat16", "bf16").replace("float16", "fp16"),
            "data": "synthetic",
            "config": {**workload_config(args, wl, world),
                       "workspace_bytes": prob_wsb,
                       "workspace": "spill modes: the tiles of all heads, one chunk; the Python API (e2e) "
                                    "takes fa2_bwd_workspace_bytes' recommendation, chunks of 2048 tiles"},
            "per_gpu_tflops": value / world,
            "frac_of_peak": {"burst": value / world / peaks["bf16"],
                             "sustained": value / world / peaks["bf16_sustained"],
                             "nominal_2250": value / world / 2250.0, "source": peaks["source"]},
            "clocks": clocks.summary(),
            "sustained": sustained,
            "strong": strong,
            "gpu_launches": launches_per_step * args.steps,
            "roofline": roofline,
            "e2e": e2e,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(b, h, n, d, dtype, qk_mul, scale_opt)
        if world == 1 and not args.no_triton_reference and args.workload in ("c2", "c3"):
            line["triton_reference"] = triton_reference(args.workload, ms_per_step)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
