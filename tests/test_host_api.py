"""Host-side mirror of the reference interface: names, defaults, config shim, partitioning."""

from __future__ import annotations

import inspect
import os
import subprocess
import sys
import textwrap

import pytest
import torch

import flash_attention_triton_b200 as fa
from conftest import ROOT
from flash_attention_triton_b200 import shard_range, shard_slab


def test_public_names_match_reference_package():
    # the reference exports exactly these four (src/flash_attention_triton/__init__.py:13)
    for name in ("KernelsConfigV2", "flash_attention_v2", "flash_attention_v2_custom", "init_to_zero_v2"):
        assert hasattr(fa, name)


def test_flash_attention_v2_signature():
    sig = inspect.signature(fa.flash_attention_v2)
    assert list(sig.parameters) == ["q", "k", "v", "softmax_scale", "deterministic"]
    assert sig.parameters["softmax_scale"].default is None
    assert sig.parameters["deterministic"].default is False
    sig = inspect.signature(fa.flash_attention_v2_custom)
    assert list(sig.parameters) == ["q", "k", "v", "softmax_scale", "kernels_configs"]


def test_cpu_tensors_are_rejected_like_the_reference():
    q = torch.randn(1, 1, 16, 32)
    with pytest.raises(AssertionError, match="CUDA"):
        fa.flash_attention_v2(q, q, q)


class _Cfg:
    def __init__(self, **kw):
        self.kwargs = kw


def test_config_shim_maps_sequence_parallel_to_determinism():
    mk = lambda seqpar: fa.KernelsConfigV2(128, 128, 32, 256, 32, 8, 16, 1, [
        _Cfg(BLOCK_Q_ROWS_SIZE=64, BLOCK_KV_COLS_SIZE=64, SEQUENCE_PARALLEL=seqpar)])
    assert mk(False).is_deterministic() is True
    assert mk(True).is_deterministic() is False
    with pytest.raises(Exception):
        mk(True).block_rows_size = 1  # frozen, like the reference dataclass


def test_init_to_zero_v2_zeroes_named_tensor():
    t = torch.ones(4)
    out = fa.init_to_zero_v2("DQ")({"DQ": t})
    assert out is t and torch.equal(t, torch.zeros(4))


@pytest.mark.parametrize("n,world", [(64, 1), (64, 2), (64, 8), (16, 8), (10, 4), (3, 8), (0, 2)])
def test_shard_ranges_partition_the_batch_head_axis(n, world):
    ranges = [shard_range(n, world, r) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == n
    for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
        assert a1 == b0
    sizes = [b - a for a, b in ranges]
    assert max(sizes) - min(sizes) <= 1


def test_shard_range_rejects_bad_rank():
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)
    with pytest.raises(ValueError):
        shard_range(8, 0, 0)


def test_shard_slab_is_a_view_of_contiguous_heads():
    t = torch.arange(2 * 4 * 3 * 2, dtype=torch.float32).view(2, 4, 3, 2)
    parts = [shard_slab(t, 4, r) for r in range(4)]
    assert all(p.shape == (1, 2, 3, 2) for p in parts)
    torch.testing.assert_close(torch.cat(parts, dim=1).view(2, 4, 3, 2), t)


GLOO_WORKER = textwrap.dedent(
    """
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, os.environ["FA2_ROOT"])
    from flash_attention_triton_b200 import shard_slab, shard_range
    from oracle.attention_oracle import naive_attention
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    g = torch.Generator().manual_seed(0)
    q, k, v, do = (torch.randn(2, 3, 40, 16, generator=g) for _ in range(4))
    mine = [shard_slab(t, world, rank) for t in (q, k, v, do)]
    r = naive_attention(*mine, dtype=torch.float32)
    # gather the per-rank slabs on rank 0 and compare with the unsharded computation
    for key in ("o", "dq", "dk", "dv"):
        parts = [None] * world
        dist.all_gather_object(parts, r[key])
        if rank == 0:
            full = naive_attention(q, k, v, do, dtype=torch.float32)[key].reshape(1, 6, 40, 16)
            assert torch.equal(torch.cat(parts, dim=1), full), key
    dist.barrier()
    dist.destroy_process_group()
    """
)


def test_two_ranks_cover_the_problem_without_a_collective_on_the_data_path(tmp_path):
    """world_size-2 gloo run: each rank computes its own (batch, head) slab with the oracle;
    the concatenation equals the unsharded result bit for bit."""
    script = tmp_path / "worker.py"
    script.write_text(GLOO_WORKER)
    env = dict(os.environ, FA2_ROOT=str(ROOT), OMP_NUM_THREADS="2")
    res = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
         "--master-addr", "127.0.0.1", "--master-port", "29511", str(script)],
        env=env, capture_output=True, text=True, timeout=240,
    )
    assert res.returncode == 0, res.stderr[-2000:]
