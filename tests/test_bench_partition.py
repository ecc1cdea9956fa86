"""bench.py's partition of a workload over ranks, on the CPU: every unit is owned by exactly
one rank, the ranks' useful FLOPs add up to the workload's, the local problem shapes are
what the kernels take, and a unit's synthetic data does not depend on the world size."""

import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402
import splash_attention_mgpu as sa  # noqa: E402

SMALL = {
    "shared": bench.Workload("causal", 2, 8, 4, 512, 64, "bf16"),
    "per_head": bench.Workload("packed_per_head", 2, 4, 4, 1024, 64, "f16", segments=True),
    "mqa_fwd": bench.Workload("full", 1, 8, 1, 256, 64, "bf16", mqa=True, forward_only=True),
}


@pytest.mark.parametrize("name", sorted(SMALL))
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_units_and_flops_add_up(name, world):
  wl = SMALL[name]
  parts = [bench.Partition(sa, wl, world, r) for r in range(world)]
  spans = [p.span for p in parts]
  assert spans[0][0] == 0 and spans[-1][1] == parts[0].num_units
  assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
  total_fwd, total_fb = parts[0].total_flops()
  assert abs(sum(p.flops()[0] for p in parts) - total_fwd) <= 1e-9 * total_fwd
  assert total_fb == (total_fwd if wl.forward_only else 3.5 * total_fwd)
  for p in parts:
    n = p.span[1] - p.span[0]
    q, k, v, do = p.host_inputs(pin=False)
    assert tuple(q.shape) == tuple(p.q_shape) and tuple(k.shape) == tuple(p.kv_shape) and do.shape == q.shape
    if n:
      assert q.shape[-2:] == (wl.seq, wl.head_dim)


def test_unit_data_is_independent_of_the_world_size():
  wl = SMALL["shared"]
  whole = bench.Partition(sa, wl, 1, 0).host_inputs(pin=False)
  for world in (2, 4):
    for r in range(world):
      p = bench.Partition(sa, wl, world, r)
      lo, hi = p.span
      for mine, full in zip(p.host_inputs(pin=False), whole):
        assert torch.equal(mine, full[lo:hi])


def test_reference_accounting_of_the_headline_workload():
  wl = bench.WORKLOADS[bench.DEFAULT_WORKLOAD]
  p = bench.Partition(sa, wl, 8, 3)
  fwd, fb = p.total_flops()
  # 2080 visible 128 x 128 blocks per head, 32 (batch, head) units (reference tools/bench.py:86-102).
  assert fwd == 4.0 * 2080 * 32 * 128 * 128 * 128 and fb == 3.5 * fwd
  assert p.span == (12, 16) and p.q_shape == (4, 1, 8192, 128)
  assert bench.base_config(bench.DEFAULT_WORKLOAD, 8)["workload"] == bench.DEFAULT_WORKLOAD
