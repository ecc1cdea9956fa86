"""Multi-GPU partition logic on CPU ranks (gloo, world_size 2 and 3): every rank runs
its (batch x kv-head) units, the gathered result equals the unsharded one.  The compute
stand-in is the CPU oracle; the partition, unit views and gather are the product code."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from splash_attention_mgpu import sharding

from common import build_mask, inputs, segments


def test_unit_ranges_cover_everything_once():
  for units in (1, 2, 7, 8, 32, 33):
    for world in (1, 2, 3, 4, 8):
      spans = [sharding.unit_range(units, world, r) for r in range(world)]
      assert spans[0][0] == 0 and spans[-1][1] == units
      assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
      sizes = [hi - lo for lo, hi in spans]
      assert max(sizes) - min(sizes) <= 1


def _free_port():
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def _worker(rank, world, port, case, results):
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  dist.init_process_group("gloo", rank=rank, world_size=world)
  try:
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import dense_attention as oracle
    b, h, kvh, s, d = case["b"], case["h"], case["kvh"], 256, 64
    _, dense = build_mask("causal", s, h, False)
    q, k, v = inputs(b, h, kvh, s, d, d, torch.float32, False, seed=3, scale=0.2)
    seg = segments(s) if case.get("seg") else None

    def fn(qu, ku, vu, sg=None):
      out, _ = oracle.attention_forward(dense, qu, ku, vu, sg)
      return torch.from_numpy(out)

    local, span = sharding.run_local(fn, q, k, v, seg, world=world, rank=rank)
    full = sharding.gather_units(local, span, (b, h, s, d))
    want, _ = oracle.attention_forward(dense, q, k, v, seg)
    results[rank] = float(np.abs(full.numpy() - want).max())
  finally:
    dist.destroy_process_group()


@pytest.mark.parametrize("case", [dict(b=2, h=4, kvh=2, world=2), dict(b=1, h=4, kvh=4, world=3, seg=True),
                                  dict(b=1, h=2, kvh=1, world=2)],
                         ids=lambda c: ",".join(f"{k}={v}" for k, v in c.items()))
def test_sharded_run_matches_unsharded(case):
  world = case["world"]
  port = _free_port()
  with mp.Manager() as manager:
    results = manager.dict()
    mp.spawn(_worker, args=(world, port, case, results), nprocs=world, join=True)
    assert len(results) == world
    assert max(results.values()) < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_gpu_sharded_forward_backward_equals_unsharded(world):
  """Every rank's slice run with the real kernels on one GPU, one after the other: outputs, dK and
  dV equal the unsharded call bit for bit (units never interact); dQ is accumulated by f32
  reduce-adds whose order is not fixed, so it is compared to rounding."""
  import splash_attention_mgpu as sa
  dev = "cuda:0"
  b, h, kvh, s, d = 2, 4, 2, 1024, 128
  q, k, v = (x.to(dev) for x in inputs(b, h, kvh, s, d, d, torch.bfloat16, False, seed=5, scale=0.3))
  do = torch.randn(q.shape, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).to(dev)
  kernel = sa.make_splash_mha(sa.CausalMask((s, s)))
  qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))
  out = kernel(qg, kg, vg)
  out.backward(do)
  want = [sharding.to_units(t, k, v)[0] for t in (out.detach(), qg.grad)] + \
         [kg.grad.reshape(b * kvh, 1, s, d), vg.grad.reshape(b * kvh, 1, s, d)]
  for rank in range(world):
    (o, dq, dk, dv), (lo, hi) = sharding.run_local_grads(kernel, q, k, v, do, world=world, rank=rank)
    sa.check_device_status()
    assert torch.equal(o, want[0][lo:hi])
    assert torch.equal(dk, want[2][lo:hi]) and torch.equal(dv, want[3][lo:hi])
    np.testing.assert_allclose(dq.float().cpu().numpy(), want[1][lo:hi].float().cpu().numpy(), atol=2e-3, rtol=2e-2)
