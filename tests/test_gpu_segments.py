"""Segment-aware block skipping: blocks whose q and kv segment ids cannot meet are left
out, blocks with one id on both sides are not compared element by element.  Results must
not change: with the scratch for it withheld (SPLASH_SEG_SKIP=0) the kernels compute every
scheduled block, and both ways must give the same bits; the oracle bounds both.
"""

import numpy as np
import pytest
import torch

import splash_attention_mgpu as sa
from oracle import dense_attention as oracle

from common import inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ids(kind, batch, s, seed):
  rng = np.random.default_rng(seed)
  ids = np.zeros((batch, s), np.int32)
  for b in range(batch):
    if kind == "packed":      # documents of 100..900 tokens, ids increasing
      pos, seg = 0, 0
      while pos < s:
        n = int(rng.integers(100, 901))
        ids[b, pos:pos + n] = seg
        pos += n
        seg += 1
    elif kind == "aligned":   # boundaries on block edges: whole blocks are skipped or uniform
      ids[b] = np.repeat(rng.permutation(s // 256), 256)
    else:                     # arbitrary ids: the range test is only conservative
      ids[b] = rng.integers(0, 3, size=s)
  return ids


def _run(kernel, q, k, v, do, seg, monkeypatch, skip):
  monkeypatch.setenv("SPLASH_SEG_SKIP", "1" if skip else "0")
  qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))
  out = kernel(qg, kg, vg, seg)
  out.backward(do)
  torch.cuda.synchronize()
  sa.check_device_status()
  return out.detach(), qg.grad, kg.grad, vg.grad


@pytest.mark.parametrize("kind", ["packed", "aligned", "random"])
@pytest.mark.parametrize("d,h,kvh,mask_name,bs", [
    (128, 2, 2, "causal", sa.BlockSizes()),
    (128, 4, 2, "full", sa.BlockSizes(block_q=128, block_kv=64)),
    (64, 2, 2, "full", sa.BlockSizes()),
    (64, 4, 1, "causal", sa.BlockSizes(block_q=256)),
])
@pytest.mark.parametrize("fused", [True, False])
def test_skipping_changes_nothing(kind, d, h, kvh, mask_name, bs, fused, monkeypatch):
  # fused=False: the dQ kernel and the dK/dV kernel of the split backward, each with its own list.
  monkeypatch.setenv("SPLASH_BWD_FUSED", "1" if fused else "0")
  s, batch = 2048, 2
  mask = sa.CausalMask((s, s)) if mask_name == "causal" else sa.FullMask((s, s))
  kernel = sa.make_splash_mha(mask, block_sizes=bs)
  q, k, v = inputs(batch, h, kvh, s, d, d, torch.bfloat16, False, seed=4, device=DEV, scale=d ** -0.5)
  do = torch.randn(q.shape, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16).to(DEV)
  ids = _ids(kind, batch, s, seed=3)
  t = torch.from_numpy(ids).to(DEV)
  seg = sa.SegmentIds(t, t)
  with_skip = _run(kernel, q, k, v, do, seg, monkeypatch, True)
  without = _run(kernel, q, k, v, do, seg, monkeypatch, False)
  for name, a, b in zip(("out", "dq", "dk", "dv"), with_skip, without):
    if name == "dq" and fused:
      # The fused backward accumulates dQ with f32 reduce-adds whose order is not fixed.
      np.testing.assert_allclose(a.float().cpu().numpy(), b.float().cpu().numpy(), atol=2e-3, rtol=2e-2, err_msg=name)
    else:
      assert torch.equal(a, b), name
  dense = np.asarray(mask[:, :])[None]
  ref_out, _ = oracle.attention_forward(dense, q, k, v, (ids, ids))
  ref = oracle.attention_backward(dense, q, k, v, do, (ids, ids))
  np.testing.assert_allclose(with_skip[0].float().cpu().numpy(), ref_out, atol=2e-2, rtol=2e-2)
  for name, g, r in zip("qkv", with_skip[1:], ref):
    g = g.float().cpu().numpy()
    assert np.abs(g - r).max() / np.abs(r).max() < 2e-2, name


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("d,bs", [(128, sa.BlockSizes()), (64, sa.BlockSizes()), (128, sa.BlockSizes(block_q=256))])
def test_q_blocks_whose_every_step_is_skipped(d, bs, fused, monkeypatch):
  """q rows whose segment id no key carries: every scheduled step of their CTAs is skipped.
  They return zeros with lse = mask_value and take no part in the gradients; KV blocks that
  no surviving q row looks at get zero dK/dV."""
  s, h = 1024, 2
  kernel = sa.make_splash_mha(sa.FullMask((s, s)), block_sizes=bs)
  q, k, v = inputs(1, h, h, s, d, d, torch.bfloat16, False, seed=6, device=DEV, scale=d ** -0.5)
  do = torch.randn(q.shape, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(DEV)
  seg_q = np.zeros((1, s), np.int32)
  seg_q[:, s // 2:] = 7                      # no key has id 7
  seg_kv = np.zeros((1, s), np.int32)
  seg_kv[:, 3 * s // 4:] = 9                 # keys no q row can see
  seg = sa.SegmentIds(torch.from_numpy(seg_q).to(DEV), torch.from_numpy(seg_kv).to(DEV))
  monkeypatch.setenv("SPLASH_SEG_SKIP", "1")
  monkeypatch.setenv("SPLASH_BWD_FUSED", "1" if fused else "0")
  out, (lse,) = kernel(q, k, v, seg, save_residuals=True)
  qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))
  kernel(qg, kg, vg, seg).backward(do)
  torch.cuda.synchronize()
  sa.check_device_status()
  assert torch.all(out[:, :, s // 2:] == 0)
  assert torch.all(lse[:, :, s // 2:] == kernel.mask_value)
  assert torch.all(qg.grad[:, :, s // 2:] == 0)
  assert torch.all(kg.grad[:, :, 3 * s // 4:] == 0) and torch.all(vg.grad[:, :, 3 * s // 4:] == 0)
  dense = np.ones((1, s, s), bool)
  ref_out, ref_lse = oracle.attention_forward(dense, q, k, v, (seg_q, seg_kv))
  ref = oracle.attention_backward(dense, q, k, v, do, (seg_q, seg_kv))
  live = slice(0, s // 2)
  np.testing.assert_allclose(out[0, :, live].float().cpu().numpy(), ref_out[0, :, live], atol=2e-2, rtol=2e-2)
  np.testing.assert_allclose(lse[0, :, live].cpu().numpy(), ref_lse[0, :, live], atol=1e-3, rtol=1e-3)
  # The oracle spreads rows that see nothing uniformly over all keys; those rows are implementation-defined
  # (reference tools/fuzz.py:116-124), so gradients are compared where only live rows contribute.
  got_dq = qg.grad[0, :, live].float().cpu().numpy()
  assert np.abs(got_dq - ref[0][0, :, live]).max() / np.abs(ref[0][0, :, live]).max() < 2e-2
