"""The benchmark configurations at their full sizes, checked through quantities that
stay cheap at any size: a sample of q rows against the CPU oracle (a row of the output,
of lse and of dQ depends only on that row of q), one whole (batch, kv-head) unit against
the oracle for dK/dV, and bit-identical results when the same unit is run on its own.
"""

import numpy as np
import pytest
import torch

import splash_attention_mgpu as sa
from oracle import dense_attention as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rand(shape, dtype, seed, scale=1.0):
  g = torch.Generator().manual_seed(seed)
  return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def _check_rows(dense_rows_fn, q, k, v, out, lse, rows, heads, *, seg=None, cap=None, mqa=False, dtype, b=0,
                dq=None, d_out=None):
  """Oracle on `rows` of q for the listed heads of batch element b."""
  tol = 2e-2 if dtype == torch.bfloat16 else 5e-3
  for h in heads:
    kvh = 0 if mqa else h // (q.shape[1] // k.shape[1])
    qs = q[b, h:h + 1, rows]
    ks = (k[b] if mqa else k[b, kvh:kvh + 1])
    vs = (v[b] if mqa else v[b, kvh:kvh + 1])
    mask_rows = dense_rows_fn(h, rows)[None]
    sg = None if seg is None else (seg[0][b, rows].cpu().numpy(), seg[1][b].cpu().numpy())
    ref, ref_lse = oracle.attention_forward(mask_rows, qs, ks[None] if mqa else ks, vs[None] if mqa else vs, sg,
                                            attn_logits_soft_cap=cap)
    got_out = out[b, h, rows].float().cpu().numpy()
    np.testing.assert_allclose(got_out, ref[0], atol=tol, rtol=tol)
    assert np.abs(got_out - ref[0]).mean() / np.abs(ref[0]).mean() <= 5e-3, "out: mean relative error"
    np.testing.assert_allclose(lse[b, h, rows].cpu().numpy(), ref_lse[0], atol=1e-3, rtol=1e-3)
    if dq is not None:
      want_dq, _, _ = oracle.attention_backward(mask_rows, qs, ks, vs, d_out[b, h:h + 1, rows], sg,
                                                attn_logits_soft_cap=cap)
      got = dq[b, h, rows].float().cpu().numpy()
      assert np.abs(got - want_dq[0]).max() / np.abs(want_dq).max() < 2e-2
      mean_rel = np.abs(got - want_dq[0]).mean() / np.abs(want_dq[0]).mean()
      assert mean_rel <= 5e-3, f"dq: mean relative error {mean_rel}"


def _grads(kernel, q, k, v, d_out, seg=None):
  qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))
  out = kernel(qg, kg, vg, seg)
  out.backward(d_out)
  sa.check_device_status()
  return out.detach(), qg.grad, kg.grad, vg.grad


def _check_unit(dense, q, k, v, d_out, dk, dv, b, kvh, *, seg=None, cap=None):
  """dK/dV of one (batch, kv head) unit against the oracle (needs every q row of its group)."""
  group = q.shape[1] // k.shape[1]
  hs = slice(kvh * group, (kvh + 1) * group)
  sg = None if seg is None else (seg[0][b].cpu().numpy(), seg[1][b].cpu().numpy())
  mask = dense if dense.shape[0] == 1 else dense[hs]
  _, want_dk, want_dv = oracle.attention_backward(mask, q[b, hs], k[b, kvh:kvh + 1], v[b, kvh:kvh + 1], d_out[b, hs],
                                                  sg, attn_logits_soft_cap=cap)
  for name, got, want in (("dk", dk[b, kvh], want_dk[0]), ("dv", dv[b, kvh], want_dv[0])):
    got = got.float().cpu().numpy()
    assert np.abs(got - want).max() / np.abs(want).max() < 2e-2
    mean_rel = np.abs(got - want).mean() / np.abs(want).mean()
    assert mean_rel <= 5e-3, f"{name}: mean relative error {mean_rel}"


def test_causal_b2_h16_s8192_d128_forward_backward():
  s, d, dtype = 8192, 128, torch.bfloat16
  q = _rand((2, 16, s, d), dtype, 0, d ** -0.5)
  k, v, do = _rand((2, 16, s, d), dtype, 1), _rand((2, 16, s, d), dtype, 2), _rand((2, 16, s, d), dtype, 3)
  rows = np.sort(np.random.default_rng(0).choice(s, 192, replace=False))
  dense_rows = lambda h, r: (np.arange(s)[None, :] <= r[:, None])
  # The two-tile ping-pong kernel, then the one-tile kernel (the automatic choice here).
  for bq in (256, 128):
    kernel = sa.make_splash_mha(sa.CausalMask((s, s)), block_sizes=sa.BlockSizes(block_q=bq))
    out, (lse,) = kernel(q, k, v, save_residuals=True)
    sa.check_device_status()
    _check_rows(dense_rows, q, k, v, out, lse, rows, heads=[0, 7, 15], dtype=dtype, b=1)
  kernel = sa.make_splash_mha(sa.CausalMask((s, s)))
  assert kernel.resolved_block_sizes(d, d).block_q == 128
  out2, dq, dk, dv = _grads(kernel, q, k, v, do)
  assert torch.equal(out2, out)
  _check_rows(dense_rows, q, k, v, out, lse, rows, heads=[3], dtype=dtype, b=0, dq=dq, d_out=do)
  _check_unit(np.tril(np.ones((s, s), bool))[None], q, k, v, do, dk, dv, b=1, kvh=5)
  # The same unit on its own gives the same bits (units never interact).
  _, dq1, dk1, dv1 = _grads(kernel, q[1:2, 5:6], k[1:2, 5:6], v[1:2, 5:6], do[1:2, 5:6])
  assert torch.equal(dk1[0, 0], dk[1, 5]) and torch.equal(dv1[0, 0], dv[1, 5])
  np.testing.assert_allclose(dq1[0, 0].float().cpu().numpy(), dq[1, 5].float().cpu().numpy(), atol=2e-3, rtol=2e-2)


def test_local_window_gqa_softcap_s16384_forward_backward():
  s, d, dtype, cap = 16384, 128, torch.bfloat16, 50.0
  q = _rand((1, 32, s, d), dtype, 0, d ** -0.5)
  k, v, do = _rand((1, 8, s, d), dtype, 1), _rand((1, 8, s, d), dtype, 2), _rand((1, 32, s, d), dtype, 3)
  mask = sa.LocalMask((s, s), (1024, 0), 0)
  kernel = sa.make_splash_mha(mask, attn_logits_soft_cap=cap)
  bs = kernel.resolved_block_sizes(d, d)
  assert (bs.block_q, bs.block_kv, bs.num_stages) == (128, 64, 2)
  out, (lse,) = kernel(q, k, v, save_residuals=True)
  sa.check_device_status()
  rows = np.sort(np.random.default_rng(1).choice(s, 192, replace=False))
  dense_rows = lambda h, r: np.asarray(mask[r, :])
  _, dq, dk, dv = _grads(kernel, q, k, v, do)
  _check_rows(dense_rows, q, k, v, out, lse, rows, heads=[0, 13, 31], cap=cap, dtype=dtype, dq=dq, d_out=do)
  _check_unit(np.asarray(mask[:, :])[None], q, k, v, do, dk, dv, b=0, kvh=3, cap=cap)


def _packed_segments(batch, s, seed):
  rng = np.random.default_rng(seed)
  ids = np.zeros((batch, s), np.int32)
  for b in range(batch):
    pos, seg = 0, 0
    while pos < s:
      n = int(rng.integers(256, 4097))
      ids[b, pos:pos + n] = seg
      pos += n
      seg += 1
  return ids


@pytest.mark.parametrize("variant", ["full", "per_head"])
def test_packed_documents_f16_d64_forward_backward(variant):
  s, d, dtype, batch, heads = 8192, 64, torch.float16, 4, 16
  q = _rand((batch, heads, s, d), dtype, 0, d ** -0.5)
  k, v = _rand((batch, heads, s, d), dtype, 1), _rand((batch, heads, s, d), dtype, 2)
  do = _rand((batch, heads, s, d), dtype, 3)
  ids = torch.from_numpy(_packed_segments(batch, s, 7)).to(DEV)
  seg = sa.SegmentIds(ids, ids)
  if variant == "full":
    masks = [sa.FullMask((s, s))] * heads
    kernel = sa.make_splash_mha(masks[0])
  else:
    masks = [sa.CausalMask((s, s)) if h % 2 == 0 else sa.ChunkedCausalMask((s, s), chunk_size=1024)
             for h in range(heads)]
    kernel = sa.make_splash_mha(sa.MultiHeadMask(masks))
    assert kernel.info.num_steps.shape[0] == heads and kernel.info.partial_mask_blocks is None
  bs = kernel.resolved_block_sizes(d, d, has_segments=True)
  assert (bs.block_q, bs.block_kv, bs.num_stages) == (128, 64, 2)
  out, (lse,) = kernel(q, k, v, seg, save_residuals=True)
  sa.check_device_status()
  rows = np.sort(np.random.default_rng(2).choice(s, 160, replace=False))
  dense_rows = lambda h, r: np.asarray(masks[h][r, :])
  _, dq, dk, dv = _grads(kernel, q, k, v, do, seg)
  _check_rows(dense_rows, q, k, v, out, lse, rows, heads=[0, 5], seg=seg, dtype=dtype, b=2, dq=dq, d_out=do)
  dense = np.stack([np.asarray(masks[h][:, :]) for h in (6, 7)])
  for h, m in zip((6, 7), dense):
    _check_unit(m[None], q, k, v, do, dk, dv, b=3, kvh=h, seg=seg)


def test_mqa_block_sparse_numpy_mask_s32768_d256_forward():
  s, d, heads, dtype = 32768, 256, 64, torch.bfloat16
  rng = np.random.default_rng(5)
  kinds = rng.choice(3, size=(s // 128, s // 64), p=[0.70, 0.10, 0.20])  # 0 empty, 1 partial, 2 full
  dense = np.zeros((s, s), bool)
  for i, j in zip(*np.nonzero(kinds == 2)):
    dense[i * 128:(i + 1) * 128, j * 64:(j + 1) * 64] = True
  for i, j in zip(*np.nonzero(kinds == 1)):
    dense[i * 128:(i + 1) * 128, j * 64:(j + 1) * 64] = rng.random((128, 64)) < 0.5
  dense[np.arange(s), np.arange(s)] = True  # no empty row
  kernel = sa.make_splash_mqa(sa.NumpyMask(dense), block_sizes=sa.BlockSizes(block_q=128, block_kv=64))
  info = kernel.fwd_info(128, 64)
  assert 0.25 < info.density < 0.36 and info.partial_mask_blocks is not None
  q = _rand((heads, s, d), dtype, 0, 1 / 16)
  k, v = _rand((s, d), dtype, 1), _rand((s, d), dtype, 2)
  out, (lse,) = kernel(q, k, v, save_residuals=True)
  sa.check_device_status()
  assert out.shape == (heads, s, d) and lse.shape == (heads, s)
  rows = np.sort(rng.choice(s, 128, replace=False))
  for h in (0, 31, 63):
    ref, ref_lse = oracle.attention_forward(dense[rows][None], q[h:h + 1, rows], k[None], v[None])
    np.testing.assert_allclose(out[h, rows].float().cpu().numpy(), ref[0], atol=2e-2, rtol=2e-2)
    np.testing.assert_allclose(lse[h, rows].cpu().numpy(), ref_lse[0], atol=1e-3, rtol=1e-3)
  # Every head sees the same K/V and mask: heads with equal q rows must agree bit for bit.
  q2 = q.clone()
  q2[1] = q2[0]
  out2 = kernel(q2, k, v)
  assert torch.equal(out2[0], out2[1]) and torch.equal(out2[0], out[0])
