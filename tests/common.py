"""Shared fixtures of the test-suite: mask zoo, seeded inputs, comparison rules.

The mask zoo, case lists and tolerances follow the reference's own tests
(tests/test_splash_attention_mgpu.py:51-125, 350-394); inputs come from a seeded
torch generator (the reference draws from jax.random, which cannot be
reproduced here).
"""

import numpy as np
import torch

import splash_attention_mgpu as sa
from oracle import dense_attention as oracle


def masks(s, seed=0):
  rng = np.random.default_rng(seed)
  dense = np.tril(np.ones((s, s), bool)) & (rng.random((s, s)) > 0.3)
  dense |= np.eye(s, dtype=bool)  # every row attends to something
  return {
      "full": sa.FullMask((s, s)),
      "causal": sa.CausalMask((s, s)),
      "local": sa.LocalMask((s, s), (100, 20), 0),
      "chunked": sa.ChunkedCausalMask((s, s), chunk_size=192),
      "dense": sa.NumpyMask(dense),
  }


def build_mask(mask_name, s, h, multi_head_mask):
  zoo = masks(s)
  if multi_head_mask:
    names = list(zoo)
    heads = [zoo[names[(names.index(mask_name) + i) % len(names)]] for i in range(h)]
    return sa.MultiHeadMask(heads), np.stack([np.asarray(m[:, :]) for m in heads])
  mask = zoo[mask_name]
  return mask, np.asarray(mask[:, :])[None]


def inputs(b, h, kvh, s, d, dv, dtype, mqa, seed=0, device="cpu", scale=1.0):
  g = torch.Generator().manual_seed(seed)
  lead = (b,) if b else ()
  kv_lead = lead + (() if mqa else (kvh,))
  q = (torch.randn(lead + (h, s, d), generator=g) * scale).to(dtype)
  k = torch.randn(kv_lead + (s, d), generator=g).to(dtype)
  v = torch.randn(kv_lead + (s, dv), generator=g).to(dtype)
  return q.to(device), k.to(device), v.to(device)


def segments(s, device="cpu"):
  ids = torch.from_numpy(np.repeat(np.arange(4), s // 4).astype(np.int32)).to(device)
  return sa.SegmentIds(ids, ids)


def tolerance(dtype):
  return 2e-2 if dtype == torch.bfloat16 else 5e-3


def assert_forward_close(out, lse, ref_out, ref_lse, dtype):
  """out/ref: max|d| <= tol (atol = rtol = 2e-2 bf16, 5e-3 f16) and mean relative
  error <= 5e-3; lse within 1e-3."""
  tol = tolerance(dtype)
  out = out.detach().float().cpu().numpy()
  np.testing.assert_allclose(out, ref_out, atol=tol, rtol=tol)
  denom = np.abs(ref_out).mean()
  assert np.abs(out - ref_out).mean() / max(denom, 1e-30) <= 5e-3
  if lse is not None:
    np.testing.assert_allclose(lse.detach().cpu().numpy(), ref_lse, atol=1e-3, rtol=1e-3)
