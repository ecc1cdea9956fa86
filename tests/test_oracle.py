"""The CPU oracle against independent implementations, and the schedule emulator
against the oracle (the CPU-runnable plumbing case: causal MHA, batch 1, 2 heads,
seq 512, head_dim 64, bf16, 128x128 blocks)."""

import numpy as np
import pytest
import torch

import splash_attention_mgpu as sa
from oracle import dense_attention as oracle
from oracle import schedule_emulator as emu

from common import build_mask, inputs, masks, segments


@pytest.mark.parametrize("name", ["full", "causal", "local", "chunked", "dense"])
def test_oracle_forward_matches_torch_sdpa(name):
  s, h, d = 256, 2, 64
  mask, dense = build_mask(name, s, h, False)
  q, k, v = inputs(None, h, h, s, d, d, torch.float32, False, scale=0.2)
  out, lse = oracle.attention_forward(dense, q, k, v)
  ref = torch.nn.functional.scaled_dot_product_attention(
      q[None], k[None], v[None], attn_mask=torch.from_numpy(dense)[None], scale=1.0)[0]
  np.testing.assert_allclose(out, ref.numpy(), atol=2e-5, rtol=2e-5)
  logits = torch.einsum("hqd,hkd->hqk", q, k).masked_fill(~torch.from_numpy(dense), -torch.inf)
  np.testing.assert_allclose(lse, torch.logsumexp(logits, -1).numpy(), atol=1e-4, rtol=1e-5)


@pytest.mark.parametrize("kw", [dict(), dict(cap=5.0), dict(seg=True), dict(kvh=1), dict(mqa=True),
                                dict(b=2, seg=True)])
def test_oracle_backward_matches_autograd(kw):
  s, h, d = 256, 2, 64
  kvh = kw.get("kvh", h)
  mqa = kw.get("mqa", False)
  b = kw.get("b")
  mask, dense = build_mask("causal", s, h, False)
  q, k, v = inputs(b, h, 1 if mqa else kvh, s, d, d, torch.float64, mqa, scale=0.3)
  seg = segments(s) if kw.get("seg") else None
  cap = kw.get("cap")
  w = torch.randn(q.shape, generator=torch.Generator().manual_seed(7), dtype=torch.float64)
  qg, kg, vg = (x.clone().requires_grad_(True) for x in (q, k, v))
  out = sa.attention_reference(dense, qg, kg, vg, seg, is_mqa=mqa, attn_logits_soft_cap=cap)
  (out.double() * w).sum().backward()
  dq, dk, dv = oracle.attention_backward(dense, q, k, v, w, seg, is_mqa=mqa, attn_logits_soft_cap=cap)
  for got, want in ((dq, qg.grad), (dk, kg.grad), (dv, vg.grad)):
    np.testing.assert_allclose(got, want.float().numpy(), atol=2e-4, rtol=2e-4)


def test_package_reference_matches_oracle():
  s, h, d = 256, 3, 64
  mask, dense = build_mask("causal", s, h, True)
  q, k, v = inputs(2, h, h, s, d, d, torch.float32, False, scale=0.2)
  seg = segments(s)
  out, (lse,) = sa.attention_reference(dense, q, k, v, seg, attn_logits_soft_cap=3.0, save_residuals=True)
  ref, ref_lse = oracle.attention_forward(dense, q, k, v, seg, attn_logits_soft_cap=3.0)
  np.testing.assert_allclose(out.numpy(), ref, atol=1e-5, rtol=1e-5)
  np.testing.assert_allclose(lse.numpy(), ref_lse, atol=1e-5, rtol=1e-5)


EMULATOR_CASES = [
    dict(mask_name="causal"),  # the CPU-runnable plumbing configuration
    dict(mask_name="full"), dict(mask_name="local"), dict(mask_name="chunked"), dict(mask_name="dense"),
    dict(mask_name="causal", seg=True), dict(mask_name="dense", seg=True),
    dict(mask_name="causal", cap=5.0), dict(mask_name="causal", h=4, kvh=2),
    dict(mask_name="causal", bkv=64), dict(mask_name="dense", bq=256, bkv=64),
    dict(mask_name="causal", multi=True, h=3), dict(mask_name="local", bq=256),
]


@pytest.mark.parametrize("kw", EMULATOR_CASES, ids=lambda kw: ",".join(f"{k}={v}" for k, v in kw.items()))
def test_schedule_emulator_matches_oracle(kw):
  s, d = 512, 64
  h, kvh = kw.get("h", 2), kw.get("kvh") or kw.get("h", 2)
  mask, dense = build_mask(kw["mask_name"], s, h, kw.get("multi", False))
  info = sa.process_mask(mask, (kw.get("bq", 128), kw.get("bkv", 128)))
  q, k, v = inputs(None, h, kvh, s, d, d, torch.bfloat16, False, scale=d ** -0.5)
  seg = segments(s) if kw.get("seg") else None
  cap = kw.get("cap")
  out, lse = emu.emulate_forward(info, q, k, v, seg, mask_value=sa.DEFAULT_MASK_VALUE,
                                 attn_logits_soft_cap=cap)
  ref, ref_lse = oracle.attention_forward(dense, q, k, v, seg, attn_logits_soft_cap=cap)
  np.testing.assert_allclose(out, ref, atol=2e-2, rtol=2e-2)
  np.testing.assert_allclose(lse, ref_lse, atol=1e-3, rtol=1e-3)


def test_emulator_empty_rows():
  s = 256
  dense = np.zeros((s, s), bool)
  dense[128:, :] = True
  info = sa.process_mask(sa.NumpyMask(dense), (128, 128))
  q, k, v = inputs(None, 1, 1, s, 64, 64, torch.bfloat16, False)
  out, lse = emu.emulate_forward(info, q, k, v, mask_value=sa.DEFAULT_MASK_VALUE)
  assert np.all(out[:, :128] == 0) and np.all(lse[:, :128] == np.float32(sa.DEFAULT_MASK_VALUE))


@pytest.mark.parametrize("growth", [0.0, 0.05, 40.0])
def test_emulator_lazy_rescaling(growth):
  # Logit maxima that grow along the KV axis force rescaling on later blocks; tiny
  # growth stays under the threshold (reference tests/...:319-342).
  s, d = 1024, 64
  info = sa.process_mask(sa.CausalMask((s, s)), (128, 128))
  q, k, v = inputs(None, 2, 2, s, d, d, torch.bfloat16, False)
  pos = torch.arange(s, dtype=torch.float32)[None, :, None] / s
  k = (k.float() * 0.3 + growth * pos).to(torch.bfloat16)
  q = (q.float().abs() * 0.3).to(torch.bfloat16)
  out, lse = emu.emulate_forward(info, q, k, v, mask_value=sa.DEFAULT_MASK_VALUE)
  ref, ref_lse = oracle.attention_forward(np.tril(np.ones((s, s), bool))[None], q, k, v)
  np.testing.assert_allclose(out, ref, atol=2e-2, rtol=2e-2)
  np.testing.assert_allclose(lse, ref_lse, atol=1e-3, rtol=1e-3)
