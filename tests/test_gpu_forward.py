"""Forward kernels on a B200 through the C ABI, against the CPU oracle.

Case lists replay the reference's GPU tiers (tests/test_splash_attention_mgpu.py:
290-316 masks/features, 465-513 ping-pong, 207-222 empty rows, 319-342 lazy
rescaling) at its sizes (s = 2048 unless stated).
"""

import numpy as np
import pytest
import torch

import splash_attention_mgpu as sa
from oracle import dense_attention as oracle

from common import assert_forward_close, build_mask, inputs, segments

pytestmark = pytest.mark.gpu

_id = lambda kw: ",".join(f"{k}={v}" for k, v in kw.items()) or "default"


def _check(mask_name, *, s=2048, b=None, h=2, kvh=None, d=64, dv=None, dtype=torch.bfloat16, mqa=False,
           segs=False, cap=None, block_sizes=sa.BlockSizes(), multi_head_mask=False):
  dv = dv or d
  kvh = kvh or h
  mask, dense = build_mask(mask_name, s, h, multi_head_mask)
  make = sa.make_splash_mqa if mqa else sa.make_splash_mha
  kernel = make(mask, block_sizes=block_sizes, attn_logits_soft_cap=cap)
  q, k, v = inputs(b, h, kvh, s, d, dv, dtype, mqa, device="cuda:0")
  seg = segments(s, "cuda:0") if segs else None
  out, (lse,) = kernel(q, k, v, seg, save_residuals=True)
  sa.check_device_status()
  ref, ref_lse = oracle.attention_forward(dense, q, k, v, seg, is_mqa=mqa, attn_logits_soft_cap=cap)
  assert_forward_close(out, lse, ref, ref_lse, dtype)
  # Same call without residuals returns the same output.
  out2 = kernel(q, k, v, seg)
  assert torch.equal(out2, out)


def test_plumbing_configuration():
  # Causal MHA, batch 1, 2 heads, seq 512, head_dim 64, bf16, q pre-scaled, 128x128 blocks.
  s, d = 512, 64
  kernel = sa.make_splash_mha(sa.CausalMask((s, s)), block_sizes=sa.BlockSizes(block_q=128, block_kv=128))
  q, k, v = inputs(1, 2, 2, s, d, d, torch.bfloat16, False, device="cuda:0", scale=d ** -0.5)
  out, (lse,) = kernel(q, k, v, save_residuals=True)
  sa.check_device_status()
  ref, ref_lse = oracle.attention_forward(np.tril(np.ones((s, s), bool))[None], q, k, v)
  assert_forward_close(out, lse, ref, ref_lse, torch.bfloat16)
  assert out.shape == (1, 2, s, d) and lse.shape == (1, 2, s) and lse.dtype == torch.float32


@pytest.mark.parametrize("name", ["full", "causal", "local", "chunked", "dense"])
@pytest.mark.parametrize("d", [64, 128])
def test_gpu_masks(name, d):
  _check(name, s=2048, h=4, d=d)


FEATURES = [
    dict(segs=True),
    dict(segs=True, mask_name="dense"),
    dict(cap=5.0),
    dict(mqa=True, b=2),
    dict(h=8, kvh=2),
    dict(b=2, segs=True),
    dict(d=128, dv=64),
    dict(d=64, dv=128),
    dict(d=192, block_sizes=sa.BlockSizes(block_kv=64)),
    dict(d=256, block_sizes=sa.BlockSizes(block_kv=64)),
    dict(block_sizes=sa.BlockSizes(block_kv=64), s=1024),
    dict(block_sizes=sa.BlockSizes(block_kv=128)),
    dict(block_sizes=sa.BlockSizes(num_stages=3)),
    dict(block_sizes=sa.BlockSizes(num_stages=3), mask_name="dense"),
    dict(d=128, block_sizes=sa.BlockSizes(block_kv=64, num_stages=4)),
    dict(multi_head_mask=True, h=5),
    dict(multi_head_mask=True, h=3, mask_name="full"),
    dict(dtype=torch.float16),
    dict(dtype=torch.float16, d=128, mask_name="dense", segs=True),
]


@pytest.mark.parametrize("kwargs", FEATURES, ids=_id)
def test_gpu_features(kwargs):
  kwargs = dict(kwargs)
  _check(kwargs.pop("mask_name", "causal"), **kwargs)


PINGPONG = sa.BlockSizes(block_q=256)
PINGPONG_CASES = [
    dict(mask_name="full"),
    dict(mask_name="causal"),
    dict(mask_name="local"),
    dict(mask_name="chunked"),
    dict(mask_name="dense", block_sizes=sa.BlockSizes(block_q=256, block_kv=64)),
    dict(mask_name="causal", segs=True),
    dict(mask_name="dense", segs=True, block_sizes=sa.BlockSizes(block_q=256, block_kv=64)),
    dict(mask_name="causal", cap=5.0),
    dict(mask_name="causal", h=4, kvh=2),
    dict(mask_name="full", mqa=True, b=2),
    dict(mask_name="causal", d=128),
    dict(mask_name="local", d=128, s=1024),
    dict(mask_name="causal", multi_head_mask=True, h=3),
    dict(mask_name="causal", dtype=torch.float16),
    dict(mask_name="causal", block_sizes=sa.BlockSizes(block_q=256, num_stages=3)),
    dict(mask_name="dense", d=128, block_sizes=sa.BlockSizes(block_q=256, block_kv=64)),
]


@pytest.mark.parametrize("kwargs", PINGPONG_CASES, ids=_id)
def test_gpu_pingpong(kwargs):
  kwargs = dict(kwargs)
  kwargs.setdefault("block_sizes", PINGPONG)
  _check(kwargs.pop("mask_name"), **kwargs)


def test_auto_tiles_at_head_dim_128():
  kernel = sa.make_splash_mha(sa.CausalMask((2048, 2048)))
  bs = kernel.resolved_block_sizes(128, 128)
  assert (bs.block_q, bs.block_kv, bs.num_stages) == (128, 64, 2)
  _check("causal", d=128, h=2)


# 128-wide KV blocks in the one-tile kernel: two softmax warpgroups alternate over the
# KV steps and pass the running row maximum to one another.
WIDE = sa.BlockSizes(block_q=128, block_kv=128)
WIDE_CASES = [
    dict(mask_name="full", d=128),
    dict(mask_name="causal", d=128),
    dict(mask_name="local", d=128),
    dict(mask_name="chunked", d=128),
    dict(mask_name="dense", d=128),
    dict(mask_name="causal", d=128, s=128),   # one step: the second group never runs one
    dict(mask_name="causal", d=128, s=256),
    dict(mask_name="full", d=128, s=384),     # odd number of steps
    dict(mask_name="causal", d=128, segs=True),
    dict(mask_name="dense", d=128, segs=True),
    dict(mask_name="causal", d=128, cap=5.0),
    dict(mask_name="causal", d=128, h=4, kvh=2),
    dict(mask_name="full", d=128, mqa=True, b=2),
    dict(mask_name="causal", d=128, multi_head_mask=True, h=3),
    dict(mask_name="causal", d=128, dtype=torch.float16),
    dict(mask_name="causal", d=64),
    dict(mask_name="dense", d=64, segs=True),
    dict(mask_name="causal", d=64, dv=128),
    dict(mask_name="causal", d=128, dv=64),
    # Many more tiles than SMs, most of them one to four steps long: several waves of short
    # CTAs, one-step tiles included.
    dict(mask_name="causal", d=128, s=512, b=4, h=40),
    dict(mask_name="local", d=64, s=1024, b=3, h=24, segs=True),
    dict(mask_name="chunked", d=128, s=1024, b=2, h=32, kvh=8, cap=5.0),
]


@pytest.mark.parametrize("kwargs", WIDE_CASES, ids=_id)
def test_gpu_alternating_warpgroups(kwargs):
  kwargs = dict(kwargs)
  kwargs.setdefault("block_sizes", WIDE)
  _check(kwargs.pop("mask_name"), **kwargs)


@pytest.mark.parametrize("bq,bkv", [(128, None), (128, 128), (256, None)])
def test_gpu_empty_rows_are_zero(bq, bkv):
  # The first q block sees nothing: its output is zero and lse = mask_value.
  s = 512
  dense = np.zeros((s, s), bool)
  dense[256:, :] = True
  kernel = sa.make_splash_mha(sa.NumpyMask(dense), block_sizes=sa.BlockSizes(block_q=bq, block_kv=bkv))
  q, k, v = inputs(None, 1, 1, s, 64, 64, torch.bfloat16, False, device="cuda:0")
  out, (lse,) = kernel(q, k, v, save_residuals=True)
  sa.check_device_status()
  assert torch.all(out[:, :256] == 0)
  assert torch.all(lse[:, :256] == np.float32(sa.DEFAULT_MASK_VALUE))
  ref, _ = oracle.attention_forward(dense[None], q, k, v)
  np.testing.assert_allclose(out[:, 256:].float().cpu().numpy(), ref[:, 256:], atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("growth", [0.0, 0.05, 40.0, -40.0])
@pytest.mark.parametrize("bq,bkv", [(128, None), (128, 128), (256, None)])
def test_gpu_lazy_rescaling(growth, bq, bkv):
  # Logits that drift up (or down) along the keys: the running maximum moves at every
  # step, at some steps only, or never, and O is rescaled accordingly.
  s, d = 1024, 64
  kernel = sa.make_splash_mha(sa.CausalMask((s, s)), block_sizes=sa.BlockSizes(block_q=bq, block_kv=bkv))
  q, k, v = inputs(None, 2, 2, s, d, d, torch.bfloat16, False)
  pos = torch.arange(s, dtype=torch.float32)[None, :, None] / s
  k = (k.float() * 0.3 + growth * pos).to(torch.bfloat16).cuda()
  q = (q.float().abs() * 0.3).to(torch.bfloat16).cuda()
  v = v.cuda()
  out, (lse,) = kernel(q, k, v, save_residuals=True)
  sa.check_device_status()
  ref, ref_lse = oracle.attention_forward(np.tril(np.ones((s, s), bool))[None], q, k, v)
  assert_forward_close(out, lse, ref, ref_lse, torch.bfloat16)


def test_rejects_oversized_configs():
  kernel = sa.make_splash_mha(sa.CausalMask((512, 512)))
  q, k, v = inputs(None, 1, 1, 512, 256, 256, torch.bfloat16, False, device="cuda:0")
  with pytest.raises(ValueError, match="TMEM budget"):
    kernel(q, k, v)
  kernel = sa.make_splash_mha(sa.CausalMask((512, 512)), block_sizes=sa.BlockSizes(block_kv=128, num_stages=4))
  q, k, v = inputs(None, 1, 1, 512, 128, 128, torch.bfloat16, False, device="cuda:0")
  with pytest.raises(ValueError, match="Shared memory budget"):
    kernel(q, k, v)
  with pytest.raises(NotImplementedError):
    kernel(q.float(), k.float(), v.float())


def test_results_are_deterministic():
  kernel = sa.make_splash_mha(sa.CausalMask((2048, 2048)), block_sizes=sa.BlockSizes(block_q=256))
  q, k, v = inputs(2, 4, 4, 2048, 128, 128, torch.bfloat16, False, device="cuda:0", scale=128 ** -0.5)
  first = kernel(q, k, v)
  for _ in range(3):
    assert torch.equal(kernel(q, k, v), first)
