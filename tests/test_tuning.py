"""The tile sweep, its summary and the library comparator (splash_attention_mgpu/tuning.py)."""

import pytest
import torch

import splash_attention_mgpu as sa
from splash_attention_mgpu import tuning


def test_candidates_cover_both_kernels_and_block_widths():
  cands = tuning.forward_candidates(128)
  tiles = {(c.block_q, c.block_kv) for c in cands}
  assert tiles == {(128, 64), (128, 128), (256, 64), (256, 128)}
  assert {c.num_stages for c in cands} == {2, 3, 4}
  # The two-tile kernel exists for head dims up to 128 only.
  assert all(c.block_q == 128 for c in tuning.forward_candidates(256))
  assert {c.num_stages_bwd for c in tuning.backward_candidates()} == {2, 3}


def test_summary_orders_by_forward_time_and_keeps_rejections():
  rs = [tuning.Timing("slow", None, 2.0, 5.0), tuning.Timing("fast", None, 1.0, 6.5),
        tuning.Timing("bad", None, None, None, "Shared memory budget exceeded")]
  text = tuning.summarize(rs, fwd_flops=1e12).splitlines()
  assert text[0].startswith("fast") and text[1].startswith("slow")
  assert "rejected: Shared memory budget exceeded" in text[2]
  assert "1000.0 TF" in text[0]                 # 1e12 FLOP in 1 ms
  assert tuning.best(rs).label == "slow"        # forward + backward decides
  assert tuning.best([rs[2]]) is None


@pytest.mark.gpu
def test_gpu_sweep_and_comparator():
  s, d = 1024, 128
  g = torch.Generator().manual_seed(0)
  q = (torch.randn(1, 2, s, d, generator=g) * d ** -0.5).to(torch.bfloat16).cuda()
  k, v, do = (torch.randn(1, 2, s, d, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
  mask = sa.CausalMask((s, s))
  cands = [sa.BlockSizes(block_q=128, block_kv=64, num_stages=2), sa.BlockSizes(block_q=256, block_kv=128, num_stages=2),
           sa.BlockSizes(block_q=128, block_kv=128, num_stages=4)]  # the last one exceeds shared memory
  rs = tuning.sweep(mask, q, k, v, do, candidates=cands, iters=3)
  assert [r.fwd_ms is not None for r in rs] == [True, True, False]
  assert "budget" in rs[2].error.lower()
  assert all(r.bwd_ms is not None and r.bwd_ms >= 0 for r in rs[:2])
  flops = tuning.useful_forward_flops(sa.make_splash_mha(mask), 2, 1, d)
  assert flops == 4.0 * 36 * 2 * 128 * 128 * d
  assert "rejected" in tuning.summarize(rs, flops)
  # The comparator either times the library kernel or reports why it could not.
  base = tuning.sdpa_baseline(q, k, v, do, causal=True, backend="cudnn", iters=3)
  assert (base.fwd_ms is not None) != (base.error is not None)
