"""Tiling configuration: validation messages and automatic block_q choice
(reference tests/test_splash_attention_mgpu.py:262-268, 537-559)."""

import numpy as np
import pytest

import splash_attention_mgpu as sa


def test_rejects_invalid_block_sizes():
  with pytest.raises(ValueError, match="num_stages"):
    sa.BlockSizes(num_stages=1)
  with pytest.raises(ValueError, match="block_kv"):
    sa.BlockSizes(block_kv=256)
  with pytest.raises(ValueError, match="block_q_dkv"):
    sa.BlockSizes(block_q_dkv=32)
  with pytest.raises(ValueError, match="block_q"):
    sa.BlockSizes(block_q=64)
  with pytest.raises(ValueError, match="block_kv_dq"):
    sa.BlockSizes(block_kv_dq=32)
  with pytest.raises(ValueError, match="num_stages_bwd"):
    sa.BlockSizes(num_stages_bwd=0)


def test_auto_forward_tiling_by_row_length():
  s = 4096
  tiles = lambda m, d: (lambda bs: (bs.block_q, bs.block_kv, bs.num_stages))(
      sa.make_splash_mha(m).resolved_block_sizes(d, d))
  # Long rows: 128-wide blocks, two alternating softmax warpgroups.
  assert tiles(sa.FullMask((s, s)), 128) == (128, 128, 2)
  assert tiles(sa.CausalMask((8192, 8192)), 128) == (128, 128, 2)
  # Short rows: 64-wide blocks and a two-stage ring (two CTAs per SM).
  assert tiles(sa.CausalMask((2048, 2048)), 128) == (128, 64, 2)
  assert tiles(sa.LocalMask((s, s), (1024, 0), 0), 128) == (128, 64, 2)
  assert tiles(sa.ChunkedCausalMask((s, s), 1024), 128) == (128, 64, 2)
  # Head dim 64: two CTAs per SM with 64-wide blocks; the two-tile kernel where its schedule is free.
  assert tiles(sa.CausalMask((s, s)), 64) == (128, 64, 2)
  assert tiles(sa.FullMask((s, s)), 64) == (256, 128, 2)
  # Other head dims keep the one-tile defaults.
  assert tiles(sa.FullMask((s, s)), 256) == (128, 128, 2)
  # The two-tile kernel runs when asked for; open fields are filled in around it.
  k = sa.make_splash_mha(sa.FullMask((s, s)), block_sizes=sa.BlockSizes(block_q=256))
  assert k.choose_block_q(128, 128) == 256
  bs = k.resolved_block_sizes(128, 128)
  assert (bs.block_q, bs.block_kv, bs.num_stages) == (256, 128, 2)
  k = sa.make_splash_mha(sa.FullMask((s, s)), block_sizes=sa.BlockSizes(block_kv=64))
  assert k.resolved_block_sizes(128, 128).block_kv == 64


def test_auto_forward_tiling_with_dense_masks():
  # Streamed mask blocks take the 128-wide tiling: with 64-wide blocks they would
  # push the kernel past the shared memory that lets two CTAs share an SM.
  dense = np.tril(np.ones((2048, 2048), bool))
  bs = sa.make_splash_mha(sa.NumpyMask(dense)).resolved_block_sizes(128, 128)
  assert (bs.block_q, bs.block_kv, bs.num_stages) == (128, 128, 2)


def test_resolved_tiles_of_the_benchmark_configs():
  k = sa.make_splash_mha(sa.CausalMask((8192, 8192)))
  bs = k.resolved_block_sizes(128, 128)
  assert (bs.block_q, bs.block_kv, bs.num_stages) == (128, 128, 2)
  assert abs(k.pingpong_extra_work - 1056 * 256 / (2080 * 128)) < 1e-9
  k = sa.make_splash_mha(sa.LocalMask((16384, 16384), (1024, 0), 0))
  bs = k.resolved_block_sizes(128, 128)
  assert (bs.block_q, bs.block_kv, bs.num_stages) == (128, 64, 2)
  k = sa.make_splash_mha(sa.FullMask((8192, 8192)))
  bs = k.resolved_block_sizes(64, 64, has_segments=True)
  assert (bs.block_q, bs.block_kv, bs.num_stages) == (128, 64, 2)


def test_numpy_masks_become_multi_head_masks():
  m = np.ones((3, 256, 256), bool)
  k = sa.make_splash_mqa(m)
  assert isinstance(k.mask, sa.MultiHeadMask) and k.mask.shape == (3, 256, 256) and k.is_mqa
  k = sa.make_splash_mha(np.ones((256, 256), bool))
  assert k.mask.shape == (1, 256, 256) and k.info.num_steps.shape[0] == 1


def test_cpu_tensors_are_refused():
  import torch
  k = sa.make_splash_mha(sa.CausalMask((256, 256)))
  q = torch.zeros(1, 256, 64, dtype=torch.bfloat16)
  with pytest.raises(RuntimeError, match="no CPU path"):
    k(q, q, q)
