"""Host schedule: block classification, compaction, transposed lists, launch orders.

Assertions mirror the reference's host-only tests
(tests/test_splash_attention_mgpu.py:133-168, 537-559).
"""

import numpy as np
import pytest

import splash_attention_mgpu as sa
from splash_attention_mgpu import mask_info as mask_info_lib

from common import masks


def _rebuild(info, dense, head=0, transposed=False):
  bq, bkv = info.block_q, info.block_kv
  rebuilt = np.zeros_like(dense)
  if not transposed:
    steps, blocks, kinds, ids, pblocks = (info.num_steps, info.kv_block, info.block_kind,
                                          info.mask_block, info.partial_mask_blocks)
  else:
    steps, blocks, kinds, ids, pblocks = (info.dkv_num_steps, info.dkv_q_block,
                                          info.dkv_block_kind, info.dkv_mask_block,
                                          info.partial_mask_blocks_t)
  for a in range(steps.shape[1]):
    for step in range(steps[head, a]):
      o = blocks[head, a, step]
      i, j = (a, o) if not transposed else (o, a)
      rows, cols = slice(i * bq, (i + 1) * bq), slice(j * bkv, (j + 1) * bkv)
      kind = kinds[head, a, step]
      if kind == mask_info_lib.FULL:
        rebuilt[rows, cols] = True
      elif pblocks is not None:
        blk = pblocks[ids[head, a, step]].astype(bool)
        rebuilt[rows, cols] = blk if not transposed else blk.T
      else:
        q_pos = np.arange(i * bq, (i + 1) * bq)[:, None]
        kv_pos = np.arange(j * bkv, (j + 1) * bkv)[None, :]
        rebuilt[rows, cols] = np.asarray(info.mask_function(q_pos, kv_pos, head))
  return rebuilt


@pytest.mark.parametrize("name", ["full", "causal", "local", "chunked", "dense"])
@pytest.mark.parametrize("bkv", [64, 128])
def test_mask_info_reconstructs_mask(name, bkv):
  s = 512
  mask = masks(s)[name]
  info = mask_info_lib.process_mask(mask, (128, bkv))
  dense = np.asarray(mask[:, :])
  np.testing.assert_array_equal(_rebuild(info, dense), dense)
  # Launch orders are permutations, heaviest rows / columns first.
  for order, steps in ((info.q_block_order, info.num_steps),
                       (info.dkv_kv_block_order, info.dkv_num_steps)):
    np.testing.assert_array_equal(np.sort(order[0]), np.arange(len(order[0])))
    assert np.all(np.diff(steps[0][order[0]]) <= 0)
  mask_info_lib.validate_schedule(info)


@pytest.mark.parametrize("name", ["full", "causal", "local", "chunked", "dense"])
@pytest.mark.parametrize("bq", [128, 256])
def test_transposed_schedule_reconstructs_mask(name, bq):
  s = 1024
  mask = masks(s)[name]
  info = mask_info_lib.process_mask(mask, (bq, 128))
  dense = np.asarray(mask[:, :])
  np.testing.assert_array_equal(_rebuild(info, dense, transposed=True), dense)


def test_padding_repeats_last_block():
  info = mask_info_lib.process_mask(sa.CausalMask((512, 512)), (128, 128))
  assert info.kv_block.shape == (1, 4, 4)
  np.testing.assert_array_equal(info.num_steps[0], [1, 2, 3, 4])
  np.testing.assert_array_equal(info.kv_block[0, 0], [0, 0, 0, 0])
  np.testing.assert_array_equal(info.kv_block[0, 1], [0, 1, 1, 1])
  np.testing.assert_array_equal(info.block_kind[0, 1], [2, 1, 0, 0])


def test_mask_info_is_sparse():
  info = mask_info_lib.process_mask(sa.LocalMask((4096, 4096), (256, 0), 0), (128, 128))
  assert info.max_steps == 3
  assert info.density < 0.1


def test_empty_rows_keep_one_slot():
  dense = np.zeros((256, 256), bool)
  dense[128:, :] = True
  info = mask_info_lib.process_mask(sa.NumpyMask(dense), (128, 128))
  assert info.num_steps[0, 0] == 0 and info.num_steps[0, 1] == 2
  assert info.kv_block.shape[-1] == 2
  assert info.partial_mask_blocks is None  # only FULL blocks: nothing to mask


def test_multi_head_mask_schedules():
  s = 512
  zoo = masks(s)
  heads = [zoo["causal"], zoo["local"], zoo["chunked"]]
  info = mask_info_lib.process_mask(sa.MultiHeadMask(heads), (128, 64))
  assert info.num_steps.shape[0] == 3
  assert info.partial_mask_blocks is None and info.mask_descriptors.shape == (3, 4)
  for h, m in enumerate(heads):
    dense = np.asarray(m[:, :])
    np.testing.assert_array_equal(_rebuild(info, dense, head=h), dense)
  # A dense head forces dense blocks for every head.
  heads.append(zoo["dense"])
  info = mask_info_lib.process_mask(sa.MultiHeadMask(heads), (128, 128))
  assert info.mask_function is None and info.partial_mask_blocks is not None
  for h, m in enumerate(heads):
    dense = np.asarray(m[:, :])
    np.testing.assert_array_equal(_rebuild(info, dense, head=h), dense)
    np.testing.assert_array_equal(_rebuild(info, dense, head=h, transposed=True), dense)


def test_identical_heads_share_one_schedule():
  m = sa.CausalMask((512, 512))
  info = mask_info_lib.process_mask(sa.MultiHeadMask([m, sa.CausalMask((512, 512))]), (128, 128))
  assert info.num_steps.shape[0] == 1


def test_partial_blocks_are_deduplicated():
  dense = np.tril(np.ones((1024, 1024), bool))
  info = mask_info_lib.process_mask(sa.NumpyMask(dense), (128, 128))
  assert len(info.partial_mask_blocks) == 1  # all diagonal blocks are the same triangle
  assert info.partial_mask_blocks.dtype == np.int8
  np.testing.assert_array_equal(info.partial_mask_blocks_t[0], info.partial_mask_blocks[0].T)


def test_block_counts_of_the_benchmark_masks():
  causal = mask_info_lib.process_mask(sa.CausalMask((8192, 8192)), (128, 128))
  assert int(causal.num_steps.sum()) == 2080
  assert int((causal.block_kind == mask_info_lib.PARTIAL).sum()) == 64
  local = mask_info_lib.process_mask(sa.LocalMask((16384, 16384), (1024, 0), 0), (128, 128))
  assert int(local.num_steps.sum()) == 1116 and local.max_steps == 9
  chunked = mask_info_lib.process_mask(sa.ChunkedCausalMask((8192, 8192), 1024), (128, 64))
  assert int(chunked.num_steps.sum()) == 576


def test_rejects_shapes_that_do_not_tile():
  with pytest.raises(ValueError, match="multiple"):
    mask_info_lib.process_mask(sa.FullMask((384, 384)), (256, 128))


def test_validator_rejects_corrupt_schedules():
  import dataclasses
  info = mask_info_lib.process_mask(masks(512)["dense"], (128, 128))
  bad = dataclasses.replace(info, kv_block=info.kv_block + 100)
  with pytest.raises(ValueError, match="kv_block"):
    mask_info_lib.validate_schedule(bad)
  bad = dataclasses.replace(info, num_steps=info.num_steps + 100)
  with pytest.raises(ValueError, match="step counts"):
    mask_info_lib.validate_schedule(bad)
  bad = dataclasses.replace(info, mask_block=info.mask_block + 10 ** 6)
  with pytest.raises(ValueError, match="mask_block"):
    mask_info_lib.validate_schedule(bad)
  bad = dataclasses.replace(info, q_block_order=np.zeros_like(info.q_block_order))
  with pytest.raises(ValueError, match="permutation"):
    mask_info_lib.validate_schedule(bad)


def test_mask_indexing_and_logical_ops():
  s = 256
  c, l = sa.CausalMask((s, s)), sa.LocalMask((s, s), (16, None), 0)
  both = c & l
  np.testing.assert_array_equal(both[:, :], np.asarray(c[:, :]) & np.asarray(l[:, :]))
  np.testing.assert_array_equal((c | l)[10:20, 5:9], np.asarray(c[10:20, 5:9]) | np.asarray(l[10:20, 5:9]))
  info = mask_info_lib.process_mask(both, (128, 128))
  np.testing.assert_array_equal(_rebuild(info, np.asarray(both[:, :])), both[:, :])
  # Causal with an offset and a local window follow the documented element rules.
  off = sa.CausalMask((s, s), offset=3)
  q, kv = np.arange(s)[:, None], np.arange(s)[None, :]
  np.testing.assert_array_equal(off[:, :], q + 3 >= kv)
  loc = sa.LocalMask((s, s), (7, 2), 1)
  np.testing.assert_array_equal(loc[:, :], (kv >= q + 1 - 7) & (kv <= q + 1 + 2))
  ch = sa.ChunkedCausalMask((s, s), chunk_size=48)
  np.testing.assert_array_equal(ch[:, :], (q >= kv) & (q // 48 == kv // 48))
