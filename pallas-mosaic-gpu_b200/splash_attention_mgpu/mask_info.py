"""Sparse block schedules: which KV blocks each q block visits, and the transpose.

Host side of the hot path.  Mirrors the reference's `mask_info.process_mask`
(`splash_attention_mgpu/mask_info.py:85-168`): same `GpuMaskInfo` fields, same
padding rule (unused step slots repeat the last visited block), same stable
heaviest-first launch orders.  The block classifier underneath (EMPTY / PARTIAL
/ FULL per block, partial-block extraction) is written here from scratch because
the reference takes it from a third-party library.

Differences from the reference, all additive:
  * classification of computable masks is analytic (O(blocks), never O(S^2));
  * compaction is vectorised numpy instead of a Python double loop;
  * `mask_descriptors` carries a per-head band descriptor `(lo, hi, chunk)` that
    the CUDA kernels evaluate in registers, so a MultiHeadMask made only of
    computable masks needs no dense blocks;
  * identical dense partial blocks are stored once.
"""

from __future__ import annotations

import dataclasses
from typing import Callable

import numpy as np

from . import splash_attention_mask as mask_lib

EMPTY = 0
PARTIAL = 1
FULL = 2

MaskFunction = Callable[..., np.ndarray]


@dataclasses.dataclass(frozen=True)
class GpuMaskInfo:
  """Per-row sparse KV schedule and its per-column transpose.

  The leading dimension of the schedule arrays is 1 (all heads share one mask)
  or the number of heads.
  """

  num_steps: np.ndarray  # i32[mask_heads, q_blocks]
  q_block_order: np.ndarray  # i32[mask_heads, q_blocks], heaviest rows first
  kv_block: np.ndarray  # i32[mask_heads, q_blocks, max_steps]
  block_kind: np.ndarray  # i32[mask_heads, q_blocks, max_steps]
  mask_block: np.ndarray | None  # i32[mask_heads, q_blocks, max_steps]
  partial_mask_blocks: np.ndarray | None  # int8[n, block_q, block_kv], 1 = attend
  mask_function: MaskFunction | None
  block_q: int
  block_kv: int
  num_kv_blocks: int
  dkv_num_steps: np.ndarray  # i32[mask_heads, kv_blocks]
  dkv_kv_block_order: np.ndarray  # i32[mask_heads, kv_blocks]
  dkv_q_block: np.ndarray  # i32[mask_heads, kv_blocks, max_dkv_steps]
  dkv_block_kind: np.ndarray  # i32[mask_heads, kv_blocks, max_dkv_steps]
  dkv_mask_block: np.ndarray | None
  partial_mask_blocks_t: np.ndarray | None  # int8[n, block_kv, block_q]
  # i32[mask_heads, 4]: (lo, hi, chunk, 0) band descriptor per mask head; None
  # when partial blocks are stored densely.
  mask_descriptors: np.ndarray | None = None

  @property
  def max_steps(self) -> int:
    return self.kv_block.shape[-1]

  @property
  def density(self) -> float:
    """Fraction of KV blocks visited compared to dense attention."""
    return float(self.num_steps.mean()) / self.num_kv_blocks


def _classify_band(mask, block_q: int, block_kv: int) -> np.ndarray:
  """Block kinds [q_blocks, kv_blocks] of a computable mask, analytically."""
  q_len, kv_len = mask.shape
  lo, hi, chunk = mask.band()
  r0 = (np.arange(q_len // block_q, dtype=np.int64) * block_q)[:, None]
  c0 = (np.arange(kv_len // block_kv, dtype=np.int64) * block_kv)[None, :]
  r1, c1 = r0 + block_q - 1, c0 + block_kv - 1
  dmin, dmax = c0 - r1, c1 - r0  # range of kv - q inside the block
  all_vis = (dmin >= lo) & (dmax <= hi)
  any_vis = (dmax >= lo) & (dmin <= hi)
  if chunk:
    same = ((r0 // chunk == r1 // chunk) & (c0 // chunk == c1 // chunk)
            & (r0 // chunk == c0 // chunk))
    overlap = (r0 // chunk <= c1 // chunk) & (c0 // chunk <= r1 // chunk)
    all_vis &= same
    any_vis &= overlap
  kinds = np.where(all_vis, FULL, EMPTY).astype(np.int32)
  # Candidates that intersect the band but are not provably full: decide them
  # exactly from the block's elements (a thin set of blocks along band edges).
  cand_r, cand_c = np.nonzero(any_vis & ~all_vis)
  for i, j in zip(cand_r.tolist(), cand_c.tolist()):
    blk = mask[i * block_q:(i + 1) * block_q, j * block_kv:(j + 1) * block_kv]
    if blk.all():
      kinds[i, j] = FULL
    elif blk.any():
      kinds[i, j] = PARTIAL
  return kinds


def _classify_dense(mask, block_q: int, block_kv: int) -> np.ndarray:
  """Block kinds of a mask known only through its elements."""
  q_len, kv_len = mask.shape
  rows, cols = q_len // block_q, kv_len // block_kv
  kinds = np.empty((rows, cols), np.int32)
  # One q-block row at a time bounds the temporary to block_q * kv_len bools.
  for i in range(rows):
    strip = np.asarray(mask[i * block_q:(i + 1) * block_q, :])
    strip = strip.reshape(block_q, cols, block_kv)
    any_v = strip.any(axis=(0, 2))
    all_v = strip.all(axis=(0, 2))
    kinds[i] = np.where(all_v, FULL, np.where(any_v, PARTIAL, EMPTY))
  return kinds


def _classify(mask, block_q, block_kv):
  if mask.band() is not None:
    return _classify_band(mask, block_q, block_kv)
  return _classify_dense(mask, block_q, block_kv)


def _compact_rows(block_mask: np.ndarray, mask_next: np.ndarray | None):
  """Compacts each row of a [heads, rows, cols] block mask into a step list.

  Follows `_compact_rows` of the reference (`mask_info.py:148-168`): step slots
  beyond `num_steps` repeat the last visited column (kind 0, mask id 0) and at
  least one slot always exists.
  """
  nonempty = block_mask != EMPTY
  num_steps = nonempty.sum(axis=-1).astype(np.int32)
  max_steps = max(1, int(num_steps.max()))
  # Stable sort on "is empty" lists the visited columns first, ascending.
  order = np.argsort(~nonempty, axis=-1, kind="stable")[..., :max_steps]
  valid = np.arange(max_steps)[None, None, :] < num_steps[..., None]
  last = np.take_along_axis(
      order, np.maximum(num_steps - 1, 0)[..., None].astype(np.int64), axis=-1)
  col = np.where(valid, order, np.where(num_steps[..., None] > 0, last, 0))
  kind = np.where(valid, np.take_along_axis(block_mask, order, axis=-1), 0)
  mask_id = None
  if mask_next is not None:
    mask_id = np.where(valid, np.take_along_axis(mask_next, order, axis=-1), 0)
    mask_id = mask_id.astype(np.int32)
  return num_steps, col.astype(np.int32), kind.astype(np.int32), mask_id


def _extract_partial_blocks(heads, kinds, block_q, block_kv):
  """Dense int8 copies of every PARTIAL block, deduplicated, and their ids."""
  blocks, where = [], []
  for h, mask in enumerate(heads):
    pr, pc = np.nonzero(kinds[h] == PARTIAL)
    if isinstance(mask, mask_lib.NumpyMask) and len(pr):
      arr = mask.array
      view = arr.reshape(arr.shape[0] // block_q, block_q,
                         arr.shape[1] // block_kv, block_kv)
      blocks.append(view[pr, :, pc, :].astype(np.int8))
    else:
      for i, j in zip(pr.tolist(), pc.tolist()):
        blk = mask[i * block_q:(i + 1) * block_q,
                   j * block_kv:(j + 1) * block_kv]
        blocks.append(np.asarray(blk, np.int8)[None])
    where.append((h, pr, pc))
  mask_next = np.zeros(kinds.shape, np.int32)
  if not blocks:
    return None, mask_next
  stacked = np.concatenate(blocks, axis=0)
  flat = np.ascontiguousarray(stacked.reshape(len(stacked), -1))
  as_void = flat.view(np.dtype((np.void, flat.shape[1]))).ravel()
  _, first, inverse = np.unique(as_void, return_index=True, return_inverse=True)
  unique_blocks = np.ascontiguousarray(stacked[first])
  pos = 0
  for h, pr, pc in where:
    mask_next[h, pr, pc] = inverse[pos:pos + len(pr)]
    pos += len(pr)
  return unique_blocks, mask_next


def _make_mask_function(heads) -> MaskFunction:
  def mask_function(q_ids, kv_ids, head: int = 0):
    return heads[head if len(heads) > 1 else 0].mask_function(q_ids, kv_ids)
  return mask_function


def process_mask(
    mask,
    block_shape: tuple[int, int],
    num_heads: int | None = None,
) -> GpuMaskInfo:
  """Builds the sparse schedule for a (multi-head) mask."""
  if isinstance(mask, mask_lib.MultiHeadMask):
    heads = list(mask.masks)
  else:
    heads = [mask] * (1 if num_heads is None else num_heads)
  block_q, block_kv = block_shape
  q_len, kv_len = heads[0].shape
  if q_len % block_q or kv_len % block_kv:
    raise ValueError(
        f"Mask shape ({q_len}, {kv_len}) must be a multiple of the block"
        f" shape ({block_q}, {block_kv}).")
  # Heads that compare equal share one schedule.
  if all(h == heads[0] for h in heads[1:]):
    heads = heads[:1]

  cache: dict = {}
  kinds_list = []
  for h in heads:
    key = id(h) if isinstance(h, mask_lib.NumpyMask) else h
    if key not in cache:
      cache[key] = _classify(h, block_q, block_kv)
    kinds_list.append(cache[key])
  block_mask = np.stack(kinds_list).astype(np.int32)
  mask_heads, q_blocks, kv_blocks = block_mask.shape

  computable = all(h.band() is not None for h in heads)
  partial_mask_blocks = mask_next = None
  mask_function = mask_descriptors = None
  if computable:
    mask_function = _make_mask_function(heads)
    mask_descriptors = np.array([list(h.band()) + [0] for h in heads], np.int32)
  elif (block_mask == PARTIAL).any():
    partial_mask_blocks, mask_next = _extract_partial_blocks(
        heads, block_mask, block_q, block_kv)

  num_steps, kv_block, block_kind, mask_block = _compact_rows(
      block_mask, mask_next)
  dkv_num_steps, dkv_q_block, dkv_block_kind, dkv_mask_block = _compact_rows(
      block_mask.transpose(0, 2, 1),
      None if mask_next is None else mask_next.transpose(0, 2, 1))

  partial_mask_blocks_t = None
  if partial_mask_blocks is not None:
    partial_mask_blocks_t = np.ascontiguousarray(
        partial_mask_blocks.transpose(0, 2, 1))
  has_mask_blocks = partial_mask_blocks is not None

  heaviest_first = lambda steps: np.argsort(
      -steps, axis=-1, kind="stable").astype(np.int32)
  return GpuMaskInfo(
      num_steps=num_steps,
      q_block_order=heaviest_first(num_steps),
      kv_block=kv_block,
      block_kind=block_kind,
      mask_block=mask_block if has_mask_blocks else None,
      partial_mask_blocks=partial_mask_blocks,
      mask_function=mask_function,
      block_q=block_q,
      block_kv=block_kv,
      num_kv_blocks=kv_blocks,
      dkv_num_steps=dkv_num_steps,
      dkv_kv_block_order=heaviest_first(dkv_num_steps),
      dkv_q_block=dkv_q_block,
      dkv_block_kind=dkv_block_kind,
      dkv_mask_block=dkv_mask_block if has_mask_blocks else None,
      partial_mask_blocks_t=partial_mask_blocks_t,
      mask_descriptors=mask_descriptors,
  )


def validate_schedule(info: GpuMaskInfo) -> None:
  """Rejects a schedule whose indices would send a kernel out of bounds.

  The kernels trust the schedule arrays; corrupt ones must be stopped on the
  host, before any launch.
  """
  q_blocks = info.num_steps.shape[1]
  for name, steps, blocks, limit in (
      ("kv_block", info.num_steps, info.kv_block, info.num_kv_blocks),
      ("dkv_q_block", info.dkv_num_steps, info.dkv_q_block, q_blocks)):
    if steps.min() < 0 or steps.max() > blocks.shape[-1]:
      raise ValueError(f"schedule step counts exceed the {name} list length")
    if blocks.min() < 0 or blocks.max() >= limit:
      raise ValueError(f"{name} index out of range [0, {limit})")
  for name, order, n in (("q_block_order", info.q_block_order, q_blocks),
                         ("dkv_kv_block_order", info.dkv_kv_block_order,
                          info.num_kv_blocks)):
    if not np.array_equal(np.sort(order, axis=-1),
                          np.broadcast_to(np.arange(n), order.shape)):
      raise ValueError(f"{name} is not a permutation")
  for kind in (info.block_kind, info.dkv_block_kind):
    if kind.min() < EMPTY or kind.max() > FULL:
      raise ValueError("block_kind outside {EMPTY, PARTIAL, FULL}")
  if info.partial_mask_blocks is not None:
    n = len(info.partial_mask_blocks)
    for ids in (info.mask_block, info.dkv_mask_block):
      if ids is None or ids.min() < 0 or ids.max() >= n:
        raise ValueError("mask_block index outside the partial block table")
  elif info.mask_descriptors is None and (info.block_kind == PARTIAL).any():
    raise ValueError("partial blocks present but no mask data to apply")
