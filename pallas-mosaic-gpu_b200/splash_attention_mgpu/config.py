"""Tiling configuration, segment ids and budget rules of the splash kernels.

`BlockSizes` and `SegmentIds` keep the field names, defaults and validation
messages of the reference (`splash_attention_mgpu/kernel.py:59-109`) because
callers construct them by keyword and tests match on the error text.  The
budget functions restate the reference's shared-memory / tensor-memory
formulas (`kernel.py:175-189`, `forward_pingpong.py:117-128,167`,
`backward.py:53-63,112-121,415-423`, `backward_fused.py:45-61`) so that a
configuration the reference rejects is rejected here with the same exception
type and wording.
"""

from __future__ import annotations

import dataclasses
from typing import Any, NamedTuple

import numpy as np

DEFAULT_MASK_VALUE = -0.7 * float(np.finfo(np.dtype("float32")).max)

TILE_ROWS = 128  # query rows handled by one softmax warpgroup (one TMEM lane each)
PINGPONG_ROWS = 2 * TILE_ROWS
TMEM_COLS = 512
# 227 KiB of dynamic shared memory per CTA on sm_100, minus room for barriers
# and the 1 KiB alignment of swizzled tiles.
SMEM_BYTES = 227 * 1024 - 4096

# At head_dim 128 the automatic forward tiling takes 128-wide KV blocks when a
# 128-row tile visits at least this many of them on average, 64-wide otherwise.
AUTO_WIDE_BLOCK_MIN_STEPS = 24


class SegmentIds(NamedTuple):
  """Tokens attend only within equal segment ids.

  q:  i32[q_len]  or i32[batch, q_len]
  kv: i32[kv_len] or i32[batch, kv_len]
  """

  q: Any
  kv: Any


@dataclasses.dataclass(frozen=True)
class BlockSizes:
  """Tiling of the forward and backward kernels.

  block_q / block_kv: granularity of the sparse schedule and of the forward
    tiles.  block_q 256 selects the two-tile ping-pong forward; None picks it
    per call where it is faster.
  num_stages: depth of the forward K/V shared-memory ring.
  block_kv_dq / block_q_dkv: contraction sub-block of the dQ / dK-dV kernels
    (64 or 128; None picks the largest that fits).
  num_stages_bwd: ring depth of the backward kernels.
  """

  block_q: int | None = None
  block_kv: int | None = None
  num_stages: int | None = None
  block_kv_dq: int | None = None
  block_q_dkv: int | None = None
  num_stages_bwd: int = 2

  def __post_init__(self):
    if self.block_q not in (None, TILE_ROWS, PINGPONG_ROWS):
      raise ValueError(f"block_q must be None, 128 or 256, got {self.block_q}")
    if self.block_kv not in (None, 64, 128):
      raise ValueError(f"block_kv must be 64 or 128, got {self.block_kv}")
    if self.num_stages is not None and self.num_stages < 2:
      # The score MMA of step s+1 is issued before P.V of step s, so a ring
      # shallower than two steps cannot make progress.
      raise ValueError(f"num_stages must be >= 2, got {self.num_stages}")
    if self.block_kv_dq not in (None, 64, 128):
      raise ValueError(f"block_kv_dq={self.block_kv_dq} must be 64 or 128")
    if self.block_q_dkv not in (None, 64, 128):
      raise ValueError(f"block_q_dkv={self.block_q_dkv} must be 64 or 128")
    if self.num_stages_bwd < 1:
      raise ValueError("num_stages_bwd must be >= 1")


def auto_forward_tiles(head_dim: int, block_q: int) -> tuple[int, int]:
  """(block_kv, num_stages) defaults (`splash_attention.py:41-45`)."""
  if head_dim <= 64 and block_q == TILE_ROWS:
    return 64, 3
  return 128, 2


# ---------------------------------------------------------------------------
# Budgets
# ---------------------------------------------------------------------------


def fwd128_tmem_cols(head_dim_v: int, block_kv: int) -> int:
  return head_dim_v + 2 * block_kv + block_kv // 2


def fwd128_smem_bytes(*, head_dim, head_dim_v, block_kv, num_stages, itemsize,
                      has_dense_mask, has_segments, save_residuals) -> int:
  bq = TILE_ROWS
  return (bq * head_dim * itemsize
          + (0 if head_dim == head_dim_v else bq * head_dim_v * itemsize)
          + num_stages * block_kv * (head_dim + head_dim_v) * itemsize
          + (num_stages * bq * block_kv if has_dense_mask else 0)
          + (bq + num_stages * block_kv) * 4 * bool(has_segments)
          + bq * 4 * bool(save_residuals))


def pingpong_tmem_cols(head_dim: int, block_kv: int) -> int:
  return 2 * (block_kv + head_dim)


def pingpong_smem_bytes(*, head_dim, block_kv, num_stages, itemsize,
                        has_dense_mask, has_segments, save_residuals) -> int:
  return (PINGPONG_ROWS * head_dim * itemsize
          + num_stages * block_kv * 2 * head_dim * itemsize
          + (num_stages * PINGPONG_ROWS * block_kv if has_dense_mask else 0)
          + (PINGPONG_ROWS + num_stages * block_kv) * 4 * bool(has_segments)
          + PINGPONG_ROWS * 4 * bool(save_residuals)
          + 2 * TILE_ROWS * 4)


def pingpong_fits(**kw) -> bool:
  return pingpong_smem_bytes(**kw) <= SMEM_BYTES


def bwd_dq_tmem_cols(head_dim: int, sub_block: int) -> int:
  return 2 * sub_block + sub_block // 2 + head_dim


def bwd_dq_smem_bytes(*, head_dim, head_dim_v, sub_block, num_stages, itemsize,
                      has_dense_mask, has_segments) -> int:
  bq = TILE_ROWS
  return (bq * (head_dim + head_dim_v) * itemsize  # Q, dO
          + num_stages * sub_block * (head_dim + head_dim_v) * itemsize
          + 2 * bq * 4  # lse, delta
          + (num_stages * bq * sub_block if has_dense_mask else 0)
          + (bq + num_stages * sub_block) * 4 * bool(has_segments))


def bwd_dkv_tmem_cols(head_dim: int, head_dim_v: int, sub_block: int,
                      nbuf: int = 1) -> int:
  return 2 * nbuf * sub_block + head_dim + head_dim_v


def bwd_dkv_smem_bytes(*, head_dim, head_dim_v, sub_block, num_stages,
                       itemsize, has_dense_mask, has_segments) -> int:
  bkv = TILE_ROWS
  return (bkv * (head_dim + head_dim_v) * itemsize  # K, V resident
          + num_stages * sub_block * (head_dim + head_dim_v) * itemsize
          + num_stages * 2 * sub_block * 4  # lse, delta per step
          + (num_stages * bkv * sub_block if has_dense_mask else 0)
          + (bkv + num_stages * sub_block) * 4 * bool(has_segments))


def fused_supported(head_dim: int, head_dim_v: int) -> bool:
  return head_dim == head_dim_v and head_dim in (64, 128)


def fused_sub_block(head_dim: int) -> int:
  """q rows per step of the fused backward (64 at either head dim)."""
  del head_dim
  return 64


def fused_tmem_cols(head_dim: int) -> int:
  """Two S^T and two dP^T buffers of 64 columns, dK and dV."""
  return 4 * fused_sub_block(head_dim) + 2 * head_dim


def fused_smem_bytes(*, head_dim, num_stages, itemsize, has_dense_mask,
                     has_segments) -> int:
  bc = fused_sub_block(head_dim)
  bkv = TILE_ROWS
  return (bkv * 2 * head_dim * itemsize  # K, V resident
          + (bkv * 128 if head_dim == 64 else 0)  # second copy of K for the dQ operand
          + num_stages * bc * 2 * head_dim * itemsize  # Q, dO ring
          + num_stages * 2 * bc * 4  # lse, delta
          + 2 * bkv * bc * itemsize  # dS^T staged as an MMA operand, 2 buffers
          + 128 * 32 * 4  # dQ^T staging for the reduce-add
          + (num_stages * bkv * bc if has_dense_mask else 0)
          + (bkv + num_stages * bc) * 4 * bool(has_segments))


def fused_fits(**kw) -> bool:
  return fused_smem_bytes(**kw) <= SMEM_BYTES


def largest_fitting_sub_block(tmem_fn, smem_fn) -> int | None:
  for sb in (128, 64):
    if tmem_fn(sb) <= TMEM_COLS and smem_fn(sb) <= SMEM_BYTES:
      return sb
  return None
