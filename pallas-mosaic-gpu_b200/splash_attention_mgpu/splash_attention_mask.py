"""Attention mask types for splash attention.

The reference project imports these names from a third-party mask library
(`splash_attention_mgpu/__init__.py:4-12`); that library is not part of the
reference's own tree, so this module defines the same constructor surface from
the contract the reference's call sites rely on
(`tests/test_splash_attention_mgpu.py:51-61`, `tools/bench.py:46-52`,
`tools/fuzz.py:61-76`):

  FullMask((q, kv)); CausalMask((q, kv), offset=0);
  LocalMask((q, kv), (left, right), offset); ChunkedCausalMask((q, kv), chunk_size=c);
  NumpyMask(bool[q, kv]); MultiHeadMask([mask, ...])

  mask.shape       -> (q_len, kv_len)  ((heads, q_len, kv_len) for MultiHeadMask)
  mask[rows, cols] -> dense numpy bool array for the indexed window

Element semantics (q = query position, kv = key position):

  causal          q + offset >= kv
  local           q + offset - left <= kv <= q + offset + right   (None = unbounded)
  chunked causal  q >= kv  and  q // chunk == kv // chunk
  full            always visible

Every computable mask reduces to one *band descriptor* `(lo, hi, chunk)`:
visible iff `lo <= kv - q <= hi` and (`chunk == 0` or same chunk).  The CUDA
kernels evaluate that descriptor in registers for partial blocks, which is how
a per-head mix of computable masks stays free of dense mask blocks.
"""

from __future__ import annotations

from typing import Sequence

import numpy as np

# Sentinels for an unbounded side of the band; they fit comfortably in int32
# arithmetic on `kv - q` for any sequence length the kernels accept.
BAND_NEG_INF = -(1 << 30)
BAND_POS_INF = (1 << 30)


def _normalize_index(idx, shape):
  if not isinstance(idx, tuple):
    idx = (idx,)
  if len(idx) > len(shape):
    raise IndexError(f"too many indices for mask of rank {len(shape)}")
  idx = idx + (slice(None),) * (len(shape) - len(idx))
  out = []
  for i, n in zip(idx, shape):
    if isinstance(i, slice):
      start, stop, step = i.indices(n)
      out.append(np.arange(start, stop, step))
    else:
      out.append(np.asarray(i))
  return out


class Mask:
  """Base class: a 2-D boolean visibility relation between q and kv positions."""

  @property
  def shape(self) -> tuple[int, ...]:
    raise NotImplementedError

  def __len__(self):
    return self.shape[0]

  def __getitem__(self, idx) -> np.ndarray:
    raise NotImplementedError

  def __bool__(self):
    raise NotImplementedError("a mask has no single truth value")

  def __or__(self, other: "Mask") -> "Mask":
    return LogicalOr(self, other)

  def __and__(self, other: "Mask") -> "Mask":
    return LogicalAnd(self, other)

  # Band descriptor (lo, hi, chunk) or None when the mask is not computable.
  def band(self) -> tuple[int, int, int] | None:
    return None


class _ComputableMask(Mask):
  """A mask defined by a band descriptor; never materialised as a whole."""

  def __init__(self, shape: tuple[int, int]):
    if len(shape) != 2:
      raise ValueError(f"mask shape must be (q_len, kv_len), got {shape}")
    self._shape = (int(shape[0]), int(shape[1]))

  @property
  def shape(self):
    return self._shape

  def mask_function(self, q_ids, kv_ids):
    """Visibility for broadcastable integer arrays of positions."""
    lo, hi, chunk = self.band()
    q_ids = np.asarray(q_ids)
    kv_ids = np.asarray(kv_ids)
    diff = kv_ids - q_ids
    vis = (diff >= lo) & (diff <= hi)
    if chunk:
      vis = vis & ((q_ids // chunk) == (kv_ids // chunk))
    return vis

  def __getitem__(self, idx):
    rows, cols = _normalize_index(idx, self.shape)
    squeeze_r, squeeze_c = rows.ndim == 0, cols.ndim == 0
    out = self.mask_function(np.atleast_1d(rows)[:, None],
                             np.atleast_1d(cols)[None, :])
    if squeeze_r:
      out = out[0]
    if squeeze_c:
      out = out[..., 0]
    return out

  def __eq__(self, other):
    return (type(self) is type(other) and self.shape == other.shape
            and self.band() == other.band())

  def __hash__(self):
    return hash((type(self).__name__, self.shape, self.band()))

  def __repr__(self):
    return f"{type(self).__name__}(shape={self.shape}, band={self.band()})"


class FullMask(_ComputableMask):
  """Every query sees every key."""

  def band(self):
    return (BAND_NEG_INF, BAND_POS_INF, 0)


class CausalMask(_ComputableMask):
  """Query q sees keys kv <= q + offset."""

  def __init__(self, shape, offset: int = 0):
    super().__init__(shape)
    self.offset = int(offset)

  def band(self):
    return (BAND_NEG_INF, self.offset, 0)


class LocalMask(_ComputableMask):
  """Sliding window: q + offset - left <= kv <= q + offset + right."""

  def __init__(self, shape, window_size: tuple[int | None, int | None],
               offset: int = 0):
    super().__init__(shape)
    left, right = window_size
    self.window_size = (left, right)
    self.offset = int(offset)

  def band(self):
    left, right = self.window_size
    lo = BAND_NEG_INF if left is None else self.offset - int(left)
    hi = BAND_POS_INF if right is None else self.offset + int(right)
    return (lo, hi, 0)


class ChunkedCausalMask(_ComputableMask):
  """Causal within chunks of `chunk_size` positions; chunks do not mix."""

  def __init__(self, shape, chunk_size: int):
    super().__init__(shape)
    if chunk_size <= 0:
      raise ValueError("chunk_size must be positive")
    self.chunk_size = int(chunk_size)

  def band(self):
    return (BAND_NEG_INF, 0, self.chunk_size)


class NumpyMask(Mask):
  """A dense boolean mask held in host memory."""

  def __init__(self, array: np.ndarray):
    array = np.asarray(array)
    if array.ndim != 2:
      raise ValueError(f"NumpyMask needs a 2-D array, got {array.shape}")
    self.array = array.astype(bool, copy=False)

  @property
  def shape(self):
    return self.array.shape

  def __getitem__(self, idx):
    return self.array[idx]

  def __eq__(self, other):
    return (isinstance(other, NumpyMask) and self.shape == other.shape
            and (self.array is other.array
                 or np.array_equal(self.array, other.array)))

  def __hash__(self):
    return hash((self.shape, self.array[:1].tobytes()))


class _Logical(Mask):
  def __init__(self, left: Mask, right: Mask):
    if left.shape != right.shape:
      raise ValueError(f"mask shapes differ: {left.shape} vs {right.shape}")
    self.left, self.right = left, right

  @property
  def shape(self):
    return self.left.shape

  def __eq__(self, other):
    return (type(self) is type(other) and self.left == other.left
            and self.right == other.right)

  def __hash__(self):
    return hash((type(self).__name__, hash(self.left), hash(self.right)))


class LogicalOr(_Logical):
  def __getitem__(self, idx):
    return self.left[idx] | self.right[idx]


class LogicalAnd(_Logical):
  def __getitem__(self, idx):
    return self.left[idx] & self.right[idx]


class MultiHeadMask:
  """One 2-D mask per attention head."""

  def __init__(self, masks: Sequence[Mask]):
    masks = tuple(masks)
    if not masks:
      raise ValueError("MultiHeadMask needs at least one head")
    first = masks[0].shape
    for m in masks:
      if isinstance(m, MultiHeadMask) or len(m.shape) != 2:
        raise ValueError("heads of a MultiHeadMask must be 2-D masks")
      if m.shape != first:
        raise ValueError(f"head mask shapes differ: {m.shape} vs {first}")
    self.masks = masks

  @property
  def shape(self):
    return (len(self.masks),) + tuple(self.masks[0].shape)

  def __len__(self):
    return len(self.masks)

  def __getitem__(self, idx):
    if not isinstance(idx, tuple):
      idx = (idx,)
    head_idx, rest = idx[0], idx[1:]
    rest = rest if rest else (slice(None), slice(None))
    if isinstance(head_idx, slice):
      return np.stack([m[rest] for m in self.masks[head_idx]])
    return self.masks[head_idx][rest]

  def __eq__(self, other):
    return isinstance(other, MultiHeadMask) and self.masks == other.masks

  def __hash__(self):
    return hash(tuple(hash(m) for m in self.masks))
