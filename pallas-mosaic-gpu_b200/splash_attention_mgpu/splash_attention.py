"""Public API of the B200 splash attention library.

Drop-in for the reference's `splash_attention_mgpu.splash_attention`
(`splash_attention.py:48-407`): same constructor functions, the same
`SplashAttentionKernel` attributes and call signature, the same exception types
and message keywords.  Arrays are `torch` CUDA tensors (the reference takes JAX
arrays); differentiation goes through `torch.autograd` where the reference uses
`jax.custom_vjp`.

    kernel = make_splash_mha(mask, block_sizes=BlockSizes())
    out = kernel(q, k, v)                     # q: [heads, q_len, head_dim]
    out = kernel(q, k, v, segment_ids)        # or with a leading batch dim
    out, (lse,) = kernel(q, k, v, save_residuals=True)   # forward only

`q` is expected to be pre-scaled; no softmax scale is applied.

All compute runs in hand-written sm_100a kernels behind `libsplash_sm100.so`.
Nothing here falls back to another implementation: without the library or
without a CUDA device a call raises.
"""

from __future__ import annotations

import ctypes
import dataclasses
import functools
import os
from typing import Any, NamedTuple

import numpy as np
import torch

from . import _ffi
from . import config as cfg
from . import mask_info as mask_info_lib
from . import splash_attention_mask as mask_lib
from .config import (DEFAULT_MASK_VALUE,
                     BlockSizes, SegmentIds, auto_forward_tiles)

_TORCH_DTYPES = {torch.bfloat16: _ffi.DTYPE_BF16, torch.float16: _ffi.DTYPE_F16}


# ---------------------------------------------------------------------------
# Device-side state
# ---------------------------------------------------------------------------

_status_words: dict = {}
# device key -> (pinned host copy of the word, event recorded after the copy, side stream that carries
# the copy, event that marks the kernels the copy has to follow)
_status_mirrors: dict = {}


def _status_word(device: torch.device) -> torch.Tensor:
  """The 4-int status word the kernels report into (one per device)."""
  key = (device.type, device.index)
  if key not in _status_words:
    _status_words[key] = torch.zeros(4, dtype=torch.int32, device=device)
  return _status_words[key]


def _raise_device_status(word: torch.Tensor, host) -> None:
  """Clears the device word (later launches would return at entry while it is set) and raises."""
  code, site, block, step = (int(x) for x in host)
  word.zero_()
  raise _ffi.SplashLibraryError(
      f"splash attention kernel: a kernel gave up waiting (code {code} at wait site {site}, block {block},"
      f" step {step}); outputs of calls since the last check are invalid.  The status word has been"
      " cleared; the call may be repeated.")


def check_device_status(device=None) -> None:
  """Synchronises and raises if a kernel abandoned a bounded wait."""
  lib = _ffi.load()
  for key, word in list(_status_words.items()):
    if device is not None and torch.device(device) != word.device:
      continue
    host = (ctypes.c_int32 * 4)()
    with torch.cuda.device(word.device):
      stream = torch.cuda.current_stream(word.device).cuda_stream
      rc = lib.splash_read_status(word.data_ptr(), ctypes.byref(host), stream)
    _status_mirrors.pop(key, None)
    if rc == _ffi.SPLASH_DEVICE_TIMEOUT:
      _raise_device_status(word, host)
    _ffi.check(rc, "splash attention kernel")


def _poll_status(device) -> None:
  """Start of a call: raises if the copy queued by an earlier call has landed and shows a failure.
  Never waits for the device."""
  mirror = _status_mirrors.get((device.type, device.index))
  if mirror is None or torch.cuda.is_current_stream_capturing():
    return
  host, event = mirror[:2]
  if event.query() and int(host[0]) != 0:
    _status_mirrors.pop((device.type, device.index), None)
    _raise_device_status(_status_word(device), host.tolist())


def _maybe_check(device) -> None:
  """End of a call.  SPLASH_CHECK_STATUS: "1" synchronises and checks now, "0" checks nothing, anything
  else (the default) queues a 16-byte copy of the status word to pinned host memory behind the
  kernels; the next call on this device, or `check_device_status`, looks at it.  The copy runs on a
  stream of its own that waits for the kernels: on the caller's stream it would sit in the copy
  engine's queue behind whatever bulk device-to-host copies the caller has in flight and hold up the
  caller's next kernels until those are done."""
  mode = os.environ.get("SPLASH_CHECK_STATUS", "async")
  if mode == "1":
    check_device_status(device)
    return
  if mode == "0" or torch.cuda.is_current_stream_capturing():
    return
  key = (device.type, device.index)
  mirror = _status_mirrors.get(key)
  if mirror is None:
    mirror = (torch.zeros(4, dtype=torch.int32).pin_memory(), torch.cuda.Event(), torch.cuda.Stream(device),
              torch.cuda.Event())
    _status_mirrors[key] = mirror
  host, event, side, launched = mirror
  launched.record(torch.cuda.current_stream(device))
  side.wait_event(launched)
  with torch.cuda.stream(side):
    host.copy_(_status_word(device), non_blocking=True)
    event.record(side)


class _DeviceSchedule(NamedTuple):
  """Schedule arrays of one tiling, resident on one device."""
  num_steps: torch.Tensor
  order: torch.Tensor
  block_list: torch.Tensor
  block_kind: torch.Tensor
  mask_block: torch.Tensor | None
  partial_blocks: torch.Tensor | None
  mask_desc: torch.Tensor | None
  mask_heads: int
  max_steps: int
  num_partial_blocks: int
  has_partial: bool


def _upload(x, device):
  if x is None:
    return None
  return torch.from_numpy(np.ascontiguousarray(x)).to(device)


def _upload_packed(blocks, device):
  """Dense partial blocks [n, rows, cols] (1 = attend) -> device bytes [n, rows, cols / 8], one bit
  per element, bit i of byte j standing for column 8 * j + i.  The kernels stream these instead of
  the int8 blocks: an eighth of the bytes per partial block and per CTA ring slot."""
  if blocks is None:
    return None
  packed = np.packbits(np.asarray(blocks).astype(bool), axis=-1, bitorder="little")
  return torch.from_numpy(np.ascontiguousarray(packed)).to(device)


def _row_schedule(info: mask_info_lib.GpuMaskInfo, device) -> _DeviceSchedule:
  has_partial = bool((info.block_kind == mask_info_lib.PARTIAL).any())
  dense = info.partial_mask_blocks is not None
  return _DeviceSchedule(
      num_steps=_upload(info.num_steps, device),
      order=_upload(info.q_block_order, device),
      block_list=_upload(info.kv_block, device),
      block_kind=_upload(info.block_kind, device),
      mask_block=_upload(info.mask_block, device) if dense else None,
      partial_blocks=_upload_packed(info.partial_mask_blocks, device) if dense else None,
      mask_desc=(_upload(info.mask_descriptors, device)
                 if (not dense and info.mask_descriptors is not None) else None),
      mask_heads=info.num_steps.shape[0],
      max_steps=info.kv_block.shape[-1],
      num_partial_blocks=0 if not dense else len(info.partial_mask_blocks),
      has_partial=has_partial,
  )


def _column_schedule(info: mask_info_lib.GpuMaskInfo, device) -> _DeviceSchedule:
  has_partial = bool((info.dkv_block_kind == mask_info_lib.PARTIAL).any())
  dense = info.partial_mask_blocks_t is not None
  return _DeviceSchedule(
      num_steps=_upload(info.dkv_num_steps, device),
      order=_upload(info.dkv_kv_block_order, device),
      block_list=_upload(info.dkv_q_block, device),
      block_kind=_upload(info.dkv_block_kind, device),
      mask_block=_upload(info.dkv_mask_block, device) if dense else None,
      partial_blocks=_upload_packed(info.partial_mask_blocks_t, device) if dense else None,
      mask_desc=(_upload(info.mask_descriptors, device)
                 if (not dense and info.mask_descriptors is not None) else None),
      mask_heads=info.dkv_num_steps.shape[0],
      max_steps=info.dkv_q_block.shape[-1],
      num_partial_blocks=0 if not dense else len(info.partial_mask_blocks_t),
      has_partial=has_partial,
  )


def _ptr(t) -> int | None:
  return None if t is None else t.data_ptr()


# ---------------------------------------------------------------------------
# Kernel object
# ---------------------------------------------------------------------------


class SplashAttentionKernel:
  """Callable holding the processed mask.

  Differentiable with respect to q, k and v.  With `save_residuals=True` the
  logsumexp is also returned and that variant is forward-only, as in the
  reference (`splash_attention.py:236-240`).

  `None` fields of `block_sizes` are chosen per call from the head dims, the
  mask and the budgets; schedules are built lazily per tiling and per device,
  the backward schedule only when a gradient is first requested.
  """

  def __init__(self, mask, *, is_mqa: bool, block_sizes: BlockSizes,
               mask_value: float, attn_logits_soft_cap: float | None,
               interpret: Any):
    self.mask = mask
    self.is_mqa = is_mqa
    self.requested_block_sizes = block_sizes
    self.mask_value = mask_value
    self.attn_logits_soft_cap = attn_logits_soft_cap
    self.interpret = interpret
    self._infos: dict = {}
    self._device_schedules: dict = {}

  @property
  def info(self) -> mask_info_lib.GpuMaskInfo:
    """128x128 schedule: backward kernels and FLOP accounting (built on first use)."""
    return self.fwd_info(128, 128)

  def fwd_info(self, block_q: int, block_kv: int) -> mask_info_lib.GpuMaskInfo:
    key = (block_q, block_kv)
    if key not in self._infos:
      self._infos[key] = mask_info_lib.process_mask(self.mask, key)
    return self._infos[key]

  @property
  def pingpong_extra_work(self) -> float | None:
    """Extra KV-block work of the 256-row schedule vs. the 128-row one."""
    if self.mask.shape[-2] % 256:
      return None
    return (float(self.fwd_info(256, 128).num_steps.sum()) * 256
            / max(1.0, float(self.fwd_info(128, 128).num_steps.sum()) * 128))

  def _auto_forward_tiling(self, head_dim: int, head_dim_v: int, *,
                           itemsize: int = 2, has_segments: bool = False,
                           save_residuals: bool = True) -> tuple[int, int, int]:
    """(block_q, block_kv, num_stages) when the caller left block_q open.

    At head_dim 128 the one-tile kernel serves every mask measured on B200 at
    least as well as the two-tile one, in one of two shapes: 64-wide KV blocks
    with a two-stage ring, which leaves room for two CTAs per SM and suits
    short rows (local windows, short sequences), and 128-wide blocks with two
    softmax warpgroups alternating over the KV steps for long rows.  The
    two-tile kernel (block_q=256) runs when asked for, and at head_dim 64 on masks
    whose 256-row schedule costs nothing extra.
    """
    if head_dim == head_dim_v == 64:
      # Measured at seq 8192 (tuning.py): 64-wide KV blocks with a two-stage ring (two CTAs per SM)
      # lead on causal-like masks; the two-tile kernel leads where its 256-row schedule visits no
      # extra blocks (full masks).  With segment ids every tiling is within 2 % of the others.
      extra = self.pingpong_extra_work
      pp = dict(head_dim=head_dim, block_kv=128, num_stages=2, itemsize=itemsize,
                has_dense_mask=self.fwd_info(128, 128).partial_mask_blocks is not None,
                has_segments=has_segments, save_residuals=save_residuals)
      if (extra is not None and extra <= 1.005 and not has_segments
          and cfg.pingpong_smem_bytes(**pp) <= cfg.SMEM_BYTES):
        return 256, 128, 2
      return 128, 64, 2
    if head_dim != head_dim_v or head_dim != 128:
      bkv, stages = auto_forward_tiles(head_dim, 128)
      return 128, bkv, stages
    info = self.fwd_info(128, 128)
    dense = info.partial_mask_blocks is not None
    mean_steps = float(info.num_steps.sum()) / max(1, info.num_steps.size)
    wide = dict(head_dim=head_dim, head_dim_v=head_dim_v, block_kv=128, num_stages=2,
                itemsize=itemsize, has_dense_mask=dense, has_segments=has_segments,
                save_residuals=save_residuals)
    wide_fits = cfg.fwd128_smem_bytes(**wide) <= cfg.SMEM_BYTES
    if (dense or mean_steps >= cfg.AUTO_WIDE_BLOCK_MIN_STEPS) and wide_fits:
      return 128, 128, 2
    return 128, 64, 2

  def choose_block_q(self, head_dim: int, head_dim_v: int, **kw) -> int:
    bs = self.requested_block_sizes
    if bs.block_q is not None:
      return bs.block_q
    return self._auto_forward_tiling(head_dim, head_dim_v, **kw)[0]

  def resolved_block_sizes(self, head_dim: int, head_dim_v: int, **kw) -> BlockSizes:
    bs = self.requested_block_sizes
    if bs.block_q is None:
      bq, bkv, stages = self._auto_forward_tiling(head_dim, head_dim_v, **kw)
    else:
      bq = bs.block_q
      bkv, stages = auto_forward_tiles(head_dim, bq)
    return dataclasses.replace(bs, block_q=bq, block_kv=bs.block_kv or bkv,
                               num_stages=bs.num_stages or stages)

  @property
  def block_sizes(self) -> BlockSizes:
    return self.requested_block_sizes

  # -- device schedules ------------------------------------------------------
  def _fwd_schedule(self, bs: BlockSizes, device) -> _DeviceSchedule:
    key = ("fwd", bs.block_q, bs.block_kv, device.type, device.index)
    if key not in self._device_schedules:
      info = self.fwd_info(bs.block_q, bs.block_kv)
      mask_info_lib.validate_schedule(info)
      self._device_schedules[key] = _row_schedule(info, device)
    return self._device_schedules[key]

  def _bwd_schedules(self, device):
    key = ("bwd", device.type, device.index)
    if key not in self._device_schedules:
      mask_info_lib.validate_schedule(self.info)
      self._device_schedules[key] = (_row_schedule(self.info, device),
                                     _column_schedule(self.info, device))
    return self._device_schedules[key]

  # -- call --------------------------------------------------------------------
  def __call__(self, q, k, v, segment_ids: SegmentIds | None = None, *,
               save_residuals: bool = False):
    if self.interpret is not None:
      raise NotImplementedError(
          "interpret= selects the reference's CPU interpreter; this library"
          " only runs on an sm_100a GPU.")
    bs = self.resolved_block_sizes(
        q.shape[-1], v.shape[-1], itemsize=q.element_size(),
        has_segments=segment_ids is not None)
    return _splash_attention(self, bs, q, k, v, segment_ids,
                             save_residuals=save_residuals)


# ---------------------------------------------------------------------------
# Shape plumbing (reference: `_splash_attention`, splash_attention.py:214-244)
# ---------------------------------------------------------------------------


def _as_segment_tensor(x, batch, device):
  if not isinstance(x, torch.Tensor):
    x = torch.as_tensor(np.asarray(x))
  x = x.to(device=device, dtype=torch.int32)
  if x.ndim == 1:
    x = x.unsqueeze(0).expand(batch, x.shape[0])
  return x.contiguous()


def _splash_attention(kernel: SplashAttentionKernel, bs: BlockSizes, q, k, v,
                      segment_ids, *, save_residuals: bool):
  if not (isinstance(q, torch.Tensor) and isinstance(k, torch.Tensor)
          and isinstance(v, torch.Tensor)):
    raise TypeError("q, k, v must be torch tensors")
  if not q.is_cuda:
    raise RuntimeError(
        "splash attention runs only on a CUDA (sm_100a) device; there is no"
        " CPU path.")
  batched = q.ndim == 4
  if not batched:
    q = q[None]
  if kernel.is_mqa:
    # [(batch,) kv_len, head_dim] -> [batch, 1, kv_len, head_dim]
    k = k.unsqueeze(-3)
    v = v.unsqueeze(-3)
  if k.ndim == 3:
    k, v = k[None], v[None]
  if segment_ids is not None:
    seg_q, seg_kv = segment_ids
    segment_ids = SegmentIds(_as_segment_tensor(seg_q, q.shape[0], q.device),
                             _as_segment_tensor(seg_kv, q.shape[0], q.device))
  if save_residuals:
    out, lse = _forward(kernel, bs, q, k, v, segment_ids, save_residuals=True)
  else:
    seg_q = segment_ids.q if segment_ids is not None else None
    seg_kv = segment_ids.kv if segment_ids is not None else None
    out = _SplashAttentionFn.apply(q, k, v, seg_q, seg_kv, kernel, bs)
    lse = None
  if not batched:
    out = out[0]
    lse = None if lse is None else lse[0]
  return (out, (lse,)) if save_residuals else out


# ---------------------------------------------------------------------------
# Forward
# ---------------------------------------------------------------------------


def _validate_forward(q, k, v, bs: BlockSizes, sched: _DeviceSchedule,
                      segment_ids, save_residuals):
  """Same checks, order and wording as the reference kernels
  (`kernel.py:156-201`, `forward_pingpong.py:155-175`)."""
  batch, num_q_heads, q_seq_len, head_dim = q.shape
  _, num_kv_heads, kv_seq_len, head_dim_v = v.shape
  bq, bkv, num_stages = bs.block_q, bs.block_kv, bs.num_stages
  if tuple(k.shape[:3]) != tuple(v.shape[:3]) or k.shape[0] != batch:
    raise ValueError(f"Incompatible k {tuple(k.shape)} / v {tuple(v.shape)} for q {tuple(q.shape)}")
  if k.shape[-1] != head_dim:
    raise ValueError(f"q and k head dims differ: {head_dim} vs {k.shape[-1]}")
  if num_q_heads % num_kv_heads:
    raise ValueError(f"{num_q_heads=} not a multiple of {num_kv_heads=}")
  if k.dtype != q.dtype or v.dtype != q.dtype:
    raise ValueError(f"q, k, v dtypes differ: {q.dtype}, {k.dtype}, {v.dtype}")
  if q.dtype not in _TORCH_DTYPES:
    raise NotImplementedError(f"Only bf16/f16 are supported, got {q.dtype}")
  has_dense = sched.partial_blocks is not None
  has_segments = segment_ids is not None
  itemsize = q.element_size()
  if bq == cfg.PINGPONG_ROWS:
    if head_dim != head_dim_v:
      raise NotImplementedError("ping-pong kernel needs head_dim == head_dim_v")
    if head_dim % 64 or head_dim > 128:
      raise NotImplementedError(
          f"ping-pong kernel supports head_dim 64/128, got {head_dim}")
    if q_seq_len % bq or kv_seq_len % bkv:
      raise ValueError(f"seq lens must be multiples of ({bq}, {bkv})")
    tmem_cols = cfg.pingpong_tmem_cols(head_dim, bkv)
    if tmem_cols > cfg.TMEM_COLS:
      raise ValueError(f"TMEM budget exceeded ({tmem_cols} > {cfg.TMEM_COLS}); "
                       "use a smaller block_kv")
    smem_bytes = cfg.pingpong_smem_bytes(
        head_dim=head_dim, block_kv=bkv, num_stages=num_stages,
        itemsize=itemsize, has_dense_mask=has_dense, has_segments=has_segments,
        save_residuals=save_residuals)
  else:
    if head_dim % 64 or head_dim_v % 64 or head_dim > 256 or head_dim_v > 256:
      raise NotImplementedError(
          f"head dims must be multiples of 64 and <= 256: {head_dim}, {head_dim_v}")
    if q_seq_len % bq or kv_seq_len % bkv:
      raise ValueError(
          f"Sequence lengths ({q_seq_len}, {kv_seq_len}) must be multiples of"
          f" the block sizes ({bq}, {bkv}).")
    tmem_cols = cfg.fwd128_tmem_cols(head_dim_v, bkv)
    if tmem_cols > cfg.TMEM_COLS:
      raise ValueError(
          f"TMEM budget exceeded ({tmem_cols} > {cfg.TMEM_COLS} columns); use a"
          " smaller block_kv.")
    smem_bytes = cfg.fwd128_smem_bytes(
        head_dim=head_dim, head_dim_v=head_dim_v, block_kv=bkv,
        num_stages=num_stages, itemsize=itemsize, has_dense_mask=has_dense,
        has_segments=has_segments, save_residuals=save_residuals)
  if smem_bytes > cfg.SMEM_BYTES:
    raise ValueError(
        f"Shared memory budget exceeded ({smem_bytes} > {cfg.SMEM_BYTES} bytes);"
        " reduce num_stages or block_kv.")
  if sched.mask_heads not in (1, num_q_heads):
    raise ValueError(f"Mask has {sched.mask_heads} heads, q has {num_q_heads}")
  if sched.num_steps.shape[1] != q_seq_len // bq:
    raise ValueError("Mask info does not match the q sequence length")


def _base_params(kernel: SplashAttentionKernel, q, k, v, segment_ids,
                 sched: _DeviceSchedule) -> _ffi.SplashParams:
  p = _ffi.SplashParams()
  p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
  if segment_ids is not None:
    p.seg_q, p.seg_kv = segment_ids.q.data_ptr(), segment_ids.kv.data_ptr()
  p.num_steps = sched.num_steps.data_ptr()
  p.block_order = sched.order.data_ptr()
  p.block_list = sched.block_list.data_ptr()
  p.block_kind = sched.block_kind.data_ptr()
  p.mask_block = _ptr(sched.mask_block)
  p.partial_blocks = _ptr(sched.partial_blocks)
  p.mask_desc = _ptr(sched.mask_desc) if sched.has_partial else None
  p.status = _status_word(q.device).data_ptr()
  p.batch, p.heads, p.q_len, p.head_dim = q.shape
  p.kv_heads, p.kv_len, p.head_dim_v = v.shape[1], v.shape[2], v.shape[3]
  p.dtype = _TORCH_DTYPES[q.dtype]
  p.mask_heads = sched.mask_heads
  p.max_steps = sched.max_steps
  p.num_partial_blocks = sched.num_partial_blocks
  p.mask_value = kernel.mask_value
  cap = kernel.attn_logits_soft_cap
  p.soft_cap = 0.0 if cap is None else float(cap)
  if segment_ids is not None and os.environ.get("SPLASH_SEG_SKIP", "1") == "1":
    # Scratch for segment-aware block skipping: the entry point fills it and the kernels leave out
    # blocks whose q and kv segment ids cannot meet.  (Freed after the launch; the caching allocator
    # reuses it only behind the kernels on this stream.)
    nbytes = int(_ffi.load().splash_seg_ranges_bytes(ctypes.byref(p)))
    if nbytes > 0:
      p._seg_ranges = torch.empty(nbytes // 4, dtype=torch.int32, device=q.device)
      p.seg_ranges = p._seg_ranges.data_ptr()
  return p


def _forward(kernel: SplashAttentionKernel, bs: BlockSizes, q, k, v,
             segment_ids, *, save_residuals: bool):
  """Runs one forward kernel; returns (out, lse or None)."""
  lib = _ffi.load()
  _poll_status(q.device)
  sched = kernel._fwd_schedule(bs, q.device)
  _validate_forward(q, k, v, bs, sched, segment_ids, save_residuals)
  q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
  batch, heads, q_len, _ = q.shape
  out = torch.empty((batch, heads, q_len, v.shape[-1]), dtype=q.dtype,
                    device=q.device)
  lse = (torch.empty((batch, heads, q_len), dtype=torch.float32, device=q.device)
         if save_residuals else None)
  p = _base_params(kernel, q, k, v, segment_ids, sched)
  p.out, p.lse_out = out.data_ptr(), _ptr(lse)
  p.block_q, p.block_kv, p.num_stages = bs.block_q, bs.block_kv, bs.num_stages
  with torch.cuda.device(q.device):
    stream = torch.cuda.current_stream(q.device).cuda_stream
    entry = lib.splash_fwd256 if bs.block_q == cfg.PINGPONG_ROWS else lib.splash_fwd128
    _ffi.check(entry(ctypes.byref(p), stream), "splash attention forward")
  _maybe_check(q.device)
  return out, lse


# ---------------------------------------------------------------------------
# Backward (reference: `_attention_bwd`, splash_attention.py:286-329)
# ---------------------------------------------------------------------------


def _use_fused_backward(q, v, bs: BlockSizes, has_dense, has_segments) -> bool:
  head_dim = q.shape[-1]
  # Head dims 64 and 128.  SPLASH_BWD_FUSED=0 forces the split kernels at any head
  # dim, SPLASH_BWD_FUSED_D64=0 at head_dim 64 only (the reference makes the fused
  # path opt-in there because its version is slower, `splash_attention.py:299-301`;
  # here it is the faster one and on by default).
  use = head_dim == 128 or (head_dim == 64
                            and os.environ.get("SPLASH_BWD_FUSED_D64", "1") == "1")
  return bool(
      use and cfg.fused_supported(head_dim, v.shape[-1])
      and cfg.fused_fits(head_dim=head_dim, num_stages=bs.num_stages_bwd,
                         itemsize=q.element_size(), has_dense_mask=has_dense,
                         has_segments=has_segments)
      and os.environ.get("SPLASH_BWD_FUSED", "1") == "1")


def _backward(kernel: SplashAttentionKernel, bs: BlockSizes, q, k, v,
              segment_ids, out, lse, d_out):
  lib = _ffi.load()
  for name in ("splash_bwd_delta", "splash_bwd_dq", "splash_bwd_dkv",
               "splash_bwd_fused"):
    if not hasattr(lib, name):
      raise _ffi.SplashLibraryError(f"{_ffi.LIB_NAME} does not export {name}")
  _poll_status(q.device)
  rows, cols = kernel._bwd_schedules(q.device)
  d_out = d_out.to(q.dtype).contiguous()
  batch, heads, q_len, head_dim = q.shape
  head_dim_v = v.shape[-1]
  if q_len % 128 or k.shape[2] % 128:
    raise ValueError(
        f"Sequence lengths ({q_len}, {k.shape[2]}) must be multiples of 128"
        " for the backward pass.")
  has_dense = rows.partial_blocks is not None
  has_segments = segment_ids is not None
  itemsize = q.element_size()
  delta = torch.empty((batch, heads, q_len), dtype=torch.float32, device=q.device)
  dq = torch.empty_like(q)
  dk = torch.empty_like(k)
  dv = torch.empty_like(v)
  fused = _use_fused_backward(q, v, bs, has_dense, has_segments)
  with torch.cuda.device(q.device):
    stream = torch.cuda.current_stream(q.device).cuda_stream
    if not fused:
      _ffi.check(lib.splash_bwd_delta(out.data_ptr(), d_out.data_ptr(),
                                      delta.data_ptr(), batch * heads * q_len,
                                      head_dim_v, _TORCH_DTYPES[q.dtype], stream),
                 "splash attention delta")

    def params(sched):
      p = _base_params(kernel, q, k, v, segment_ids, sched)
      p.d_out, p.lse, p.delta = d_out.data_ptr(), lse.data_ptr(), delta.data_ptr()
      p.dq, p.dk, p.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
      p.block_q, p.block_kv = 128, 128  # the backward schedule is always 128x128
      p.num_stages = bs.num_stages_bwd
      return p

    if fused:
      p = params(cols)
      p.out = out.data_ptr()  # delta is computed in the pass that clears the accumulator
      nbytes = lib.splash_bwd_fused_workspace_bytes(ctypes.byref(p))
      acc = torch.empty(max(int(nbytes), 4) // 4, dtype=torch.float32,
                        device=q.device)
      p.dq_acc = acc.data_ptr()
      _ffi.check(lib.splash_bwd_fused(ctypes.byref(p), stream),
                 "splash attention fused backward")
    else:
      def pick(requested, tmem_fn, smem_fn, name):
        sb = requested or cfg.largest_fitting_sub_block(tmem_fn, smem_fn) or 64
        tmem_cols, smem_bytes = tmem_fn(sb), smem_fn(sb)
        if tmem_cols > cfg.TMEM_COLS:
          raise ValueError(
              f"{name}: TMEM budget exceeded ({tmem_cols} > {cfg.TMEM_COLS} columns)."
              " The backward pass supports head dims up to 128.")
        if smem_bytes > cfg.SMEM_BYTES:
          raise ValueError(
              f"{name}: shared memory budget exceeded ({smem_bytes} >"
              f" {cfg.SMEM_BYTES} bytes); reduce num_stages or the sub-block sizes.")
        return sb

      common = dict(num_stages=bs.num_stages_bwd, itemsize=itemsize,
                    has_dense_mask=has_dense, has_segments=has_segments)
      p = params(rows)
      p.sub_block = pick(
          bs.block_kv_dq,
          lambda sb: cfg.bwd_dq_tmem_cols(head_dim, sb),
          lambda sb: cfg.bwd_dq_smem_bytes(head_dim=head_dim, head_dim_v=head_dim_v,
                                           sub_block=sb, **common),
          "dQ kernel")
      _ffi.check(lib.splash_bwd_dq(ctypes.byref(p), stream),
                 "splash attention dQ")
      p = params(cols)
      # The dK/dV kernel always works in 64-row steps; `block_q_dkv` is accepted for compatibility
      # with the reference's BlockSizes, and the budgets are checked for the tiling that runs.
      p.sub_block = pick(
          64,
          lambda sb: cfg.bwd_dkv_tmem_cols(head_dim, head_dim_v, sb),
          lambda sb: cfg.bwd_dkv_smem_bytes(head_dim=head_dim, head_dim_v=head_dim_v,
                                            sub_block=sb, **common),
          "dKV kernel")
      _ffi.check(lib.splash_bwd_dkv(ctypes.byref(p), stream),
                 "splash attention dK/dV")
  _maybe_check(q.device)
  return dq, dk, dv


class _SplashAttentionFn(torch.autograd.Function):
  """Custom VJP: forward saves (q, k, v, out, lse); backward runs the dQ/dK/dV kernels."""

  @staticmethod
  def forward(ctx, q, k, v, seg_q, seg_kv, kernel, bs):
    segment_ids = None if seg_q is None else SegmentIds(seg_q, seg_kv)
    need_grad = any(ctx.needs_input_grad[:3])
    out, lse = _forward(kernel, bs, q, k, v, segment_ids,
                        save_residuals=need_grad)
    if need_grad:
      ctx.save_for_backward(q, k, v, out, lse, *(() if seg_q is None else (seg_q, seg_kv)))
      ctx.kernel, ctx.bs = kernel, bs
    return out

  @staticmethod
  def backward(ctx, d_out):
    saved = ctx.saved_tensors
    q, k, v, out, lse = saved[:5]
    segment_ids = SegmentIds(saved[5], saved[6]) if len(saved) > 5 else None
    dq, dk, dv = _backward(ctx.kernel, ctx.bs, q.contiguous(), k.contiguous(),
                           v.contiguous(), segment_ids, out, lse, d_out)
    return dq, dk, dv, None, None, None, None


# ---------------------------------------------------------------------------
# Constructors
# ---------------------------------------------------------------------------


def _make_splash_attention(
    mask,
    *,
    is_mqa: bool,
    block_sizes: BlockSizes | None = None,
    mask_value: float = DEFAULT_MASK_VALUE,
    attn_logits_soft_cap: float | None = None,
    interpret: Any = None,
) -> SplashAttentionKernel:
  if block_sizes is None:
    block_sizes = BlockSizes()
  if isinstance(mask, np.ndarray):
    if mask.ndim == 2:
      mask = mask[None]
    mask = mask_lib.MultiHeadMask([mask_lib.NumpyMask(m) for m in mask])
  return SplashAttentionKernel(
      mask,
      is_mqa=is_mqa,
      block_sizes=block_sizes,
      mask_value=mask_value,
      attn_logits_soft_cap=attn_logits_soft_cap,
      interpret=interpret,
  )


make_splash_mha = functools.partial(_make_splash_attention, is_mqa=False)
make_splash_mqa = functools.partial(_make_splash_attention, is_mqa=True)


def attention_reference(
    mask,  # bool[heads or 1, q_len, kv_len], numpy or torch
    q, k, v,
    segment_ids: SegmentIds | None = None,
    *,
    is_mqa: bool = False,
    mask_value: float = DEFAULT_MASK_VALUE,
    attn_logits_soft_cap: float | None = None,
    save_residuals: bool = False,
):
  """Dense f32 masked attention on the tensors' own device, in plain torch ops.

  Same operation order as the reference's `attention_reference`
  (`splash_attention.py:366-407`).  It materialises the [heads, q, kv] logits,
  so it is meant for checking small problems, not for production use; the
  kernels never call it.
  """
  batched = q.ndim == 4
  if not batched:
    q, k, v = q[None], k[None], v[None]
  if is_mqa:
    k, v = k[:, None], v[:, None]
  q, k, v = (x.to(torch.float32) for x in (q, k, v))
  rep = q.shape[1] // k.shape[1]
  k = k.repeat_interleave(rep, dim=1)
  v = v.repeat_interleave(rep, dim=1)
  logits = torch.einsum("bhqd,bhkd->bhqk", q, k)
  if attn_logits_soft_cap is not None:
    logits = torch.tanh(logits / attn_logits_soft_cap) * attn_logits_soft_cap
  full_mask = torch.as_tensor(np.asarray(mask) if not isinstance(mask, torch.Tensor)
                              else mask).to(device=q.device, dtype=torch.bool)
  full_mask = full_mask[None].expand(logits.shape)
  if segment_ids is not None:
    seg_q, seg_kv = (torch.as_tensor(np.asarray(s) if not isinstance(s, torch.Tensor) else s)
                     .to(q.device) for s in segment_ids)
    seg_q = seg_q.expand(q.shape[0], q.shape[2])
    seg_kv = seg_kv.expand(q.shape[0], k.shape[2])
    full_mask = full_mask & (seg_q[:, None, :, None] == seg_kv[:, None, None, :])
  logits = torch.where(full_mask, logits, torch.tensor(mask_value, device=q.device))
  m = logits.max(dim=-1, keepdim=True).values
  p = torch.exp(logits - m)
  l = p.sum(dim=-1, keepdim=True)
  out = torch.einsum("bhqk,bhkd->bhqd", p / l, v)
  lse = (torch.log(l) + m)[..., 0]
  if not batched:
    out, lse = out[0], lse[0]
  return (out, (lse,)) if save_residuals else out
