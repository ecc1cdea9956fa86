"""Partition of splash attention across the GPUs of one box.

The unit of work is one (batch index, KV head) pair together with the q heads of
its group: the forward needs only that KV head's K/V, and dK/dV are reduced over
the group inside one CTA, so units never exchange data.  The reference has no
distributed code at all (it farms independent jobs to GPUs,
tools/gpu_farm.py:148-156); this module is what a multi-GPU caller of the
library uses instead.  There is no collective on the data path: `all_gather`
appears only in `gather_units`, which exists for checking results.

Ranks own contiguous slices of the flattened (batch x kv_head) index.  A slice is
presented to the kernel as a batch of single-KV-head problems
([units, group, q_len, d] / [units, 1, kv_len, d]), which is valid whenever all
heads share one mask; per-head masks are partitioned by batch index only.
"""

from __future__ import annotations

import torch


def unit_range(num_units: int, world: int, rank: int) -> tuple[int, int]:
  """Contiguous [lo, hi) slice of `num_units` for `rank`; sizes differ by at most one."""
  base, extra = divmod(num_units, world)
  lo = rank * base + min(rank, extra)
  return lo, lo + base + (1 if rank < extra else 0)


def to_units(q, k, v, segment_ids=None):
  """[B,H,S,D], [B,KVH,S,D] -> unit-major views [B*KVH, G, S, D], [B*KVH, 1, S, D]."""
  batch, heads, q_len, d = q.shape
  kv_heads = k.shape[1]
  group = heads // kv_heads
  qu = q.reshape(batch, kv_heads, group, q_len, d).reshape(batch * kv_heads, group, q_len, d)
  ku = k.reshape(batch * kv_heads, 1, k.shape[2], k.shape[3])
  vu = v.reshape(batch * kv_heads, 1, v.shape[2], v.shape[3])
  seg = None
  if segment_ids is not None:
    seg_q, seg_kv = segment_ids
    if seg_q.ndim == 1:
      seg_q = seg_q[None].expand(batch, -1)
      seg_kv = seg_kv[None].expand(batch, -1)
    seg = (seg_q.repeat_interleave(kv_heads, dim=0), seg_kv.repeat_interleave(kv_heads, dim=0))
  return qu, ku, vu, seg


def local_units(q, k, v, segment_ids, world: int, rank: int):
  """This rank's slice of the unit-major problem (may be empty when world > units)."""
  qu, ku, vu, seg = to_units(q, k, v, segment_ids)
  lo, hi = unit_range(qu.shape[0], world, rank)
  seg_local = None if seg is None else (seg[0][lo:hi].contiguous(), seg[1][lo:hi].contiguous())
  return qu[lo:hi].contiguous(), ku[lo:hi].contiguous(), vu[lo:hi].contiguous(), seg_local, (lo, hi)


def run_local(fn, q, k, v, segment_ids=None, *, world: int, rank: int):
  """Runs `fn(q_units, k_units, v_units, segment_ids)` on this rank's units.

  `fn` is a SplashAttentionKernel built with a shared (single-head) mask, or any
  callable with that signature.  Returns (local_out [units, G, S, Dv], (lo, hi)).
  """
  ql, kl, vl, seg, span = local_units(q, k, v, segment_ids, world, rank)
  if ql.shape[0] == 0:
    return ql.new_zeros((0,) + tuple(ql.shape[1:3]) + (v.shape[-1],)), span
  out = fn(ql, kl, vl, seg) if seg is not None else fn(ql, kl, vl)
  return out, span


def run_local_grads(fn, q, k, v, d_out, segment_ids=None, *, world: int, rank: int):
  """Forward and backward of this rank's units: `fn` as for `run_local`, `d_out` like the
  forward output.  Returns ((out, dq, dk, dv) in unit-major layout, (lo, hi)); nothing
  crosses ranks, dK/dV of a unit are complete on the rank that owns it.
  """
  ql, kl, vl, seg, span = local_units(q, k, v, segment_ids, world, rank)
  lo, hi = span
  dol = to_units(d_out, k, v)[0][lo:hi].contiguous()
  if ql.shape[0] == 0:
    empty_out = ql.new_zeros((0,) + tuple(ql.shape[1:3]) + (v.shape[-1],))
    return (empty_out, torch.zeros_like(ql), torch.zeros_like(kl), torch.zeros_like(vl)), span
  ql, kl, vl = (x.detach().requires_grad_(True) for x in (ql, kl, vl))
  out = fn(ql, kl, vl, seg) if seg is not None else fn(ql, kl, vl)
  out.backward(dol)
  return (out.detach(), ql.grad, kl.grad, vl.grad), span


def gather_units(local_out, span, full_shape, group=None):
  """All-gathers per-rank unit outputs into the full [B, H, S, Dv] tensor (for checking only)."""
  import torch.distributed as dist
  world = dist.get_world_size(group)
  batch, heads, q_len, dv = full_shape
  spans = [None] * world
  dist.all_gather_object(spans, span, group=group)
  max_units = max(hi - lo for lo, hi in spans)
  grp = local_out.shape[1] if local_out.shape[0] else None
  grps = [None] * world
  dist.all_gather_object(grps, grp, group=group)
  grp = next(g for g in grps if g is not None)
  pad = local_out.new_zeros((max_units, grp, q_len, dv))
  pad[: local_out.shape[0]] = local_out
  parts = [torch.empty_like(pad) for _ in range(world)]
  dist.all_gather(parts, pad, group=group)
  units = torch.cat([p[: hi - lo] for p, (lo, hi) in zip(parts, spans)], dim=0)
  return units.reshape(batch, heads // grp, grp, q_len, dv).reshape(batch, heads, q_len, dv)
