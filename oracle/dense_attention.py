"""CPU oracle for splash attention: dense f32 masked softmax attention and its gradients.

TEST INFRASTRUCTURE ONLY.  Imported by `tests/`, by `__graft_entry__.smoke()` and by
the CPU-baseline legs of `bench.py`; the product package never imports it.

What it restates
  * forward + logsumexp: the reference's `attention_reference`
    (splash_attention_mgpu/splash_attention.py:366-407) -- f32 casts, Q K^T,
    soft-cap, mask AND segment mask, `where(mask, logits, mask_value)`, stable
    softmax, P V, `lse = log(l) + m`, in that order;
  * gradients: the closed form the reference's backward kernels implement
    (splash_attention_mgpu/backward.py:66-84 and the reference test's
    `jax.grad` of the dense function, tests/test_splash_attention_mgpu.py:371-390):
    P = exp(S - lse), dV = P^T dO, dP = dO V^T, delta = rowsum(dO * O),
    dS = P * (dP - delta) [* (1 - tanh^2(S_raw / cap))], dQ = dS K, dK = dS^T Q,
    with dK/dV summed over the q heads that share a KV head.

PARITY UNPINNED: the reference ships no golden vectors, and neither its kernels nor
its own dense function can run here (JAX is not installed).  This file is checked
against an independent implementation (`torch.nn.functional.scaled_dot_product_attention`
with an explicit mask, and torch autograd through the forward) in tests/test_oracle.py.

Work is tiled per (batch, head) so the [q_len, kv_len] logits never exceed one
head's worth of memory.
"""

from __future__ import annotations

import numpy as np
import torch

DEFAULT_MASK_VALUE = -0.7 * float(np.finfo(np.float32).max)


def _to_f32(x) -> torch.Tensor:
  if isinstance(x, torch.Tensor):
    return x.detach().to(device="cpu", dtype=torch.float32)
  return torch.from_numpy(np.asarray(x, dtype=np.float32))


def _normalise(q, k, v, is_mqa):
  q, k, v = _to_f32(q), _to_f32(k), _to_f32(v)
  batched = q.ndim == 4
  if not batched:
    q, k, v = q[None], k[None], v[None]
  if is_mqa:
    k, v = k[:, None], v[:, None]
  return q, k, v, batched


def _head_mask(mask, h):
  mask = np.asarray(mask)
  if mask.ndim == 2:
    return mask
  return mask[h if mask.shape[0] > 1 else 0]


def _segment_mask(segment_ids, b, q_len, kv_len):
  if segment_ids is None:
    return None
  seg_q, seg_kv = (np.asarray(s.cpu() if isinstance(s, torch.Tensor) else s)
                   for s in segment_ids)
  seg_q = seg_q if seg_q.ndim == 1 else seg_q[b]
  seg_kv = seg_kv if seg_kv.ndim == 1 else seg_kv[b]
  return seg_q[:, None] == seg_kv[None, :]


def attention_forward(mask, q, k, v, segment_ids=None, *, is_mqa=False,
                      mask_value=DEFAULT_MASK_VALUE, attn_logits_soft_cap=None,
                      heads=None):
  """Returns (out f32 [.., heads, q, dv], lse f32 [.., heads, q]) as numpy arrays.

  `heads`: optional iterable of q-head indices to evaluate (others stay zero);
  used by the benchmark's bounded CPU sample.
  """
  q, k, v, batched = _normalise(q, k, v, is_mqa)
  batch, num_heads, q_len, _ = q.shape
  kv_heads, kv_len = k.shape[1], k.shape[2]
  rep = num_heads // kv_heads
  out = torch.zeros((batch, num_heads, q_len, v.shape[-1]), dtype=torch.float32)
  lse = torch.zeros((batch, num_heads, q_len), dtype=torch.float32)
  head_list = range(num_heads) if heads is None else heads
  for b in range(batch):
    seg = _segment_mask(segment_ids, b, q_len, kv_len)
    for h in head_list:
      logits = q[b, h] @ k[b, h // rep].T
      if attn_logits_soft_cap is not None:
        logits = torch.tanh(logits / attn_logits_soft_cap) * attn_logits_soft_cap
      vis = _head_mask(mask, h)
      if seg is not None:
        vis = vis & seg
      logits = torch.where(torch.from_numpy(np.ascontiguousarray(vis)), logits,
                           torch.tensor(mask_value, dtype=torch.float32))
      m = logits.max(dim=-1, keepdim=True).values
      p = torch.exp(logits - m)
      l = p.sum(dim=-1, keepdim=True)
      out[b, h] = (p / l) @ v[b, h // rep]
      lse[b, h] = (torch.log(l) + m)[:, 0]
  if not batched:
    out, lse = out[0], lse[0]
  return out.numpy(), lse.numpy()


def attention_backward(mask, q, k, v, d_out, segment_ids=None, *, is_mqa=False,
                       mask_value=DEFAULT_MASK_VALUE, attn_logits_soft_cap=None):
  """Analytic gradients (dq, dk, dv) of sum(out * d_out), as f32 numpy arrays shaped like q, k, v."""
  qf, kf, vf, batched = _normalise(q, k, v, is_mqa)
  do = _to_f32(d_out)
  if not batched:
    do = do[None]
  batch, num_heads, q_len, _ = qf.shape
  kv_heads, kv_len = kf.shape[1], kf.shape[2]
  rep = num_heads // kv_heads
  dq = torch.zeros_like(qf)
  dk = torch.zeros_like(kf)
  dv = torch.zeros_like(vf)
  for b in range(batch):
    seg = _segment_mask(segment_ids, b, q_len, kv_len)
    for h in range(num_heads):
      g = h // rep
      raw = qf[b, h] @ kf[b, g].T
      if attn_logits_soft_cap is not None:
        t = torch.tanh(raw / attn_logits_soft_cap)
        logits = t * attn_logits_soft_cap
      else:
        logits = raw
      vis = _head_mask(mask, h)
      if seg is not None:
        vis = vis & seg
      vis_t = torch.from_numpy(np.ascontiguousarray(vis))
      logits = torch.where(vis_t, logits, torch.tensor(mask_value, dtype=torch.float32))
      m = logits.max(dim=-1, keepdim=True).values
      p = torch.exp(logits - m)
      p = p / p.sum(dim=-1, keepdim=True)
      o = p @ vf[b, g]
      dv[b, g] += p.T @ do[b, h]
      dp = do[b, h] @ vf[b, g].T
      delta = (do[b, h] * o).sum(dim=-1, keepdim=True)
      ds = p * (dp - delta)
      # Masked logits are the constant mask_value: no gradient flows through them.
      ds = torch.where(vis_t, ds, torch.zeros((), dtype=torch.float32))
      if attn_logits_soft_cap is not None:
        ds = ds * (1.0 - t * t)
      dq[b, h] = ds @ kf[b, g]
      dk[b, g] += ds.T @ qf[b, h]
  if is_mqa:
    dk, dv = dk[:, 0], dv[:, 0]
  if not batched:
    dq, dk, dv = dq[0], dk[0], dv[0]
  return dq.numpy(), dk.numpy(), dv.numpy()


def visible_rows(mask, segment_ids=None, batch=None):
  """bool[(batch,) heads or 1, q_len]: rows that see at least one key.

  Rows that see none are implementation-defined in the reference
  (tools/fuzz.py:116-124 excludes them from comparison); tests use this to do
  the same.
  """
  mask = np.asarray(mask)
  if mask.ndim == 2:
    mask = mask[None]
  if segment_ids is None:
    return mask.any(axis=-1)
  seg_q, seg_kv = (np.asarray(s.cpu() if isinstance(s, torch.Tensor) else s)
                   for s in segment_ids)
  if seg_q.ndim == 1:
    seg_q, seg_kv = seg_q[None], seg_kv[None]
  same = seg_q[:, None, :, None] == seg_kv[:, None, None, :]
  return (mask[None] & same).any(axis=-1)
