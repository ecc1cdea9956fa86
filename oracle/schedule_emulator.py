"""CPU emulator of the forward kernels' block schedule and arithmetic order.

TEST INFRASTRUCTURE ONLY (see oracle/dense_attention.py for the rules).

It walks the schedule arrays of a `GpuMaskInfo` exactly as a CTA does -- q blocks
in `q_block_order`, `num_steps` visited KV blocks from `kv_block`, FULL blocks
unmasked, PARTIAL blocks masked from the dense int8 block or the band descriptor --
and applies the kernels' numerics: running maximum kept stale until it moves by
more than 2^8 (reference splash_attention_mgpu/kernel.py:396-428), P rounded to
the 16-bit input type before P V, f32 accumulation, `lse = m + log(l)`, zeros and
`lse = mask_value` for rows that never see a key (kernel.py:446-452).

A schedule bug (wrong block list, wrong kind, wrong mask-block id, wrong
descriptor) therefore shows up on the CPU as a mismatch against the dense oracle,
without a GPU.
"""

from __future__ import annotations

import numpy as np
import torch

FULL = 2
PARTIAL = 1
RESCALE_THRESHOLD = 8.0
LOG2E = 1.4426950408889634


def _round_to(x: np.ndarray, dtype: torch.dtype) -> np.ndarray:
  return torch.from_numpy(np.ascontiguousarray(x)).to(dtype).to(torch.float32).numpy()


def emulate_forward(info, q, k, v, segment_ids=None, *, mask_value,
                    attn_logits_soft_cap=None, dtype=torch.bfloat16):
  """q: [heads, q_len, d]; k, v: [kv_heads, kv_len, d] (numpy or torch, any float type).

  Returns (out f32 [heads, q_len, dv], lse f32 [heads, q_len]).
  """
  to_np = lambda x: (x.detach().cpu().to(torch.float32).numpy()
                     if isinstance(x, torch.Tensor) else np.asarray(x, np.float32))
  q, k, v = to_np(q), to_np(k), to_np(v)
  heads, q_len, _ = q.shape
  kv_heads = k.shape[0]
  rep = heads // kv_heads
  bq, bkv = info.block_q, info.block_kv
  out = np.zeros((heads, q_len, v.shape[-1]), np.float32)
  lse = np.zeros((heads, q_len), np.float32)
  seg_q = seg_kv = None
  if segment_ids is not None:
    seg_q, seg_kv = (np.asarray(s) for s in segment_ids)
  mask_heads = info.num_steps.shape[0]
  for h in range(heads):
    mh = h if mask_heads > 1 else 0
    for qi in info.q_block_order[mh]:
      rows = slice(qi * bq, (qi + 1) * bq)
      n = int(info.num_steps[mh, qi])
      m_run = np.full((bq,), -np.inf, np.float32)
      l_run = np.zeros((bq,), np.float32)
      acc = np.zeros((bq, v.shape[-1]), np.float32)
      for s in range(n):
        j = int(info.kv_block[mh, qi, s])
        cols = slice(j * bkv, (j + 1) * bkv)
        logits = q[h, rows] @ k[h // rep, cols].T
        if attn_logits_soft_cap is not None:
          logits = np.tanh(logits / attn_logits_soft_cap) * attn_logits_soft_cap
        vis = np.ones((bq, bkv), bool)
        if info.block_kind[mh, qi, s] == PARTIAL:
          if info.partial_mask_blocks is not None:
            vis &= info.partial_mask_blocks[info.mask_block[mh, qi, s]].astype(bool)
          else:
            lo, hi, chunk, _ = info.mask_descriptors[mh]
            qp = np.arange(qi * bq, (qi + 1) * bq)[:, None]
            kp = np.arange(j * bkv, (j + 1) * bkv)[None, :]
            vis &= (kp - qp >= lo) & (kp - qp <= hi)
            if chunk:
              vis &= (qp // chunk) == (kp // chunk)
        else:
          assert info.block_kind[mh, qi, s] == FULL
        if seg_q is not None:
          vis &= seg_q[rows][:, None] == seg_kv[cols][None, :]
        logits = np.where(vis, logits, -np.inf).astype(np.float32)
        m_new = np.maximum(m_run, logits.max(axis=-1))
        with np.errstate(invalid="ignore"):
          moved = (m_new - m_run) * LOG2E > RESCALE_THRESHOLD
        with np.errstate(invalid="ignore"):
          alpha = np.where(moved, np.exp2((m_run - m_new) * LOG2E), 1.0).astype(np.float32)
        alpha = np.where(np.isnan(alpha), 0.0, alpha)
        m_run = np.where(moved, m_new, m_run)
        l_run = l_run * alpha
        acc = acc * alpha[:, None]
        base = np.where(np.isinf(m_run), 0.0, m_run)
        p = np.exp2((logits - base[:, None]) * LOG2E).astype(np.float32)
        l_run = l_run + p.sum(axis=-1)
        acc = acc + _round_to(p, dtype) @ _round_to(v[h // rep, cols], dtype)
      seen = l_run > 0
      safe_l = np.where(seen, l_run, 1.0)
      out[h, rows] = np.where(seen[:, None], acc / safe_l[:, None], 0.0)
      lse[h, rows] = np.where(seen, np.where(seen, m_run, 0.0) + np.log(safe_l),
                              np.float32(mask_value))
  return out, lse
