"""Tile sweeps and a same-GPU library comparator for the splash attention kernels.

The reference keeps three scripts for this: `tools/sweep.py:28-44` (time a grid of
block sizes), `tools/summarize.py:17-37` (tabulate the results) and
`tools/baseline.py:22-42` (time a vendor attention on the same device).  Here they
are functions of the package plus a small command line:

  python -m splash_attention_mgpu.tuning --mask causal --seq 8192 --heads 16 --batch 2

Everything below times with CUDA events on the current stream after warm-up and
reports the median.  Nothing here is on the product path: the kernels never call
into this module, and the defaults in `config.py` are plain constants.
"""

from __future__ import annotations

import argparse
import dataclasses
import itertools
import json
from typing import Callable, Iterable, Sequence

import torch

from . import splash_attention as splash
from . import splash_attention_mask as mask_lib
from .config import BlockSizes


@dataclasses.dataclass
class Timing:
  """One timed configuration. `ms` is None when the configuration was rejected."""
  label: str
  block_sizes: BlockSizes | None
  fwd_ms: float | None
  bwd_ms: float | None = None
  error: str | None = None

  def tflops(self, fwd_flops: float) -> tuple[float | None, float | None]:
    f = fwd_flops / (self.fwd_ms * 1e9) if self.fwd_ms else None
    b = 2.5 * fwd_flops / (self.bwd_ms * 1e9) if self.bwd_ms else None
    return f, b


def time_cuda(fn: Callable[[], object], *, iters: int = 10, warmup: int = 3) -> float:
  """Median milliseconds of `fn` over `iters` runs, timed with CUDA events."""
  for _ in range(warmup):
    fn()
  torch.cuda.synchronize()
  events = [torch.cuda.Event(enable_timing=True) for _ in range(iters + 1)]
  events[0].record()
  for i in range(iters):
    fn()
    events[i + 1].record()
  torch.cuda.synchronize()
  times = sorted(events[i].elapsed_time(events[i + 1]) for i in range(iters))
  return times[len(times) // 2]


def forward_candidates(head_dim: int) -> list[BlockSizes]:
  """The forward tilings worth timing for a head dim: both kernels, both KV block
  widths, ring depths that can fit."""
  out = []
  for bq, bkv, stages in itertools.product((128, 256), (64, 128), (2, 3, 4)):
    if bq == 256 and head_dim > 128:
      continue
    out.append(BlockSizes(block_q=bq, block_kv=bkv, num_stages=stages))
  return out


def backward_candidates() -> list[BlockSizes]:
  """Ring depths of the backward kernels and the split kernels' sub-block sizes."""
  out = [BlockSizes(num_stages_bwd=s) for s in (2, 3)]
  out += [BlockSizes(num_stages_bwd=2, block_kv_dq=sb, block_q_dkv=sb) for sb in (64, 128)]
  return out


def useful_forward_flops(kernel, heads: int, batch: int, head_dim: int) -> float:
  """4 * visible 128x128 blocks * 128 * 128 * head_dim (reference tools/bench.py:86-89)."""
  info = kernel.info
  visible = float(info.num_steps.sum()) * (heads if info.num_steps.shape[0] == 1 else 1) * batch
  return 4.0 * visible * 128 * 128 * head_dim


def sweep(mask, q, k, v, d_out=None, *, segment_ids=None, attn_logits_soft_cap=None,
          is_mqa: bool = False, candidates: Iterable[BlockSizes] | None = None,
          iters: int = 10) -> list[Timing]:
  """Times the forward (and the backward when `d_out` is given) for each candidate.

  Candidates the kernels reject (budgets, divisibility) are kept in the result with
  their error text, the way the reference's sweep records failures.
  """
  make = splash.make_splash_mqa if is_mqa else splash.make_splash_mha
  if candidates is None:
    candidates = forward_candidates(q.shape[-1])
  results = []
  for bs in candidates:
    label = (f"bq={bs.block_q} bkv={bs.block_kv} stages={bs.num_stages} "
             f"bwd_stages={bs.num_stages_bwd} dq_sb={bs.block_kv_dq} dkv_sb={bs.block_q_dkv}")
    try:
      kernel = make(mask, block_sizes=bs, attn_logits_soft_cap=attn_logits_soft_cap)
      fwd_ms = time_cuda(lambda: kernel(q, k, v, segment_ids, save_residuals=True), iters=iters)
      bwd_ms = None
      if d_out is not None:
        qg, kg, vg = (x.detach().clone().requires_grad_(True) for x in (q, k, v))

        def both():
          qg.grad = kg.grad = vg.grad = None
          kernel(qg, kg, vg, segment_ids).backward(d_out)

        bwd_ms = max(time_cuda(both, iters=iters) - fwd_ms, 0.0)
      splash.check_device_status()
      results.append(Timing(label, bs, fwd_ms, bwd_ms))
    except (ValueError, NotImplementedError) as e:
      results.append(Timing(label, bs, None, None, str(e).splitlines()[0][:120]))
  return results


def summarize(results: Sequence[Timing], fwd_flops: float | None = None) -> str:
  """A table of the sweep, fastest forward first, rejected candidates last."""
  ok = sorted((r for r in results if r.fwd_ms is not None), key=lambda r: r.fwd_ms)
  bad = [r for r in results if r.fwd_ms is None]
  lines = []
  for r in ok:
    line = f"{r.label:72s} fwd {r.fwd_ms * 1e3:9.1f} us"
    if r.bwd_ms is not None:
      line += f"  bwd {r.bwd_ms * 1e3:9.1f} us"
    if fwd_flops:
      f, b = r.tflops(fwd_flops)
      line += f"  {f:7.1f} TF"
      if b is not None:
        line += f" / {b:7.1f} TF"
    lines.append(line)
  for r in bad:
    lines.append(f"{r.label:72s} rejected: {r.error}")
  return "\n".join(lines)


def best(results: Sequence[Timing]) -> Timing | None:
  ok = [r for r in results if r.fwd_ms is not None]
  return min(ok, key=lambda r: r.fwd_ms + (r.bwd_ms or 0.0)) if ok else None


def sdpa_baseline(q, k, v, d_out=None, *, causal: bool, backend: str = "cudnn",
                  iters: int = 10) -> Timing:
  """torch.nn.functional.scaled_dot_product_attention on the same device and inputs
  (q pre-scaled, so scale=1), restricted to one backend: "cudnn" or "flash".

  A library comparator for full and causal masks only; it is never part of the
  product path.  GQA inputs are expanded to MHA first, as SDPA expects equal heads.
  """
  from torch.nn.attention import SDPBackend, sdpa_kernel
  import torch.nn.functional as F
  which = {"cudnn": SDPBackend.CUDNN_ATTENTION, "flash": SDPBackend.FLASH_ATTENTION}[backend]
  if k.shape[1] != q.shape[1]:
    rep = q.shape[1] // k.shape[1]
    k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
  label = f"torch SDPA ({backend})"
  try:
    with sdpa_kernel(which):
      call = lambda a, b, c: F.scaled_dot_product_attention(a, b, c, is_causal=causal, scale=1.0)
      fwd_ms = time_cuda(lambda: call(q, k, v), iters=iters)
      bwd_ms = None
      if d_out is not None:
        qg, kg, vg = (x.detach().clone().requires_grad_(True) for x in (q, k, v))

        def both():
          qg.grad = kg.grad = vg.grad = None
          call(qg, kg, vg).backward(d_out)

        bwd_ms = max(time_cuda(both, iters=iters) - fwd_ms, 0.0)
    return Timing(label, None, fwd_ms, bwd_ms)
  except RuntimeError as e:
    return Timing(label, None, None, None, str(e).splitlines()[0][:160])


def _build_mask(name: str, seq: int, window: int, chunk: int):
  shape = (seq, seq)
  if name == "full":
    return mask_lib.FullMask(shape)
  if name == "causal":
    return mask_lib.CausalMask(shape)
  if name == "local":
    return mask_lib.LocalMask(shape, (window, 0), 0)
  if name == "chunked":
    return mask_lib.ChunkedCausalMask(shape, chunk_size=chunk)
  raise ValueError(name)


def main(argv=None) -> None:
  p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
  p.add_argument("--mask", default="causal", choices=["full", "causal", "local", "chunked"])
  p.add_argument("--seq", type=int, default=8192)
  p.add_argument("--batch", type=int, default=2)
  p.add_argument("--heads", type=int, default=16)
  p.add_argument("--kv-heads", type=int, default=None)
  p.add_argument("--head-dim", type=int, default=128)
  p.add_argument("--dtype", default="bf16", choices=["bf16", "f16"])
  p.add_argument("--window", type=int, default=1024)
  p.add_argument("--chunk", type=int, default=1024)
  p.add_argument("--soft-cap", type=float, default=None)
  p.add_argument("--backward", action="store_true", help="time the backward pass as well")
  p.add_argument("--sdpa", action="store_true", help="also time torch SDPA (cuDNN, flash) on full/causal masks")
  p.add_argument("--iters", type=int, default=10)
  p.add_argument("--json", action="store_true", help="print the results as JSON lines instead of a table")
  args = p.parse_args(argv)

  dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float16
  kvh = args.kv_heads or args.heads
  g = torch.Generator().manual_seed(0)
  d = args.head_dim
  q = (torch.randn(args.batch, args.heads, args.seq, d, generator=g) * d ** -0.5).to(dtype).cuda()
  k = torch.randn(args.batch, kvh, args.seq, d, generator=g).to(dtype).cuda()
  v = torch.randn(args.batch, kvh, args.seq, d, generator=g).to(dtype).cuda()
  d_out = torch.randn(args.batch, args.heads, args.seq, d, generator=g).to(dtype).cuda() if args.backward else None
  mask = _build_mask(args.mask, args.seq, args.window, args.chunk)

  cands = forward_candidates(d)
  if args.backward:
    cands = cands + backward_candidates()
  results = sweep(mask, q, k, v, d_out, attn_logits_soft_cap=args.soft_cap, candidates=cands, iters=args.iters)
  auto = sweep(mask, q, k, v, d_out, attn_logits_soft_cap=args.soft_cap, candidates=[BlockSizes()], iters=args.iters)
  auto[0].label = "automatic: " + auto[0].label
  results += auto
  if args.sdpa and args.mask in ("full", "causal") and args.soft_cap is None:
    for backend in ("cudnn", "flash"):
      results.append(sdpa_baseline(q, k, v, d_out, causal=args.mask == "causal", backend=backend, iters=args.iters))
  flops = useful_forward_flops(splash.make_splash_mha(mask), args.heads, args.batch, d)
  if args.json:
    for r in results:
      print(json.dumps(dict(label=r.label, fwd_ms=r.fwd_ms, bwd_ms=r.bwd_ms, error=r.error)))
  else:
    print(summarize(results, flops))
    top = best(results)
    if top is not None:
      print("fastest:", top.label)


if __name__ == "__main__":
  main()
