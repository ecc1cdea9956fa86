"""Benchmark of the splash attention hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one forward + one backward pass of splash attention over one batch of
seeded synthetic inputs.  The default workload is the one the headline metric is
quoted on: CausalMask MHA, batch 2, 16 heads, seq 8192, head_dim 128, bf16 with f32
accumulation, q pre-scaled by 1/sqrt(128), automatic tiles (128-row forward with
128-wide KV blocks and two alternating softmax warpgroups, fused backward).  Useful FLOPs follow the reference's accounting
(tools/bench.py:86-102): 4 * visible 128x128 blocks * 128 * 128 * head_dim per
forward, 3.5x that for forward + backward.

Prints ONE JSON line.  `value` is forward+backward useful TFLOP/s summed over all
ranks with inputs resident in HBM; `e2e` is the same metric through the public API
with host buffers (pinned host -> device copies of q, k, v, dO and device -> host
copies of out, dq, dk, dv of every step inside the timed region, pipelined over a
copy-in, a compute and a copy-out stream).

Multi-GPU: one process per GPU (torchrun), every rank runs its own copy of the
workload -- the (batch x kv-head) units are independent, so there is no collective
on the data path ("weak" scaling); NCCL carries only the barrier and the max of the
per-rank times.

`sdpa` (rank 0, one GPU, full and causal workloads) is torch's scaled_dot_product_attention
restricted to its cuDNN backend on the same GPU and inputs: a library comparator, not
part of the measured path; --no-sdpa skips it.

--impl reference times the CPU restatement of the reference's dense f32 attention
(oracle/dense_attention.py) on the host cores over a bounded sample of the same
workload; the reference's own code needs JAX, which this image does not have.
"""

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "pallas-mosaic-gpu_b200"))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "useful_attention_tflops_fwd_bwd"
UNIT = "TFLOP/s"

WORKLOADS = {
    # name: (mask kind, batch, heads, kv_heads, seq, head_dim, dtype, soft cap)
    "causal_b2_h16_s8192_d128_bf16": ("causal", 2, 16, 16, 8192, 128, "bf16", None),
    "local1k_gqa_b1_h32_kv8_s16384_d128_bf16_cap50": ("local1k", 1, 32, 8, 16384, 128, "bf16", 50.0),
    "causal_b4_h16_s8192_d64_f16": ("causal", 4, 16, 16, 8192, 64, "f16", None),
    "full_b1_h16_s16384_d128_bf16": ("full", 1, 16, 16, 16384, 128, "bf16", None),
}
DEFAULT_WORKLOAD = "causal_b2_h16_s8192_d128_bf16"


def measured_peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  if os.path.exists(path):
    with open(path) as f:
      p = json.load(f)
    return dict(burst=p["bf16_tflops"], sustained=p["bf16_tflops_sustained"], hbm=p["hbm_gbs"], source="measured")
  return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


def make_mask(sa, kind, seq):
  if kind == "causal":
    return sa.CausalMask((seq, seq))
  if kind == "full":
    return sa.FullMask((seq, seq))
  if kind == "local1k":
    return sa.LocalMask((seq, seq), (1024, 0), 0)
  raise ValueError(kind)


def useful_flops(info, heads, batch, head_dim):
  visible = float(info.num_steps.sum()) * (heads if info.num_steps.shape[0] == 1 else 1) * batch
  fwd = 4.0 * visible * info.block_q * info.block_kv * head_dim
  return fwd, 3.5 * fwd


def host_inputs(batch, heads, kv_heads, seq, d, dtype, seed, pin):
  g = torch.Generator().manual_seed(seed)
  q = (torch.randn(batch, heads, seq, d, generator=g) * d ** -0.5).to(dtype)
  k = torch.randn(batch, kv_heads, seq, d, generator=g).to(dtype)
  v = torch.randn(batch, kv_heads, seq, d, generator=g).to(dtype)
  do = torch.randn(batch, heads, seq, d, generator=g).to(dtype)
  if pin:
    q, k, v, do = (x.pin_memory() for x in (q, k, v, do))
  return q, k, v, do


class ClockSampler:
  """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

  QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
           "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
           "clocks_event_reasons.sw_power_cap")

  def __init__(self, index):
    self.index = index
    self.proc = None
    self.lines = []

  def start(self):
    try:
      self.proc = subprocess.Popen(
          ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
           "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
      self.thread = threading.Thread(target=self._read, daemon=True)
      self.thread.start()
    except OSError:
      self.proc = None

  def _read(self):
    for line in self.proc.stdout:
      self.lines.append(line.strip())

  def stop(self):
    if self.proc is None:
      return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
    time.sleep(0.15)
    self.proc.terminate()
    self.thread.join(timeout=2)
    sm, mx, reasons = [], [], set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for line in self.lines:
      parts = [p.strip() for p in line.split(",")]
      if len(parts) < 7:
        continue
      try:
        sm.append(float(parts[0]))
        mx.append(float(parts[1]))
      except ValueError:
        continue
      for name, val in zip(names, parts[3:7]):
        if val.lower().startswith("active"):
          reasons.add(name)
    return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None,
                reasons=sorted(reasons), samples=len(sm))


def cpu_sample(workload, heads_sampled, cores=None):
  """Times the CPU oracle (forward + analytic backward) on `heads_sampled` (batch, head)
  units of the workload; returns (useful TFLOP/s, seconds, threads)."""
  from oracle import dense_attention as oracle
  import splash_attention_mgpu as sa
  kind, batch, heads, kv_heads, seq, d, dt, cap = WORKLOADS[workload]
  dtype = torch.bfloat16 if dt == "bf16" else torch.float16
  group = heads // kv_heads
  mask = make_mask(sa, kind, seq)
  info = sa.process_mask(mask, (128, 128))
  dense = np.asarray(mask[:, :])[None]
  n = heads_sampled
  g = torch.Generator().manual_seed(1)
  # `n` q heads that share ceil(n / group) KV heads, batch 1: same per-unit work as the workload.
  kvh = max(1, -(-n // group))
  n = kvh * group if group > 1 else n
  q = (torch.randn(1, n, seq, d, generator=g) * d ** -0.5).to(dtype)
  k = torch.randn(1, kvh, seq, d, generator=g).to(dtype)
  v = torch.randn(1, kvh, seq, d, generator=g).to(dtype)
  do = torch.randn(1, n, seq, d, generator=g).to(dtype)
  if cores:
    torch.set_num_threads(cores)
  t0 = time.perf_counter()
  oracle.attention_forward(dense, q, k, v, attn_logits_soft_cap=cap)
  oracle.attention_backward(dense, q, k, v, do, attn_logits_soft_cap=cap)
  dt_s = time.perf_counter() - t0
  _, fb = useful_flops(info, n, 1, d)
  return fb / dt_s / 1e12, dt_s, torch.get_num_threads(), n


def run_reference(args):
  """CPU arm: the oracle restatement of the reference's dense attention on host cores."""
  rank = int(os.environ.get("RANK", "0"))
  if rank != 0:
    return
  workload = args.workload
  kind, batch, heads, kv_heads, seq, d, dt, cap = WORKLOADS[workload]
  sample_heads = 1
  for _ in range(args.warmup):
    cpu_sample(workload, sample_heads)
  times, vals = [], []
  for _ in range(args.steps):
    val, sec, threads, n = cpu_sample(workload, sample_heads)
    times.append(sec)
    vals.append(val)
  total = sum(times)
  import splash_attention_mgpu as sa
  info = sa.process_mask(make_mask(sa, kind, seq), (128, 128))
  _, fb = useful_flops(info, n, 1, d)
  value = fb * len(times) / total / 1e12
  sample = (f"{n} of {batch * heads} (batch, head) units per step, dense f32 forward + analytic backward, "
            f"torch CPU matmuls")
  line = dict(
      impl="reference", metric=METRIC, value=value, unit=UNIT, n_gpus=args.gpus, steps=args.steps,
      warmup=args.warmup, ms_per_step=1e3 * total / len(times), higher_is_better=True, scaling="weak",
      vs_baseline=None, dtype="f32", data="synthetic",
      config=dict(workload=workload, note="CPU restatement of the reference's dense attention; the reference "
                  "itself needs JAX, which is not installed"),
      cpu_baseline=dict(value=value, unit=UNIT, cores=threads, kind="port", sample=sample),
      e2e=dict(value=value, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0),
  )
  print(json.dumps(line), flush=True)


def run_ours(args):
  import splash_attention_mgpu as sa
  rank = int(os.environ.get("RANK", "0"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))
  torch.cuda.set_device(local_rank)
  dev = torch.device("cuda", local_rank)
  dist = None
  if world > 1:
    import torch.distributed as dist
    dist.init_process_group("nccl", device_id=dev)

  workload = args.workload
  kind, batch, heads, kv_heads, seq, d, dt, cap = WORKLOADS[workload]
  dtype = torch.bfloat16 if dt == "bf16" else torch.float16
  kernel = sa.make_splash_mha(make_mask(sa, kind, seq), attn_logits_soft_cap=cap)
  bs = kernel.resolved_block_sizes(d, d)
  fwd_flops, fb_flops = useful_flops(kernel.info, heads, batch, d)

  hq, hk, hv, hdo = host_inputs(batch, heads, kv_heads, seq, d, dtype, seed=rank, pin=True)
  q, k, v, do = (x.to(dev) for x in (hq, hk, hv, hdo))
  q.requires_grad_(True)
  k.requires_grad_(True)
  v.requires_grad_(True)

  def step():
    q.grad = k.grad = v.grad = None
    out = kernel(q, k, v)
    out.backward(do)
    return out

  def barrier():
    torch.cuda.synchronize(dev)
    if dist is not None:
      dist.barrier()
    torch.cuda.synchronize(dev)

  for _ in range(max(args.warmup, 3)):
    step()
  torch.cuda.synchronize(dev)
  sa.check_device_status()

  # ---- device-resident timing ----------------------------------------------------
  sampler = ClockSampler(local_rank)
  if rank == 0:
    sampler.start()
  ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
  barrier()
  start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  start.record()
  for i in range(args.steps):
    q.grad = k.grad = v.grad = None
    ev[i][0].record()
    out = kernel(q, k, v)
    ev[i][1].record()
    out.backward(do)
    ev[i][2].record()
  end.record()
  barrier()
  clocks = sampler.stop() if rank == 0 else None
  elapsed_ms = start.elapsed_time(end)
  fwd_ms = float(np.mean([e[0].elapsed_time(e[1]) for e in ev]))
  bwd_ms = float(np.mean([e[1].elapsed_time(e[2]) for e in ev]))
  sa.check_device_status()

  # ---- end to end through the public API with host buffers ------------------------
  out_h = torch.empty((batch, heads, seq, d), dtype=dtype).pin_memory()
  dq_h, dk_h, dv_h = (torch.empty_like(x).pin_memory() for x in (hq, hk, hv))

  # Three streams, the way a caller that feeds host batches would run it: the inputs of
  # step i+1 are copied in while step i computes and the results of step i-1 are copied
  # out (PCIe carries both directions at once).  Two sets of device input buffers; a set
  # is reused only after the step that read it has finished.
  copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
  compute = torch.cuda.current_stream(dev)
  dev_in = [[torch.empty_like(x, device=dev) for x in (hq, hk, hv, hdo)] for _ in range(2)]
  in_ready = [torch.cuda.Event() for _ in range(2)]
  in_free = [torch.cuda.Event() for _ in range(2)]
  out_done = torch.cuda.Event()

  def e2e_step(i):
    slot = i % 2
    with torch.cuda.stream(copy_in):
      if i >= 2:
        copy_in.wait_event(in_free[slot])
      for dst, src in zip(dev_in[slot], (hq, hk, hv, hdo)):
        dst.copy_(src, non_blocking=True)
      in_ready[slot].record(copy_in)
    compute.wait_event(in_ready[slot])
    qd, kd, vd = (x.detach().requires_grad_(True) for x in dev_in[slot][:3])
    o = kernel(qd, kd, vd)
    o.backward(dev_in[slot][3])
    in_free[slot].record(compute)
    results = (o.detach(), qd.grad, kd.grad, vd.grad)
    with torch.cuda.stream(copy_out):
      copy_out.wait_event(in_free[slot])
      for dst, src in zip((out_h, dq_h, dk_h, dv_h), results):
        src.record_stream(copy_out)
        dst.copy_(src, non_blocking=True)
      out_done.record(copy_out)

  e2e_ms = float("nan")
  if not args.no_e2e:
    for i in range(2):
      e2e_step(i)
    barrier()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for i in range(args.steps):
      e2e_step(i + 2)
    compute.wait_event(out_done)  # the last step's results have reached the host
    e_end.record()
    barrier()
    e2e_ms = e_start.elapsed_time(e_end)
  h2d = sum(x.numel() * x.element_size() for x in (hq, hk, hv, hdo))
  d2h = sum(x.numel() * x.element_size() for x in (out_h, dq_h, dk_h, dv_h))

  times = torch.tensor([elapsed_ms, e2e_ms, fwd_ms, bwd_ms], dtype=torch.float64, device=dev)
  if dist is not None:
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
  elapsed_ms, e2e_ms, fwd_ms, bwd_ms = times.tolist()

  if rank == 0:
    peaks = measured_peaks()
    ms_per_step = elapsed_ms / args.steps
    value = world * fb_flops / (ms_per_step * 1e-3) / 1e12
    fwd_tflops = fwd_flops / (fwd_ms * 1e-3) / 1e12
    bwd_tflops = (fb_flops - fwd_flops) / (bwd_ms * 1e-3) / 1e12
    # Dominant launch group: the backward call (delta pass that also clears the dQ
    # accumulator, fused kernel, transpose-cast); its algorithmic work is 2.5x the forward FLOPs.
    # `traffic`: dram__bytes_read + dram__bytes_write of that kernel from the committed ncu
    # capture of this same workload (profiles/ncu_*_causal_s8192_d128.md), bytes per launch.
    default_wl = workload == DEFAULT_WORKLOAD
    roofline = dict(bound="tensor", achieved=bwd_tflops, peak=peaks["sustained"], unit="TFLOP/s",
                    frac=bwd_tflops / peaks["sustained"], traffic=630.9e6 if default_wl else None,
                    peak_source=peaks["source"] + " sustained bf16",
                    kernel=f"splash_bwd_col_kernel<{d},fused> (about 95% of the backward launch group; timed with its "
                           "delta pass, which also clears the dQ accumulator, and the transpose-cast)",
                    frac_of_nominal_2250=bwd_tflops / 2250.0)
    roofline_fwd = dict(bound="tensor", achieved=fwd_tflops, peak=peaks["sustained"], unit="TFLOP/s",
                        frac=fwd_tflops / peaks["sustained"], traffic=255.0e6 if default_wl else None,
                        kernel=f"splash_fwd_kernel<block_q={bs.block_q},block_kv={bs.block_kv}>",
                        frac_of_nominal_2250=fwd_tflops / 2250.0)
    sdpa = None
    if world == 1 and not args.no_sdpa and kind in ("full", "causal") and cap is None:
      from splash_attention_mgpu import tuning
      t = tuning.sdpa_baseline(q.detach(), k.detach(), v.detach(), do, causal=kind == "causal", backend="cudnn")
      if t.fwd_ms is None:
        sdpa = dict(backend="cudnn", unavailable=t.error)
      else:
        sdpa = dict(backend="cudnn", fwd_tflops=fwd_flops / (t.fwd_ms * 1e9),
                    bwd_tflops=(fb_flops - fwd_flops) / (t.bwd_ms * 1e9) if t.bwd_ms else None,
                    fwd_bwd_tflops=fb_flops / ((t.fwd_ms + (t.bwd_ms or 0.0)) * 1e9) if t.bwd_ms else None,
                    fwd_ms=t.fwd_ms, bwd_ms=t.bwd_ms, note="torch SDPA on the same GPU and inputs; a library "
                    "comparator outside the measured path")
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
      val, sec, threads, n = cpu_sample(workload, 2)
      cpu = dict(value=val, unit=UNIT, cores=threads, kind="port",
                 sample=f"{n} of {batch * heads} (batch, head) units, dense f32 forward + analytic backward "
                        f"(oracle/dense_attention.py), {sec:.1f} s")
    launches_per_step = 1 + 3  # forward; delta (+ accumulator clear), fused backward, transpose-cast
    line = dict(
        metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
        ms_per_step=ms_per_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16" if dt == "bf16" else "f16",
        data="synthetic",
        config=dict(workload=workload, block_q=bs.block_q, block_kv=bs.block_kv, num_stages=bs.num_stages,
                    backward="fused", l2="inputs larger than L2 (q,k,v,dO,out,dq,dk,dv "
                    f"= {8 * batch * heads * seq * d * 2 / 2**20:.0f} MiB per step)",
                    per_rank="every rank runs the whole workload"),
        fwd_tflops=world * fwd_tflops, fwd_ms=fwd_ms, bwd_ms=bwd_ms,
        roofline=roofline, roofline_fwd=roofline_fwd, cpu_baseline=cpu, sdpa=sdpa,
        e2e=dict(value=world * fb_flops / (e2e_ms / args.steps * 1e-3) / 1e12, unit=UNIT,
                 h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h, ms_per_step=e2e_ms / args.steps),
        gpu_launches=launches_per_step * args.steps, clocks=clocks,
    )
    print(json.dumps(line), flush=True)
  if dist is not None:
    dist.destroy_process_group()


def main():
  p = argparse.ArgumentParser()
  p.add_argument("--gpus", type=int, default=1)
  p.add_argument("--steps", type=int, default=20)
  p.add_argument("--warmup", type=int, default=3)
  p.add_argument("--impl", default="ours", choices=["ours", "reference"])
  p.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
  p.add_argument("--no-cpu-baseline", action="store_true")
  p.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (used when profiling)")
  p.add_argument("--no-sdpa", action="store_true", help="skip the torch SDPA (cuDNN) comparator")
  args = p.parse_args()
  if args.impl == "reference":
    run_reference(args)
  else:
    run_ours(args)


if __name__ == "__main__":
  main()
