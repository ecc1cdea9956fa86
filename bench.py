"""Benchmark of the splash attention hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one forward + one backward pass of splash attention over one batch of
seeded synthetic inputs (forward only for the workload that has no backward).  The
default workload is the one the headline metric is quoted on: CausalMask MHA, batch 2,
16 heads, seq 8192, head_dim 128, bf16 with f32 accumulation, q pre-scaled by
1/sqrt(128), automatic tiles.  Useful FLOPs follow the reference's accounting
(tools/bench.py:86-102): 4 * visible 128x128 blocks * 128 * 128 * head_dim per forward,
3.5x that for forward + backward.

Prints ONE JSON line.  `value` is forward+backward useful TFLOP/s of the whole job with
inputs resident in HBM; `e2e` is the same metric through the public API with host
buffers (pinned host -> device copies of q, k, v, dO and device -> host copies of out,
dq, dk, dv of every step inside the timed region, pipelined over a copy-in, a compute
and a copy-out stream).

Multi-GPU: one process per GPU (torchrun).  The workload's (batch x kv-head) units are
split over the ranks in contiguous slices (splash_attention_mgpu.sharding); a unit
needs nothing from any other unit, so there is no collective on the data path and the
total work is fixed ("strong" scaling).  NCCL carries the barrier, the max of the
per-rank times and -- once, outside the timed region -- an all-gather of the outputs,
which rank 0 checks against its own recomputation of one unit per rank.

`sdpa` (rank 0, one GPU, full and causal workloads) is torch's
scaled_dot_product_attention restricted to its cuDNN backend on the same GPU and
inputs: a library comparator, not part of the measured path; --no-sdpa skips it.

--impl reference times the CPU restatement of the reference's dense f32 attention
(oracle/dense_attention.py) on the host cores over a bounded sample of the same
workload; the reference's own code needs JAX, which this image does not have.
"""

import argparse
import dataclasses
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


@dataclasses.dataclass(frozen=True)
class Workload:
  mask: str            # full | causal | local1k | packed_full | packed_per_head | block_sparse
  batch: int
  heads: int
  kv_heads: int
  seq: int
  head_dim: int
  dtype: str           # bf16 | f16
  soft_cap: float | None = None
  segments: bool = False     # packed documents: segment ids per batch row
  mqa: bool = False
  forward_only: bool = False
  block_q: int | None = None
  block_kv: int | None = None
  # Granularity at which useful blocks are counted: the 128 x 128 schedule, as the reference does,
  # unless the mask itself is defined on another grid.
  count_blocks: tuple = (128, 128)


WORKLOADS = {
    # The benchmark configurations of the reference project's baseline, in its order.
    "causal_b2_h16_s8192_d128_bf16": Workload("causal", 2, 16, 16, 8192, 128, "bf16"),
    "local1k_gqa_b1_h32_kv8_s16384_d128_bf16_cap50": Workload("local1k", 1, 32, 8, 16384, 128, "bf16", soft_cap=50.0),
    "packed_full_b4_h16_s8192_d64_f16": Workload("packed_full", 4, 16, 16, 8192, 64, "f16", segments=True),
    "packed_per_head_b4_h16_s8192_d64_f16": Workload("packed_per_head", 4, 16, 16, 8192, 64, "f16", segments=True),
    "mqa_block_sparse_h64_s32768_d256_bf16": Workload("block_sparse", 1, 64, 1, 32768, 256, "bf16", mqa=True,
                                                      forward_only=True, block_q=128, block_kv=64,
                                                      count_blocks=(128, 64)),
    # The same mask with 8 q heads: small enough for a profiler capture (a few hundred MB on the device).
    "mqa_block_sparse_h8_s32768_d256_bf16": Workload("block_sparse", 1, 8, 1, 32768, 256, "bf16", mqa=True,
                                                     forward_only=True, block_q=128, block_kv=64,
                                                     count_blocks=(128, 64)),
    # Extra shapes.
    "full_b1_h16_s16384_d128_bf16": Workload("full", 1, 16, 16, 16384, 128, "bf16"),
    "causal_b4_h16_s8192_d64_f16": Workload("causal", 4, 16, 16, 8192, 64, "f16"),
}
DEFAULT_WORKLOAD = "causal_b2_h16_s8192_d128_bf16"


def measured_peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  if os.path.exists(path):
    with open(path) as f:
      p = json.load(f)
    return dict(burst=p["bf16_tflops"], sustained=p["bf16_tflops_sustained"], hbm=p["hbm_gbs"], source="measured")
  return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


def ncu_traffic(kernel_key):
  """DRAM bytes per launch of a kernel from the committed ncu captures (profiles/traffic.json)."""
  path = os.path.join(ROOT, "profiles", "traffic.json")
  if not os.path.exists(path):
    return None
  with open(path) as f:
    return json.load(f).get(kernel_key)


def torch_dtype(wl):
  return torch.bfloat16 if wl.dtype == "bf16" else torch.float16


def block_sparse_mask(seq, seed=5):
  """128x64 blocks: empty w.p. 0.70, full 0.20, partial 0.10 (iid Bernoulli(0.5) elements);
  diagonal forced on so no row is empty."""
  rng = np.random.default_rng(seed)
  kinds = rng.choice(3, size=(seq // 128, seq // 64), p=[0.70, 0.10, 0.20])  # 0 empty, 1 partial, 2 full
  dense = np.zeros((seq, seq), bool)
  for i, j in zip(*np.nonzero(kinds == 2)):
    dense[i * 128:(i + 1) * 128, j * 64:(j + 1) * 64] = True
  for i, j in zip(*np.nonzero(kinds == 1)):
    dense[i * 128:(i + 1) * 128, j * 64:(j + 1) * 64] = rng.random((128, 64)) < 0.5
  dense[np.arange(seq), np.arange(seq)] = True
  return dense


def head_masks(sa, wl):
  """One mask object per q head (a single-element list when all heads share it)."""
  s = wl.seq
  if wl.mask == "causal":
    return [sa.CausalMask((s, s))]
  if wl.mask in ("full", "packed_full"):
    return [sa.FullMask((s, s))]
  if wl.mask == "local1k":
    return [sa.LocalMask((s, s), (1024, 0), 0)]
  if wl.mask == "packed_per_head":
    return [sa.CausalMask((s, s)) if h % 2 == 0 else sa.ChunkedCausalMask((s, s), chunk_size=1024)
            for h in range(wl.heads)]
  if wl.mask == "block_sparse":
    return [sa.NumpyMask(block_sparse_mask(s))]
  raise ValueError(wl.mask)


def packed_segments(batch, seq, seed=7):
  """Segment lengths drawn uniformly from [256, 4096], truncated to fill the sequence."""
  rng = np.random.default_rng(seed)
  ids = np.zeros((batch, seq), np.int32)
  for b in range(batch):
    pos, seg = 0, 0
    while pos < seq:
      n = int(rng.integers(256, 4097))
      ids[b, pos:pos + n] = seg
      pos += n
      seg += 1
  return ids


def visible_blocks_per_head(sa, wl, masks):
  """Visible schedule blocks of each q head and the FLOPs of one block (reference accounting)."""
  bq, bkv = wl.count_blocks
  per_head = []
  for m in (masks if len(masks) > 1 else masks[:1]):
    info = sa.process_mask(m, (bq, bkv))
    per_head.append(float(info.num_steps.sum()))
  if len(per_head) == 1:
    per_head = per_head * wl.heads
  return per_head, 4.0 * bq * bkv * wl.head_dim


class Partition:
  """This rank's share of a workload: contiguous (batch x kv-head) units, presented to the
  kernel as a batch of problems.  A shared mask gives [units, group, S, D] / [units, 1, S, D];
  per-head masks keep [batches, heads', S, D] with the rank's head range; the MQA forward-only
  workload (one unit) shards its q heads instead, K/V replicated."""

  def __init__(self, sa, wl, world, rank):
    from splash_attention_mgpu import sharding
    self.wl, self.world, self.rank = wl, world, rank
    masks = head_masks(sa, wl)
    self.per_head_blocks, self.block_flops = visible_blocks_per_head(sa, wl, masks)
    group = wl.heads // wl.kv_heads
    bs = sa.BlockSizes(block_q=wl.block_q, block_kv=wl.block_kv)
    make = sa.make_splash_mqa if wl.mqa else sa.make_splash_mha
    self.shard_q_heads = wl.mqa and wl.batch * wl.kv_heads == 1
    if self.shard_q_heads:
      self.num_units = wl.heads
      lo, hi = sharding.unit_range(self.num_units, world, rank)
      # unit = one q head; the kernel sees [heads', S, D] and the shared [S, D] K/V.
      self.unit_heads = [[h] for h in range(lo, hi)]
      self.kernel = make(masks[0], block_sizes=bs, attn_logits_soft_cap=wl.soft_cap)
      self.q_shape = (hi - lo, wl.seq, wl.head_dim)
      self.kv_shape = (wl.seq, wl.head_dim)
    else:
      self.num_units = wl.batch * wl.kv_heads
      lo, hi = sharding.unit_range(self.num_units, world, rank)
      self.unit_heads = [[(u % wl.kv_heads) * group + g for g in range(group)] for u in range(lo, hi)]
      if len(masks) == 1:
        self.kernel = make(masks[0], block_sizes=bs, attn_logits_soft_cap=wl.soft_cap)
        self.q_shape = (hi - lo, group, wl.seq, wl.head_dim)
        self.kv_shape = (hi - lo, 1, wl.seq, wl.head_dim)
      else:
        # Per-head masks: whole batches, or a head range inside one batch.
        n = hi - lo
        if n % wl.kv_heads == 0 and lo % wl.kv_heads == 0:
          batches, kvh0, kvh1 = n // wl.kv_heads, 0, wl.kv_heads
        elif n and wl.kv_heads % n == 0 and lo // wl.kv_heads == (hi - 1) // wl.kv_heads:
          batches, kvh0, kvh1 = 1, lo % wl.kv_heads, lo % wl.kv_heads + n
        elif n == 0:
          batches, kvh0, kvh1 = 0, 0, 1
        else:
          raise ValueError(f"{wl.mask}: {self.num_units} units do not split into head ranges over {world} ranks")
        sub = masks[kvh0 * group:kvh1 * group]
        self.kernel = make(sa.MultiHeadMask(sub), block_sizes=bs, attn_logits_soft_cap=wl.soft_cap)
        self.q_shape = (batches, (kvh1 - kvh0) * group, wl.seq, wl.head_dim)
        self.kv_shape = (batches, kvh1 - kvh0, wl.seq, wl.head_dim)
    self.span = (lo, hi)
    self.unit_batch = [u // wl.kv_heads for u in range(lo, hi)] if not self.shard_q_heads else [0] * (hi - lo)

  def flops(self, span=None):
    """(forward, forward+backward) useful FLOPs of the units in `span` (default: this rank's)."""
    if span is None:
      heads = [h for hs in self.unit_heads for h in hs]
    else:
      group = self.wl.heads // self.wl.kv_heads
      heads = ([h for h in range(*span)] if self.shard_q_heads else
               [(u % self.wl.kv_heads) * group + g for u in range(*span) for g in range(group)])
    fwd = sum(self.per_head_blocks[h] for h in heads) * self.block_flops
    return fwd, fwd if self.wl.forward_only else 3.5 * fwd

  def total_flops(self):
    return self.flops((0, self.num_units))

  def host_inputs(self, pin, span=None):
    """q, k, v, dO of the units in `span` (default: this rank's) on the host; every unit is drawn
    from a generator seeded by its index, so a unit's data does not depend on the partition."""
    wl = self.wl
    dtype = torch_dtype(wl)
    lo, hi = self.span if span is None else span
    group = wl.heads // wl.kv_heads
    d, s = wl.head_dim, wl.seq
    qs, ks, vs, dos = [], [], [], []
    if self.shard_q_heads:
      g = torch.Generator().manual_seed(10_000)
      k = torch.randn(s, d, generator=g).to(dtype)
      v = torch.randn(s, d, generator=g).to(dtype)
    for u in range(lo, hi):
      g = torch.Generator().manual_seed(u)
      rows = 1 if self.shard_q_heads else group
      qs.append((torch.randn(rows, s, d, generator=g) * d ** -0.5).to(dtype))
      dos.append(torch.randn(rows, s, d, generator=g).to(dtype))
      if not self.shard_q_heads:
        ks.append(torch.randn(1, s, d, generator=g).to(dtype))
        vs.append(torch.randn(1, s, d, generator=g).to(dtype))
    n = hi - lo
    if self.shard_q_heads:
      q = torch.cat(qs).reshape(n, s, d) if n else torch.empty((0, s, d), dtype=dtype)
      do = torch.cat(dos).reshape(n, s, d) if n else torch.empty((0, s, d), dtype=dtype)
    else:
      shape_q = self.q_shape if span is None else (n, group, s, d)
      shape_kv = self.kv_shape if span is None else (n, 1, s, d)
      q = torch.stack(qs).reshape(shape_q) if n else torch.empty(shape_q, dtype=dtype)
      do = torch.stack(dos).reshape(shape_q) if n else torch.empty(shape_q, dtype=dtype)
      k = torch.stack(ks).reshape(shape_kv) if n else torch.empty(shape_kv, dtype=dtype)
      v = torch.stack(vs).reshape(shape_kv) if n else torch.empty(shape_kv, dtype=dtype)
    out = [q, k, v, do]
    if pin:
      out = [x.pin_memory() for x in out]
    return out

  def segment_ids(self, sa, device, span=None):
    wl = self.wl
    if not wl.segments:
      return None
    ids = packed_segments(wl.batch, wl.seq)
    lo, hi = self.span if span is None else span
    if self.q_shape[0] == hi - lo or span is not None:   # unit-major batch: one row per unit
      rows = [u // wl.kv_heads for u in range(lo, hi)]
    else:                                                # per-head masks: one row per batch element
      rows = sorted(set(u // wl.kv_heads for u in range(lo, hi)))
    t = torch.from_numpy(ids[rows]).to(device)
    return sa.SegmentIds(t, t)


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

  def mark(self):
    return len(self.lines)

  def summary(self, first=0, last=None):
    sm, mx, reasons = [], [], set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for line in self.lines[first:last]:
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

  def stop(self):
    if self.proc is None:
      return
    time.sleep(0.15)
    self.proc.terminate()
    self.thread.join(timeout=2)


def host_threads():
  try:
    return len(os.sched_getaffinity(0))
  except AttributeError:
    return os.cpu_count() or 1


def cpu_sample(wl_name, units_sampled=1):
  """Times the CPU oracle (forward + analytic backward) on `units_sampled` (batch, kv-head) units of
  the workload with every host thread this process may use; returns (TFLOP/s, seconds, threads, units)."""
  from oracle import dense_attention as oracle
  import splash_attention_mgpu as sa
  wl = WORKLOADS[wl_name]
  torch.set_num_threads(host_threads())   # torchrun exports OMP_NUM_THREADS=1
  part = Partition(sa, wl, 1, 0)
  n = min(units_sampled, part.num_units)
  q, k, v, do = part.host_inputs(pin=False, span=(0, n))
  masks = head_masks(sa, wl)
  group = wl.heads // wl.kv_heads
  seg_all = packed_segments(wl.batch, wl.seq) if wl.segments else None
  t0 = time.perf_counter()
  for u in range(n):
    heads = [0] if part.shard_q_heads else [(u % wl.kv_heads) * group + g for g in range(group)]
    dense = np.stack([np.asarray(masks[h if len(masks) > 1 else 0][:, :]) for h in heads])
    if len(masks) == 1:
      dense = dense[:1]
    seg = None if seg_all is None else (seg_all[u // wl.kv_heads], seg_all[u // wl.kv_heads])
    qu = q[u:u + 1] if not part.shard_q_heads else q[u:u + 1][None]
    ku = k[u:u + 1] if not part.shard_q_heads else k[None, None]
    vu = v[u:u + 1] if not part.shard_q_heads else v[None, None]
    dou = do[u:u + 1] if not part.shard_q_heads else do[u:u + 1][None]
    oracle.attention_forward(dense, qu, ku, vu, seg, attn_logits_soft_cap=wl.soft_cap)
    if not wl.forward_only:
      oracle.attention_backward(dense, qu, ku, vu, dou, seg, attn_logits_soft_cap=wl.soft_cap)
  dt_s = time.perf_counter() - t0
  _, fb = part.flops((0, n))
  return fb / dt_s / 1e12, dt_s, torch.get_num_threads(), n, part.num_units


def base_config(wl_name, world):
  """The part of `config` both arms print identically."""
  wl = WORKLOADS[wl_name]
  per_step = 8 * wl.batch * wl.heads * wl.seq * wl.head_dim * 2 / 2 ** 20
  return dict(workload=wl_name,
              partition=f"{wl.batch * wl.kv_heads if not (wl.mqa and wl.batch * wl.kv_heads == 1) else wl.heads} "
                        f"independent units in contiguous slices over {world} rank(s)",
              l2=f"inputs larger than L2 (q,k,v,dO,out,dq,dk,dv = {per_step:.0f} MiB per step over all ranks)")


def run_reference(args):
  """CPU arm: the oracle restatement of the reference's dense attention on host cores."""
  rank = int(os.environ.get("RANK", "0"))
  if rank != 0:
    return
  wl_name = args.workload
  for _ in range(args.warmup):
    cpu_sample(wl_name, 1)
  times, vals = [], []
  for _ in range(args.steps):
    val, sec, threads, n, units = cpu_sample(wl_name, 1)
    times.append(sec)
    vals.append(val)
  total = sum(times)
  value = sum(v * t for v, t in zip(vals, times)) / total   # sampled FLOPs / time over all steps
  sample = (f"{n} of {units} (batch, kv-head) units per step, dense f32 forward + analytic backward, "
            f"torch CPU matmuls on {threads} threads")
  line = dict(
      impl="reference", metric=METRIC, value=value, unit=UNIT, n_gpus=args.gpus, steps=args.steps,
      warmup=args.warmup, ms_per_step=1e3 * total / len(times), higher_is_better=True, scaling="strong",
      vs_baseline=None, dtype="f32", data="synthetic", config=base_config(wl_name, max(1, args.gpus)),
      note="CPU restatement of the reference's dense attention; the reference itself needs JAX, which is not installed",
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

  # The timed loops run on torch's current stream; the one-off graph warm-up on a side stream is the only
  # place where gradients are accumulated on another stream, which autograd would warn about.
  torch.autograd.graph.set_warn_on_accumulate_grad_stream_mismatch(False)
  wl_name = args.workload
  wl = WORKLOADS[wl_name]
  if args.block_q or args.block_kv:   # tiling override (profiling a particular kernel)
    wl = dataclasses.replace(wl, block_q=args.block_q or wl.block_q, block_kv=args.block_kv or wl.block_kv)
  dtype = torch_dtype(wl)
  part = Partition(sa, wl, world, rank)
  kernel = part.kernel
  n_local = part.span[1] - part.span[0]
  d = wl.head_dim
  bs = kernel.resolved_block_sizes(d, d, has_segments=wl.segments)
  fwd_flops, fb_flops = part.total_flops()          # whole job
  local_fwd_flops, _ = part.flops()
  seg = part.segment_ids(sa, dev)

  host = part.host_inputs(pin=True)
  hq, hk, hv, hdo = host
  q, k, v, do = (x.to(dev) for x in host)
  if not wl.forward_only:
    q.requires_grad_(True)
    k.requires_grad_(True)
    v.requires_grad_(True)

  def step(qq=q, kk=k, vv=v, dd=do):
    if n_local == 0:
      return None
    if wl.forward_only:
      out, _ = kernel(qq, kk, vv, seg, save_residuals=True)
      return out
    qq.grad = kk.grad = vv.grad = None
    out = kernel(qq, kk, vv, seg)
    out.backward(dd)
    return out

  def barrier():
    torch.cuda.synchronize(dev)
    if dist is not None:
      dist.barrier()
    torch.cuda.synchronize(dev)

  warmup = max(args.warmup, 3)
  for _ in range(warmup):
    step()
  torch.cuda.synchronize(dev)
  sa.check_device_status()

  # ---- one CUDA graph of the step (the library's calls are capturable: no allocation, no sync) ------
  graph, fwd_graph, graph_error = None, None, None
  if not args.no_graph and n_local > 0:
    try:
      side = torch.cuda.Stream(dev)
      side.wait_stream(torch.cuda.current_stream(dev))
      with torch.cuda.stream(side):
        step()
      torch.cuda.current_stream(dev).wait_stream(side)
      graph = torch.cuda.CUDAGraph()
      if not wl.forward_only:
        q.grad = k.grad = v.grad = None
      with torch.cuda.graph(graph):
        graph_out = step()
      graph.replay()
      torch.cuda.synchronize(dev)
      sa.check_device_status()
      if not wl.forward_only:
        # The forward on its own (with its logsumexp residual), for the forward / backward split.
        qd, kd, vd = q.detach(), k.detach(), v.detach()
        kernel(qd, kd, vd, seg, save_residuals=True)
        fwd_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(fwd_graph):
          fwd_graph_out = kernel(qd, kd, vd, seg, save_residuals=True)
        fwd_graph.replay()
        torch.cuda.synchronize(dev)
    except Exception as e:  # capture is an optimisation of the launch path only
      graph = None
      graph_error = f"{type(e).__name__}: {str(e).splitlines()[0][:160]}"
      torch.cuda.synchronize(dev)

  # ---- device-resident timing -------------------------------------------------------------------
  sampler = ClockSampler(local_rank)
  if rank == 0:
    sampler.start()

  def timed_loop(steps, use_graph, split=False):
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)] if split else None
    barrier()
    first = sampler.mark()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
      if n_local == 0:
        continue
      if use_graph:
        graph.replay()
      elif split and not wl.forward_only:
        q.grad = k.grad = v.grad = None
        ev[i][0].record()
        out = kernel(q, k, v, seg)
        ev[i][1].record()
        out.backward(do)
        ev[i][2].record()
      else:
        step()
    end.record()
    barrier()
    ms = start.elapsed_time(end)
    fwd = bwd = float("nan")
    if split and not wl.forward_only and n_local:
      # Medians: an eager step that the host was late to launch would otherwise count idle time.
      fwd = float(np.median([e[0].elapsed_time(e[1]) for e in ev]))
      bwd = float(np.median([e[1].elapsed_time(e[2]) for e in ev]))
    return ms, fwd, bwd, (first, sampler.mark())

  for _ in range(3):   # eager warm-up again: the capture above changed the allocator's state
    step()
  eager_ms, fwd_in_step_ms, eager_bwd_ms, eager_marks = timed_loop(args.steps, False, split=True)
  bwd_ms = eager_bwd_ms
  # The forward on its own, as the reference's benchmark times it (tools/bench.py:70-76: the forward
  # with its logsumexp residual in a loop of its own, then forward + backward): a replay of its graph
  # when there is one, eager calls otherwise.
  fwd_ms = eager_ms / args.steps
  if not wl.forward_only:
    qd, kd, vd = q.detach(), k.detach(), v.detach()
    for _ in range(3):
      if n_local:
        kernel(qd, kd, vd, seg, save_residuals=True)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
      if fwd_graph is not None:
        fwd_graph.replay()
      elif n_local:
        kernel(qd, kd, vd, seg, save_residuals=True)
    f1.record()
    barrier()
    fwd_ms = f0.elapsed_time(f1) / args.steps
  graph_ms, _, _, graph_marks = timed_loop(args.steps, True) if graph is not None else (float("nan"), 0, 0, eager_marks)
  if graph is not None and fwd_graph is not None and graph_ms <= eager_ms:
    # Backward = replayed step minus replayed forward: free of host launch gaps.
    bwd_ms = graph_ms / args.steps - fwd_ms
  sa.check_device_status()

  # A loop of at least two seconds: the clocks settle at the power cap there.
  sus_ms, n_sus, sus_marks = -1.0, 0, (0, 0)
  if not args.no_sustained:
    est = (graph_ms if graph is not None else eager_ms) / args.steps
    n_sus = int(min(20000, max(args.steps, 2200.0 / max(est, 1e-3))))
    sus_ms, _, _, sus_marks = timed_loop(n_sus, graph is not None)
  # ---- end to end through the public API with host buffers --------------------------------------
  out_h = torch.empty(tuple(q.shape[:-1]) + (v.shape[-1],), dtype=dtype).pin_memory()
  grads_h = [] if wl.forward_only else [torch.empty_like(x).pin_memory() for x in (hq, hk, hv)]

  # Three streams, the way a caller that feeds host batches would run it: the inputs of step i+1 are
  # copied in while step i computes and the results of step i-1 are copied out (PCIe carries both
  # directions at once).  Two sets of device input buffers; a set is reused only after the step that
  # read it has finished.
  copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
  compute = torch.cuda.current_stream(dev)
  dev_in = [[torch.empty_like(x, device=dev) for x in host] for _ in range(2)]
  in_ready = [torch.cuda.Event() for _ in range(2)]
  in_free = [torch.cuda.Event() for _ in range(2)]
  out_done = torch.cuda.Event()

  def e2e_step(i):
    slot = i % 2
    with torch.cuda.stream(copy_in):
      if i >= 2:
        copy_in.wait_event(in_free[slot])
      for dst, src in zip(dev_in[slot], host):
        dst.copy_(src, non_blocking=True)
      in_ready[slot].record(copy_in)
    compute.wait_event(in_ready[slot])
    if n_local == 0:
      in_free[slot].record(compute)
      out_done.record(copy_out)
      return
    if wl.forward_only:
      o, _ = kernel(*dev_in[slot][:3], seg, save_residuals=True)
      results = (o,)
    else:
      qd, kd, vd = (x.detach().requires_grad_(True) for x in dev_in[slot][:3])
      o = kernel(qd, kd, vd, seg)
      o.backward(dev_in[slot][3])
      results = (o.detach(), qd.grad, kd.grad, vd.grad)
    in_free[slot].record(compute)
    with torch.cuda.stream(copy_out):
      copy_out.wait_event(in_free[slot])
      for dst, src in zip([out_h] + grads_h, results):
        src.record_stream(copy_out)
        dst.copy_(src, non_blocking=True)
      out_done.record(copy_out)

  e2e_ms = float("nan")
  if not args.no_e2e:
    # Untimed steps first: they fill the pipeline and let the caching allocator settle on the
    # result buffers it recycles between the compute and the copy-out stream.
    e2e_warm = 4
    for i in range(e2e_warm):
      e2e_step(i)
    torch.cuda.synchronize(dev)
    barrier()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for i in range(args.steps):
      e2e_step(i + e2e_warm)
    compute.wait_event(out_done)  # the last step's results have reached the host
    e_end.record()
    barrier()
    e2e_ms = e_start.elapsed_time(e_end)
  h2d_local = sum(x.numel() * x.element_size() for x in (host if not wl.forward_only else host[:3]))
  d2h_local = sum(x.numel() * x.element_size() for x in [out_h] + grads_h)

  # ---- gather for checking (once, outside every timed region) ------------------------------------
  check = None
  out_dev = step()
  torch.cuda.synchronize(dev)
  if dist is not None and not part.shard_q_heads and len(head_masks(sa, wl)) == 1:
    from splash_attention_mgpu import sharding
    full = sharding.gather_units(out_dev.detach(), part.span, (wl.batch, wl.heads, wl.seq, d))
    if rank == 0:
      # Rank 0 recomputes the first unit of every rank on its own GPU: the bits must agree.
      group = wl.heads // wl.kv_heads
      units = full.reshape(wl.batch * wl.kv_heads, group, wl.seq, d)
      same, n_checked = True, 0
      for r in range(world):
        lo, hi = sharding.unit_range(part.num_units, world, r)
        if hi == lo:
          continue
        uq, uk, uv, _ = (x.to(dev) for x in part.host_inputs(pin=False, span=(lo, lo + 1)))
        useg = part.segment_ids(sa, dev, span=(lo, lo + 1))
        with torch.no_grad():
          mine = kernel(uq, uk, uv, useg)
        same = same and bool(torch.equal(mine[0], units[lo]))
        n_checked += 1
      check = dict(gathered_units=int(units.shape[0]), recomputed_on_rank0=n_checked, bit_identical=same,
                   how="NCCL all_gather of the forward outputs, then one unit per rank recomputed on rank 0")

  nan_to = lambda x: x if x == x else -1.0
  stats = [eager_ms, graph_ms if graph is not None else -1.0, e2e_ms, fwd_ms, nan_to(bwd_ms), sus_ms,
           nan_to(fwd_in_step_ms), nan_to(eager_bwd_ms)]
  times = torch.tensor(stats, dtype=torch.float64, device=dev)
  sums = torch.tensor([float(h2d_local), float(d2h_local), local_fwd_flops], dtype=torch.float64, device=dev)
  if dist is not None:
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dist.all_reduce(sums, op=dist.ReduceOp.SUM)
  eager_ms, graph_ms, e2e_ms, fwd_ms, bwd_ms, sus_ms, fwd_in_step_ms, eager_bwd_ms = times.tolist()
  h2d, d2h, fwd_flops_sum = sums.tolist()
  assert abs(fwd_flops_sum - fwd_flops) <= 1e-6 * fwd_flops, "the ranks' units do not add up to the workload"

  if rank == 0:
    sampler.stop()
    peaks = measured_peaks()
    use_graph = graph_ms > 0 and graph_ms <= eager_ms
    timed_ms = graph_ms if use_graph else eager_ms
    ms_per_step = timed_ms / args.steps
    clocks = sampler.summary(*(graph_marks if use_graph else eager_marks))
    if not clocks["samples"]:
      # A timed region shorter than the 20 ms sampling period: take the samples of both loops, and of the
      # whole run if those are still empty.
      clocks = sampler.summary(eager_marks[0], graph_marks[1])
      if not clocks["samples"]:
        clocks = sampler.summary()
      clocks["window"] = "timed region shorter than the sampling period; samples of the surrounding loops"
    value = fb_flops / (ms_per_step * 1e-3) / 1e12
    fwd_tflops = fwd_flops / (fwd_ms * 1e-3) / 1e12
    bwd_tflops = (fb_flops - fwd_flops) / (bwd_ms * 1e-3) / 1e12 if not wl.forward_only else None
    # The peak a number is held against: the burst GEMM rate when the timed region is short (the clocks
    # have not yet settled at the power cap), the sustained one for a loop of seconds.
    def peak_for(ms):
      return (peaks["burst"], "burst") if ms < 1000.0 else (peaks["sustained"], "sustained")

    peak, which = peak_for(timed_ms)
    default_wl = wl_name == DEFAULT_WORKLOAD
    io_bytes = wl.batch * wl.seq * d * 2 * (2 * wl.heads + 2 * wl.kv_heads) + wl.batch * wl.heads * wl.seq * 4
    if wl.forward_only:
      info = kernel.fwd_info(bs.block_q, bs.block_kv)
      mask_bytes = 0 if info.partial_mask_blocks is None else int(np.asarray(info.partial_mask_blocks).size)
      # Compulsory bytes: q, out, k, v, lse once; every dense partial mask block once per q head.
      model = io_bytes + mask_bytes * wl.heads
      gbs = model / (fwd_ms * 1e-3) / 1e9
      roofline = dict(bound="hbm", achieved=gbs, peak=peaks["hbm"], unit="GB/s", frac=gbs / peaks["hbm"],
                      traffic=ncu_traffic(f"fwd:{wl_name}"), traffic_model=model,
                      peak_source=peaks["source"] + " copy bandwidth",
                      kernel=f"splash_fwd_kernel<block_q={bs.block_q},block_kv={bs.block_kv}> (streams int8 mask "
                             "blocks per head; also reported against the tensor peak in roofline_fwd)")
    else:
      # Dominant launch group: the backward call (delta pass that also clears the dQ accumulator, fused
      # kernel, transpose-cast); its algorithmic work is 2.5x the forward FLOPs.
      acc_bytes = wl.batch * wl.heads * wl.seq * d * 4
      model = 2 * io_bytes + 3 * acc_bytes   # q,k,v,dO,out,lse,delta in; dq,dk,dv out; accumulator cleared, reduced, read
      roofline = dict(bound="tensor", achieved=bwd_tflops / world, peak=peak, unit="TFLOP/s",
                      frac=bwd_tflops / world / peak,
                      traffic=ncu_traffic("bwd:" + wl_name) if world == 1 else None, traffic_model=model / world,
                      peak_source=f"{peaks['source']} {which} bf16 GEMM",
                      kernel=f"fused backward kernel, head_dim {d} (about 95% of the backward launch group; timed with "
                             "its delta pass, which also clears the dQ accumulator, and the transpose-cast); per GPU",
                      frac_of_nominal_2250=bwd_tflops / world / 2250.0)
    roofline_fwd = dict(bound="tensor", achieved=fwd_tflops / world, peak=peak, unit="TFLOP/s",
                        frac=fwd_tflops / world / peak,
                        traffic=ncu_traffic("fwd:" + wl_name) if world == 1 else None,
                        traffic_model=io_bytes / world,
                        kernel=f"splash_fwd_kernel<block_q={bs.block_q},block_kv={bs.block_kv}>; per GPU",
                        frac_of_nominal_2250=fwd_tflops / world / 2250.0)
    sus = None
    if sus_ms > 0:
      sus_clocks = sampler.summary(*sus_marks)
      sus_value = fb_flops * n_sus / (sus_ms * 1e-3) / 1e12
      sus = dict(seconds=sus_ms / 1e3, steps=n_sus, ms_per_step=sus_ms / n_sus, value=sus_value, unit=UNIT,
                 frac_of_sustained_peak=sus_value / world / peaks["sustained"], clocks=sus_clocks)
    sdpa = None
    if world == 1 and not args.no_sdpa and wl.mask in ("full", "causal") and wl.soft_cap is None:
      from splash_attention_mgpu import tuning
      t = tuning.sdpa_baseline(q.detach(), k.detach(), v.detach(), do, causal=wl.mask == "causal", backend="cudnn")
      if t.fwd_ms is None:
        sdpa = dict(backend="cudnn", unavailable=t.error)
      else:
        sdpa = dict(backend="cudnn", fwd_tflops=fwd_flops / (t.fwd_ms * 1e9),
                    bwd_tflops=(fb_flops - fwd_flops) / (t.bwd_ms * 1e9) if t.bwd_ms else None,
                    fwd_bwd_tflops=fb_flops / ((t.fwd_ms + (t.bwd_ms or 0.0)) * 1e9) if t.bwd_ms else None,
                    fwd_ms=t.fwd_ms, bwd_ms=t.bwd_ms, note="torch SDPA on the same GPU and inputs; a library "
                    "comparator outside the measured path")
    fwd256 = None
    if world == 1 and default_wl and not args.no_sdpa:
      from splash_attention_mgpu import tuning
      k256 = sa.make_splash_mha(head_masks(sa, wl)[0], block_sizes=sa.BlockSizes(block_q=256))
      ms256 = tuning.time_cuda(lambda: k256(q.detach(), k.detach(), v.detach(), save_residuals=True))
      fwd256 = fwd_flops / (ms256 * 1e9)
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
      val, sec, threads, n, units = cpu_sample(wl_name, 2)
      cpu = dict(value=val, unit=UNIT, cores=threads, kind="port",
                 sample=f"{n} of {units} (batch, kv-head) units, dense f32 forward + analytic backward "
                        f"(oracle/dense_attention.py), {sec:.1f} s")
    launches_per_step = 1 if wl.forward_only else 1 + 3  # forward; delta (+ accumulator clear), fused backward, transpose-cast
    config = base_config(wl_name, world)
    line = dict(
        metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=args.steps, warmup=warmup,
        ms_per_step=ms_per_step, higher_is_better=True, scaling="strong", vs_baseline=None, dtype=wl.dtype,
        data="synthetic", config=config,
        details=dict(block_q=bs.block_q, block_kv=bs.block_kv, num_stages=bs.num_stages,
                     backward=None if wl.forward_only else "fused",
                     launch="cuda graph replay of the public API calls" if use_graph else "eager public API calls",
                     per_rank=f"rank r runs units [r*{part.num_units}//{world} ...): {n_local} of {part.num_units} on rank 0",
                     eager_ms_per_step=eager_ms / args.steps,
                     graph_ms_per_step=graph_ms / args.steps if graph_ms > 0 else None, graph_error=graph_error),
        fwd_tflops=fwd_tflops, fwd_ms=fwd_ms, bwd_ms=None if wl.forward_only else bwd_ms,
        eager_split=None if wl.forward_only else dict(fwd_ms=fwd_in_step_ms, bwd_ms=eager_bwd_ms,
                                                      note="medians of events between the halves of eager steps"),
        fwd256_tflops=fwd256,
        roofline=roofline, roofline_fwd=roofline_fwd, sustained=sus, cpu_baseline=cpu, sdpa=sdpa, check=check,
        e2e=dict(value=fb_flops / (e2e_ms / args.steps * 1e-3) / 1e12, unit=UNIT,
                 h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h, ms_per_step=e2e_ms / args.steps),
        gpu_launches=launches_per_step * args.steps * world, clocks=clocks,
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
  p.add_argument("--no-graph", action="store_true", help="time eager calls only")
  p.add_argument("--no-sustained", action="store_true", help="skip the two-second loop")
  p.add_argument("--block-q", type=int, default=None, help="forward tile rows (128 or 256) instead of the automatic choice")
  p.add_argument("--block-kv", type=int, default=None, help="forward KV block width (64 or 128)")
  args = p.parse_args()
  if args.impl == "reference":
    run_reference(args)
  else:
    run_ours(args)


if __name__ == "__main__":
  main()
