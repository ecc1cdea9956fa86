"""Turns Nsight Compute reports of the library's kernels into the short text summaries
and the traffic table the benchmark reads.

  python -m splash_attention_mgpu.profiling summary REPORT.ncu-rep --title "..." \
      --command "ncu ... python bench.py ..." --out profiles/NAME.md \
      [--traffic-key fwd:WORKLOAD --traffic-json profiles/traffic.json] [--notes "..."]
  python -m splash_attention_mgpu.profiling launches LAUNCHES.csv --title "..." \
      --command "ncu --metrics gpu__time_duration.sum ..." --out profiles/NAME.md

`summary` reads one captured launch (`ncu -i REPORT --page raw --csv`, which needs no
GPU) and writes the counters that say what bounds the kernel: duration and clock, tensor,
special-function and FMA pipe use, the shared-memory data pipe split into tensor-core
operand reads and load/store traffic, L2 and DRAM bytes, registers, the top warp stall
reasons.  With --traffic-key it also records `dram__bytes_read.sum +
dram__bytes_write.sum` of that launch under the key in a JSON table; `bench.py` reports
that figure as `roofline.traffic`.  `launches` aggregates the launch list of a whole
command (the `gpu__time_duration.sum` pass) per kernel: launches, total time, share.

The reference keeps its profiling notes in its README (README.md:197-235); nothing here
is on the product path.
"""

from __future__ import annotations

import argparse
import collections
import csv
import json
import os
import subprocess

KEYS = [
    ("gpu__time_duration.sum", "kernel duration"),
    ("sm__cycles_elapsed.avg.per_second", "SM clock during capture"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed", "tensor pipe active, % of peak"),
    ("sm__inst_executed_pipe_xu.avg.pct_of_peak_sustained_elapsed", "XU (ex2) pipe, % of peak"),
    ("sm__inst_executed_pipe_fma.avg.pct_of_peak_sustained_active", "FMA pipe, % of peak"),
    ("smsp__issue_active.avg.pct_of_peak_sustained_active", "issue slots busy, %"),
    ("l1tex__data_pipe_tc_wavefronts_mem_shared.sum.pct_of_peak_sustained_elapsed",
     "shared-memory data pipe: tensor-core operand reads, % of peak"),
    ("l1tex__data_pipe_lsu_wavefronts_mem_shared.sum.pct_of_peak_sustained_elapsed",
     "shared-memory data pipe: ld/st.shared, % of peak"),
    ("l1tex__data_bank_conflicts_pipe_lsu_mem_shared.sum", "shared-memory bank conflicts"),
    ("l1tex__m_xbar2l1tex_read_bytes_mem_global_op_tma_ld.sum", "TMA loads, L2 -> SM"),
    ("l1tex__m_l1tex2xbar_write_bytes_mem_global_op_tma_red.sum", "TMA add-reductions, SM -> L2"),
    ("lts__t_sector_hit_rate.pct", "L2 hit rate, %"),
    ("dram__bytes_read.sum", "DRAM bytes read"),
    ("dram__bytes_write.sum", "DRAM bytes written"),
    ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "DRAM throughput, % of peak"),
    ("sm__warps_active.avg.pct_of_peak_sustained_active", "achieved occupancy, %"),
    ("launch__registers_per_thread", "registers / thread"),
    ("smsp__inst_executed.sum", "warp instructions executed"),
    ("launch__grid_size", "grid"),
    ("launch__block_size", "block"),
]

_UNIT_BYTES = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12}


def read_report(path: str, launch: int = 0) -> dict[str, tuple[str, str]]:
  """{metric: (unit, value)} of one captured launch of an .ncu-rep file, or of the CSV that
  `ncu -i REPORT --page raw --csv` printed for it."""
  if path.endswith(".csv"):
    with open(path) as f:
      out = f.read()
  else:
    out = subprocess.run(["ncu", "-i", path, "--page", "raw", "--csv"], capture_output=True, text=True, check=True).stdout
  rows = list(csv.reader(out.splitlines()))
  header, units, values = rows[0], rows[1], rows[2 + launch]
  return {h: (u, v) for h, u, v in zip(header, units, values)}


def dram_bytes(metrics) -> float | None:
  total = 0.0
  for key in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
    if key not in metrics:
      return None
    unit, value = metrics[key]
    total += float(value.replace(",", "")) * _UNIT_BYTES.get(unit, 1.0)
  return total


def summary_text(metrics, title: str, command: str, notes: str = "") -> str:
  lines = [f"# {title}", "", "Command (one B200; the same command had just exited 0 without ncu):", "",
           f"    {command}", "", "| metric | value |", "|---|---|"]
  for key, label in KEYS:
    if key in metrics:
      unit, value = metrics[key]
      lines.append(f"| {label} (`{key}`) | {value} {unit} |")
  stalls = []
  for name, (_, value) in metrics.items():
    if "smsp__average_warps_issue_stalled" in name and name.endswith("_per_issue_active.ratio") and "not_issued" not in name:
      try:
        stalls.append((name.split("issue_stalled_")[1].split("_per_issue")[0], float(value.replace(",", ""))))
      except ValueError:
        pass
  stalls.sort(key=lambda x: -x[1])
  if stalls:
    lines += ["", "Top warp stall reasons (stalled warps per issue-active cycle):", ""]
    lines += [f"* {name}: {value:.2f}" for name, value in stalls[:6]]
  if notes:
    lines += ["", notes]
  return "\n".join(lines) + "\n"


def launches_text(csv_path: str, title: str, command: str, notes: str = "") -> str:
  rows = list(csv.reader(open(csv_path)))
  header, agg = None, collections.OrderedDict()
  for r in rows:
    if r and r[0] == "ID":
      header = r
      continue
    if header and len(r) == len(header):
      d = dict(zip(header, r))
      name = d["Kernel Name"].split("(")[0].replace("void ", "")[:90]
      value = float(d["Metric Value"].replace(",", ""))
      scale = {"ns": 1e-3, "us": 1.0, "ms": 1e3, "s": 1e6, "nsecond": 1e-3, "usecond": 1.0, "msecond": 1e3,
               "second": 1e6}.get(d.get("Metric Unit", "ns"), 1e-3)
      a = agg.setdefault((name, d["Grid Size"], d["Block Size"]), [0, 0.0])
      a[0] += 1
      a[1] += value * scale
  total = sum(a[1] for a in agg.values()) or 1.0
  out = [f"# {title}", "", "Command (on one B200, after the same command exited 0 without ncu):", "",
         f"    {command}", "",
         "Per-launch times under ncu are cold-cache and serialised; the SHARE column is what carries over.", "",
         "| kernel | grid | block | launches | total us | share |", "|---|---|---|---|---|---|"]
  for (name, grid, block), (count, us) in agg.items():
    out.append(f"| `{name}` | {grid} | {block} | {count} | {us:.1f} | {100 * us / total:.1f}% |")
  if notes:
    out += ["", notes]
  return "\n".join(out) + "\n"


def main(argv=None) -> None:
  p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
  sub = p.add_subparsers(dest="mode", required=True)
  s = sub.add_parser("summary")
  s.add_argument("report")
  s.add_argument("--launch", type=int, default=0, help="which captured launch of the report")
  s.add_argument("--traffic-key")
  s.add_argument("--traffic-json", default=os.path.join("profiles", "traffic.json"))
  l = sub.add_parser("launches")
  l.add_argument("report")
  for q in (s, l):
    q.add_argument("--title", required=True)
    q.add_argument("--command", required=True)
    q.add_argument("--out", required=True)
    q.add_argument("--notes", default="")
  args = p.parse_args(argv)
  if args.mode == "summary":
    metrics = read_report(args.report, args.launch)
    text = summary_text(metrics, args.title, args.command, args.notes)
    if args.traffic_key:
      table = {}
      if os.path.exists(args.traffic_json):
        with open(args.traffic_json) as f:
          table = json.load(f)
      table[args.traffic_key] = dram_bytes(metrics)
      with open(args.traffic_json, "w") as f:
        json.dump(table, f, indent=1, sort_keys=True)
        f.write("\n")
  else:
    text = launches_text(args.report, args.title, args.command, args.notes)
  with open(args.out, "w") as f:
    f.write(text)
  print(text)


if __name__ == "__main__":
  main()
