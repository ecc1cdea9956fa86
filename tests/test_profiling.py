"""The ncu-summary helper on a hand-made raw CSV (the layout `ncu --page raw --csv` prints:
a header row, a units row, one row per captured launch) and a hand-made launch list."""

import json

from splash_attention_mgpu import profiling


def _write_raw(path):
  header = ["ID", "Kernel Name", "gpu__time_duration.sum", "dram__bytes_read.sum", "dram__bytes_write.sum",
            "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed",
            "smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio",
            "smsp__average_warps_issue_stalled_wait_per_issue_active.ratio"]
  units = ["", "", "ms", "Mbyte", "Mbyte", "%", "inst", "inst"]
  rows = [["0", "k0", "1.5", "400.0", "200.0", "61.0", "4.25", "1.30"],
          ["1", "k1", "0.5", "1.0", "2.0", "30.0", "0.5", "2.5"]]
  with open(path, "w") as f:
    for r in (header, units, *rows):
      f.write(",".join(f'"{x}"' for x in r) + "\n")


def test_summary_and_traffic_table(tmp_path):
  raw = tmp_path / "raw.csv"
  _write_raw(raw)
  out, table = tmp_path / "k.md", tmp_path / "traffic.json"
  profiling.main(["summary", str(raw), "--title", "a kernel", "--command", "ncu ... python bench.py", "--out", str(out),
                  "--traffic-key", "bwd:w", "--traffic-json", str(table), "--notes", "Reading: none."])
  text = out.read_text()
  assert text.startswith("# a kernel") and "ncu ... python bench.py" in text and "Reading: none." in text
  assert "| kernel duration (`gpu__time_duration.sum`) | 1.5 ms |" in text
  assert text.index("long_scoreboard: 4.25") < text.index("wait: 1.30")
  assert json.loads(table.read_text()) == {"bwd:w": 600e6}
  # The second captured launch of the same report, added to the same table.
  profiling.main(["summary", str(raw), "--launch", "1", "--title", "t", "--command", "c", "--out", str(out),
                  "--traffic-key", "fwd:w", "--traffic-json", str(table)])
  assert json.loads(table.read_text()) == {"bwd:w": 600e6, "fwd:w": 3e6}
  assert "wait: 2.50" in out.read_text()


def test_launch_list(tmp_path):
  csv_path = tmp_path / "launches.csv"
  lines = ['==PROF== Connected', '"ID","Process ID","Kernel Name","Grid Size","Block Size","Metric Name","Metric Unit","Metric Value"',
           '"0","1","void splash::a<1>(int)","(8, 1, 1)","(256, 1, 1)","gpu__time_duration.sum","us","10.0"',
           '"1","1","void splash::b<2>(int)","(4, 1, 1)","(128, 1, 1)","gpu__time_duration.sum","us","30.0"',
           '"2","1","void splash::a<1>(int)","(8, 1, 1)","(256, 1, 1)","gpu__time_duration.sum","ns","10000"']
  csv_path.write_text("\n".join(lines) + "\n")
  out = tmp_path / "l.md"
  profiling.main(["launches", str(csv_path), "--title", "list", "--command", "ncu --metrics ...", "--out", str(out)])
  text = out.read_text()
  assert "| `splash::a<1>` | (8, 1, 1) | (256, 1, 1) | 2 | 20.0 | 40.0% |" in text
  assert "| `splash::b<2>` | (4, 1, 1) | (128, 1, 1) | 1 | 30.0 | 60.0% |" in text
