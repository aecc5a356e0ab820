"""Local results database for benchmark runs (the role of benchmarks/benchmark_db_writer/ and upload_metrics_to_bq.py, which
write to BigQuery): one SQLite file, one row per run, the metrics as columns and the full configuration as JSON.

  python -m maxtext_b200.benchmarks.results_db add runs.sqlite '{"metric": ..., "value": ...}'      # e.g. a bench.py JSON line
  python -m maxtext_b200.benchmarks.results_db best runs.sqlite --model llama3-8b --gpus 8
"""
from __future__ import annotations

import json
import sqlite3
import sys
import time

SCHEMA = """CREATE TABLE IF NOT EXISTS runs (
  id INTEGER PRIMARY KEY AUTOINCREMENT, created REAL, model TEXT, metric TEXT, value REAL, unit TEXT, n_gpus INTEGER, ms_per_step REAL,
  e2e_value REAL, parallelism TEXT, dtype TEXT, sm_mhz REAL, throttle TEXT, software TEXT, record TEXT)"""


class ResultsDB:
  def __init__(self, path: str):
    self.con = sqlite3.connect(path)
    self.con.execute(SCHEMA)
    self.con.commit()

  def add(self, record: dict, software: str = "") -> int:
    """`record`: the JSON line `bench.py` prints (other dictionaries with `metric` / `value` work too)."""
    if "metric" not in record or "value" not in record:
      raise ValueError("a run record needs `metric` and `value`")
    cfg, clocks, e2e = record.get("config") or {}, record.get("clocks") or {}, record.get("e2e") or {}
    cur = self.con.execute(
        "INSERT INTO runs (created, model, metric, value, unit, n_gpus, ms_per_step, e2e_value, parallelism, dtype, sm_mhz, throttle, software, record)"
        " VALUES (?,?,?,?,?,?,?,?,?,?,?,?,?,?)",
        (time.time(), str(cfg.get("model", record.get("model", ""))), str(record["metric"]), float(record["value"]), str(record.get("unit", "")),
         int(record.get("n_gpus", 1)), float(record.get("ms_per_step", 0.0) or 0.0), float(e2e.get("value", 0.0) or 0.0),
         str(cfg.get("parallelism", "")), str(record.get("dtype", "")), float(clocks.get("sm_mhz", 0.0) or 0.0),
         ",".join(clocks.get("reasons") or []), software, json.dumps(record)))
    self.con.commit()
    return int(cur.lastrowid)

  def query(self, model: str | None = None, gpus: int | None = None, metric: str | None = None) -> list[dict]:
    q, args = "SELECT id, created, model, metric, value, unit, n_gpus, ms_per_step, e2e_value, parallelism, throttle FROM runs WHERE 1=1", []
    for col, v in (("model", model), ("n_gpus", gpus), ("metric", metric)):
      if v is not None:
        q += f" AND {col} = ?"
        args.append(v)
    cols = ["id", "created", "model", "metric", "value", "unit", "n_gpus", "ms_per_step", "e2e_value", "parallelism", "throttle"]
    return [dict(zip(cols, row)) for row in self.con.execute(q + " ORDER BY id", args)]

  def best(self, model: str | None = None, gpus: int | None = None, metric: str | None = None, higher_is_better: bool = True,
           ignore_throttled: bool = True) -> dict | None:
    """The best run; runs whose clock record shows a thermal or hardware slowdown are left out (their numbers are not valid)."""
    rows = self.query(model, gpus, metric)
    if ignore_throttled:
      rows = [r for r in rows if not any(t in r["throttle"] for t in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"))]
    if not rows:
      return None
    return (max if higher_is_better else min)(rows, key=lambda r: r["value"])

  def record(self, run_id: int) -> dict:
    row = self.con.execute("SELECT record FROM runs WHERE id = ?", (run_id,)).fetchone()
    return json.loads(row[0]) if row else {}

  def close(self):
    self.con.close()


def main(argv=None):
  argv = list(sys.argv[1:] if argv is None else argv)
  if len(argv) >= 3 and argv[0] == "add":
    db = ResultsDB(argv[1])
    print(db.add(json.loads(argv[2] if argv[2] != "-" else sys.stdin.read())))
    return 0
  if len(argv) >= 2 and argv[0] == "best":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--model")
    ap.add_argument("--gpus", type=int)
    ap.add_argument("--metric")
    a = ap.parse_args(argv[2:])
    print(json.dumps(ResultsDB(argv[1]).best(a.model, a.gpus, a.metric)))
    return 0
  print(__doc__)
  return 2


if __name__ == "__main__":
  sys.exit(main())
