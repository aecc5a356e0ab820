"""MLPerf-inference Offline scenario for the serving engine (src/maxtext/inference/mlperf/offline_mode.py:55-485,
offline_inference.py).

The Offline scenario hands the system under test ALL queries at once and measures samples per second. Here:

  * queries are sorted into prefill-length buckets (`--prefill_lengths_and_batch_sizes "256,80|512,40|1024,20"`: a query goes
    to the smallest bucket that holds its prompt; each bucket runs with its own number of decode slots);
  * every bucket is served by an `OfflineEngine` (continuous batching over the bucket's slots) on one shared `MaxEngine`;
  * the run writes `mlperf_log_accuracy.json` in LoadGen's format (one entry per sample: `qsl_idx` and the generated token
    ids as little-endian int64 bytes in hex) and `mlperf_log_summary.txt` (samples/s, tokens/s, per-bucket counts).

When the `mlperf_loadgen` package is importable the same system under test is driven by the real LoadGen
(`--use_loadgen`); it is not part of this environment, so the built-in driver below is what the tests exercise.
The dataset is a JSON-lines file or a pandas pickle with the columns `tok_input` (token ids) and optionally `tok_input_length`
and `output` / `tok_output` (reference), the layout of the OpenOrca and Llama-2-70B MLPerf sets.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import numpy as np
import torch


def parse_args(argv=None):
  p = argparse.ArgumentParser(description="MLPerf-style offline inference run")
  p.add_argument("config", nargs="*", help="base.yml followed by key=value overrides for the engine")
  p.add_argument("--mlperf_test_mode", default="performance", choices=["performance", "accuracy", "submission"])
  p.add_argument("--dataset_path", required=True)
  p.add_argument("--total_sample_count", type=int, default=24576)
  p.add_argument("--output_log_dir", default="output-logs")
  p.add_argument("--prefill_lengths_and_batch_sizes", default="256,80|512,40|1024,20")
  p.add_argument("--tok_outlen_multiplier", type=float, default=3.0, help="output budget = multiplier x prompt length, capped by the cache")
  p.add_argument("--max_new_tokens", type=int, default=0, help="fixed output budget (overrides the multiplier)")
  p.add_argument("--allow_skipping_queries", action="store_true", help="skip prompts longer than the largest bucket instead of failing")
  p.add_argument("--rename_dataset_cols", default="", help='JSON dict, e.g. {"tok_input_len": "tok_input_length"}')
  p.add_argument("--skip_warmup", action="store_true")
  p.add_argument("--use_loadgen", action="store_true")
  return p.parse_args(argv)


def load_dataset(path: str, rename: str = "", limit: int = 0) -> list[dict]:
  """-> [{"tok_input": [...], "tok_input_length": n, ...}] in file order."""
  ren = json.loads(rename) if rename else {}
  if path.endswith((".pkl", ".pickle")):
    import pandas as pd
    df = pd.read_pickle(path)
    if ren:
      df = df.rename(columns=ren)
    rows = df.to_dict("records")
  else:
    with open(path, "r", encoding="utf-8") as fh:
      rows = [json.loads(line) for line in fh if line.strip()]
    rows = [{ren.get(k, k): v for k, v in r.items()} for r in rows]
  out = []
  for r in rows[: limit or None]:
    toks = [int(t) for t in r["tok_input"]]
    out.append({**r, "tok_input": toks, "tok_input_length": int(r.get("tok_input_length", len(toks)))})
  return out


def parse_buckets(spec: str) -> list[tuple[int, int]]:
  out = sorted((int(a), int(b)) for a, b in (item.split(",") for item in spec.split("|") if item))
  if not out:
    raise ValueError("no prefill buckets given")
  return out


def classify(rows: list[dict], buckets: list[tuple[int, int]], allow_skip: bool) -> dict[int, list[int]]:
  """bucket length -> sample indices whose prompt fits it (smallest fitting bucket)."""
  by = {length: [] for length, _ in buckets}
  for i, r in enumerate(rows):
    n = r["tok_input_length"]
    fit = [length for length, _ in buckets if n <= length]
    if fit:
      by[fit[0]].append(i)
    elif not allow_skip:
      raise ValueError(f"sample {i}: prompt of {n} tokens exceeds the largest prefill bucket {buckets[-1][0]} (pass --allow_skipping_queries to drop it)")
  return by


def response_bytes(token_ids) -> str:
  """LoadGen's accuracy log stores the response buffer as hex: int64 token ids, little endian."""
  return np.asarray(list(token_ids), dtype="<i8").tobytes().hex()


class SUT:
  """System under test: serves buckets one after another, largest batch first, on one engine."""

  def __init__(self, engine, rows, buckets, args, eos_id: int = -1):
    self.engine, self.rows, self.buckets, self.args, self.eos_id = engine, rows, buckets, args, eos_id
    self.max_len = int(engine.config.max_target_length)

  def budget(self, n_prompt: int) -> int:
    if self.args.max_new_tokens > 0:
      want = self.args.max_new_tokens
    else:
      want = int(math_ceil(self.args.tok_outlen_multiplier * n_prompt))
    return max(1, min(want, self.max_len - n_prompt - 1))

  def issue_queries(self, indices: list[int]) -> dict[int, list[int]]:
    from ..offline_engine import OfflineEngine
    by = classify([self.rows[i] for i in indices], self.buckets, self.args.allow_skipping_queries)
    results: dict[int, list[int]] = {}
    for length, slots in sorted(self.buckets, key=lambda b: -b[1]):
      local = by.get(length, [])
      if not local:
        continue
      off = OfflineEngine(self.engine, slots=min(slots, max(1, len(local))), eos_id=self.eos_id)
      reqs = []
      for j in local:
        row = self.rows[indices[j]]
        toks = row["tok_input"][: row["tok_input_length"]]
        reqs.append((indices[j], off.submit(toks, max_new_tokens=self.budget(len(toks)))))
      off.run_until_done()
      for idx, r in reqs:
        results[idx] = list(r.output)
    return results


def math_ceil(x: float) -> int:
  return int(-(-x // 1))


def run(args, engine=None) -> dict:
  from ...config import pyconfig
  from ..maxengine import MaxEngine
  if engine is None:
    cfg = pyconfig.initialize(["mlperf"] + list(args.config))
    engine = MaxEngine(cfg)
    engine.load_params()
  rows = load_dataset(args.dataset_path, args.rename_dataset_cols, args.total_sample_count)
  buckets = parse_buckets(args.prefill_lengths_and_batch_sizes)
  for length, _ in buckets:
    if length >= int(engine.config.max_target_length):
      raise ValueError(f"prefill bucket {length} leaves no room to generate within max_target_length={engine.config.max_target_length}")
  sut = SUT(engine, rows, buckets, args)
  indices = list(range(len(rows)))
  if not args.skip_warmup and indices:
    sut.issue_queries(indices[: min(2, len(indices))])              # builds caches / graphs outside the timed region
  if args.use_loadgen:
    return _run_with_loadgen(sut, indices, args)
  if engine.device.type == "cuda":
    torch.cuda.synchronize()
  t0 = time.perf_counter()
  results = sut.issue_queries(indices)
  if engine.device.type == "cuda":
    torch.cuda.synchronize()
  dt = time.perf_counter() - t0
  n_tok = sum(len(v) for v in results.values())
  summary = {"scenario": "Offline", "mode": args.mlperf_test_mode, "samples": len(results), "skipped": len(indices) - len(results),
             "seconds": dt, "samples_per_second": len(results) / dt if dt > 0 else 0.0, "tokens_per_second": n_tok / dt if dt > 0 else 0.0,
             "generated_tokens": n_tok, "buckets": {str(k): len(v) for k, v in classify(rows, buckets, True).items()}}
  os.makedirs(args.output_log_dir, exist_ok=True)
  with open(os.path.join(args.output_log_dir, "mlperf_log_summary.txt"), "w", encoding="utf-8") as fh:
    fh.write("================================================\nMLPerf Results Summary (built-in offline driver)\n================================================\n")
    for k, v in summary.items():
      fh.write(f"{k} : {v}\n")
  if args.mlperf_test_mode in ("accuracy", "submission"):
    log = [{"seq_id": n, "qsl_idx": i, "data": response_bytes(results[i]), "token_count": len(results[i])} for n, i in enumerate(sorted(results))]
    with open(os.path.join(args.output_log_dir, "mlperf_log_accuracy.json"), "w", encoding="utf-8") as fh:
      json.dump(log, fh)
  return summary


def _run_with_loadgen(sut: SUT, indices, args) -> dict:
  """The same system under test behind the real LoadGen (only when `mlperf_loadgen` is installed)."""
  import array
  import mlperf_loadgen as lg                                     # pylint: disable=import-error
  settings = lg.TestSettings()
  settings.scenario = lg.TestScenario.Offline
  settings.mode = lg.TestMode.AccuracyOnly if args.mlperf_test_mode == "accuracy" else lg.TestMode.PerformanceOnly
  keep = []

  def issue(queries):
    res = sut.issue_queries([q.index for q in queries])
    out = []
    for q in queries:
      buf = array.array("B", np.asarray(res.get(q.index, []), dtype="<i8").tobytes())
      keep.append(buf)
      addr, n = buf.buffer_info()
      out.append(lg.QuerySampleResponse(q.id, addr, n * buf.itemsize, len(res.get(q.index, []))))
    lg.QuerySamplesComplete(out)
  s = lg.ConstructSUT(issue, lambda: None)
  q = lg.ConstructQSL(len(indices), len(indices), lambda _: None, lambda _: None)
  log_settings = lg.LogSettings()
  log_settings.log_output.outdir = args.output_log_dir
  os.makedirs(args.output_log_dir, exist_ok=True)
  lg.StartTestWithLogSettings(s, q, settings, log_settings)
  lg.DestroyQSL(q)
  lg.DestroySUT(s)
  return {"scenario": "Offline", "driver": "mlperf_loadgen", "log_dir": args.output_log_dir}


def main(argv=None):
  print(json.dumps(run(parse_args(argv))))


if __name__ == "__main__":
  main()
