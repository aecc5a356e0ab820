"""Scores an `mlperf_log_accuracy.json` against the dataset's references (src/maxtext/inference/mlperf/evaluate-accuracy.py):
ROUGE-1 / 2 / L of the decoded generations, generated-token statistics.

  python -m maxtext_b200.inference.mlperf.evaluate_accuracy --mlperf-accuracy-file LOG --dataset-file DATA base.yml tokenizer_type=...
"""
from __future__ import annotations

import argparse
import json

import numpy as np


def decode_log(path: str) -> dict[int, list[int]]:
  with open(path, "r", encoding="utf-8") as fh:
    log = json.load(fh)
  out = {}
  for e in log:
    if e["qsl_idx"] in out:
      continue                                                    # LoadGen may log a sample twice; the first entry counts
    out[int(e["qsl_idx"])] = np.frombuffer(bytes.fromhex(e["data"]), dtype="<i8").tolist()
  return out


def evaluate(log_path: str, rows: list[dict], tokenizer) -> dict:
  from ...eval.scoring import rouge
  gen = decode_log(log_path)
  idx = sorted(gen)
  preds = [tokenizer.decode([t for t in gen[i] if t >= 0]) for i in idx]
  refs = []
  for i in idx:
    r = rows[i]
    refs.append(r["output"] if "output" in r else tokenizer.decode(list(r.get("tok_output", []))))
  res = rouge(preds, refs)
  lens = [len(gen[i]) for i in idx]
  res.update(gen_len=int(sum(lens)), gen_num=len(idx), tokens_per_sample=float(np.mean(lens)) if lens else 0.0)
  return res


def main(argv=None):
  from ...config import pyconfig
  from ...input_pipeline.tokenizer import build_tokenizer
  from .offline_mode import load_dataset
  p = argparse.ArgumentParser()
  p.add_argument("config", nargs="+")
  p.add_argument("--mlperf-accuracy-file", required=True)
  p.add_argument("--dataset-file", required=True)
  a = p.parse_args(argv)
  cfg = pyconfig.initialize(["eval"] + list(a.config))
  print(json.dumps(evaluate(a.mlperf_accuracy_file, load_dataset(a.dataset_file), build_tokenizer(cfg))))


if __name__ == "__main__":
  main()
