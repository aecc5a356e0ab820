"""Run a named recipe on this node: `python -m maxtext_b200.benchmarks.benchmark_runner --recipe llama3_8b_8192_fsdp8 [--dry-run]`.

The role of benchmarks/benchmark_runner.py (on-device mode): resolve the recipe, launch one process per GPU with
torch.distributed.run on 127.0.0.1, stream the training log and print the last throughput line as JSON. `--plan` prints the
ahead-of-time memory / traffic plan instead of running (no GPU needed); `--list` shows the table.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys

from .recipes import RECIPES

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
BASE = os.path.join(ROOT, "maxtext_b200", "configs", "base.yml")


def command(recipe, extra=()) -> list[str]:
  over = recipe.overrides() + list(extra)
  if recipe.gpus == 1:
    return [sys.executable, "-m", "maxtext_b200.train.train", BASE] + over
  return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={recipe.gpus}", "--master-addr", "127.0.0.1",
          "--master-port", "29611", "-m", "maxtext_b200.train.train", BASE] + over


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument("--recipe", default="")
  ap.add_argument("--list", action="store_true")
  ap.add_argument("--dry-run", action="store_true", help="print the command only")
  ap.add_argument("--plan", action="store_true", help="ahead-of-time plan (memory, traffic, roofline) instead of running")
  ap.add_argument("overrides", nargs="*", help="extra key=value overrides")
  a = ap.parse_args(argv)
  if a.list or not a.recipe:
    for r in RECIPES.values():
      print(f"{r.name:34s} {r.model:16s} gpus={r.gpus}  {r.note}")
    return 0
  r = RECIPES[a.recipe]
  if a.plan:
    from ..config import pyconfig
    from ..train import train_compile
    cfg = pyconfig.initialize(["plan", BASE] + r.overrides() + list(a.overrides) + ["log_config=false"], num_devices=r.gpus)
    p = train_compile.plan(cfg, r.gpus)
    print(json.dumps({k: v for k, v in p.items() if k != "units"}, indent=1))
    return 0 if p["fits"] else 1
  cmd = command(r, a.overrides)
  if a.dry_run:
    print(" ".join(cmd))
    return 0
  last = None
  with subprocess.Popen(cmd, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) as proc:
    for line in proc.stdout:
      sys.stdout.write(line)
      m = re.search(r"completed step: (\d+), seconds: ([0-9.]+), TFLOP/s/device: ([0-9.]+), Tokens/s/device: ([0-9.]+)", line)
      if m:
        last = {"step": int(m.group(1)), "seconds": float(m.group(2)), "tflops_per_device": float(m.group(3)),
                "tokens_per_s_per_device": float(m.group(4))}
    rc = proc.wait()
  print(json.dumps({"recipe": r.name, "gpus": r.gpus, "returncode": rc, "last_step": last}))
  return rc


if __name__ == "__main__":
  sys.exit(main())
