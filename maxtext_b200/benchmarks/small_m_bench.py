"""Decode-sized GEMM (M <= 64): the weight-streaming kernel against the library's `torch.mm`, as a fraction of the HBM floor.

  python -m maxtext_b200.benchmarks.small_m_bench [--out FILE]

Shapes are Llama-3-8B's decode projections (qkv 6144 x 4096, out 4096 x 4096, gate|up 28672 x 4096, down 4096 x 14336, head
128256 x 4096). Each timed call uses the next of several weight copies that together exceed the L2 cache, so every call streams
from HBM; CUDA events, 3 warm-up + 20 timed calls. The floor is N * K * 2 bytes over the measured copy bandwidth
(`MEASURED_PEAKS.json` `hbm_gbs`, else 6650 GB/s)."""
from __future__ import annotations

import argparse
import json
import os

import torch

SHAPES = [("qkv", 6144, 4096), ("attn_out", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336), ("head", 128256, 4096)]


def _time(fn, n_warm=3, n=20):
  for i in range(n_warm):
    fn(i)
  torch.cuda.synchronize()
  a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  a.record()
  for i in range(n):
    fn(n_warm + i)
  b.record()
  torch.cuda.synchronize()
  return a.elapsed_time(b) / n * 1e-3


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument("--out", default="")
  ap.add_argument("--m", default="1,8,32,64")
  args = ap.parse_args(argv)
  from maxtext_b200.ops import backend
  E = backend.ext(required=True)
  peak = 6650.0
  root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
  try:
    peak = float(json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))["hbm_gbs"])
  except Exception:  # pylint: disable=broad-except
    pass
  rows = []
  for name, N, K in SHAPES:
    copies = max(2, int(300e6 // (N * K * 2)) + 1)                 # > 126 MB of L2 between two uses of the same copy
    ws = [torch.randn(N, K, device="cuda").bfloat16() for _ in range(copies)]
    for M in [int(v) for v in args.m.split(",")]:
      x = torch.randn(M, K, device="cuda").bfloat16()
      out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
      t_own = _time(lambda i: E.gemm_small_m(x, ws[i % copies], out))
      t_lib = _time(lambda i: torch.mm(x, ws[i % copies].t(), out=out))
      floor = N * K * 2 / (peak * 1e9)
      rows.append({"shape": name, "M": M, "N": N, "K": K, "own_us": round(t_own * 1e6, 2), "library_us": round(t_lib * 1e6, 2),
                   "floor_us": round(floor * 1e6, 2), "own_frac_of_measured_hbm": round(floor / t_own, 3),
                   "library_frac_of_measured_hbm": round(floor / t_lib, 3)})
      print(json.dumps(rows[-1]), flush=True)
    del ws
    torch.cuda.empty_cache()
  if args.out:
    with open(args.out, "w") as fh:
      json.dump(rows, fh, indent=1)


if __name__ == "__main__":
  main()
