"""Compare two sets of weights tensor by tensor (tools/weight_inspector/weight_inspector.py).

  python -m maxtext_b200.utils.weight_inspector --lhs a.safetensors --rhs b.safetensors [--atol 1e-5] [--rtol 1e-3] [--pattern 'layers_0']

Each side is a .safetensors file, a directory of them (HuggingFace shards), or a torch `.pt` state dict loaded with
`weights_only=True` (pickles that execute code are not loaded). Reports keys present on one side only, shape or dtype
mismatches, and for every common tensor the largest absolute and relative difference; the exit code is 1 if anything differs
beyond the tolerances."""
from __future__ import annotations

import argparse
import glob
import json
import os
import re
import sys

import torch


def load_weights(path: str) -> dict:
  if os.path.isdir(path):
    out = {}
    for f in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
      out.update(load_weights(f))
    if not out:
      raise FileNotFoundError(f"no .safetensors files under {path}")
    return out
  if path.endswith(".safetensors"):
    from safetensors.torch import load_file
    return load_file(path)
  obj = torch.load(path, map_location="cpu", weights_only=True)
  return obj.get("state_dict", obj) if isinstance(obj, dict) else obj


def compare(lhs: dict, rhs: dict, atol: float = 1e-5, rtol: float = 1e-3, pattern: str | None = None) -> dict:
  rx = re.compile(pattern) if pattern else None
  keep = lambda k: rx is None or rx.search(k)           # noqa: E731
  lk, rk = {k for k in lhs if keep(k)}, {k for k in rhs if keep(k)}
  rep = {"only_lhs": sorted(lk - rk), "only_rhs": sorted(rk - lk), "shape_mismatch": [], "dtype_mismatch": [], "different": [], "equal": 0}
  for k in sorted(lk & rk):
    a, b = lhs[k], rhs[k]
    if tuple(a.shape) != tuple(b.shape):
      rep["shape_mismatch"].append({"key": k, "lhs": list(a.shape), "rhs": list(b.shape)})
      continue
    if a.dtype != b.dtype:
      rep["dtype_mismatch"].append({"key": k, "lhs": str(a.dtype), "rhs": str(b.dtype)})
    af, bf = a.float(), b.float()
    diff = (af - bf).abs()
    if bool((diff <= atol + rtol * bf.abs()).all()):
      rep["equal"] += 1
    else:
      i = int(diff.argmax())
      rep["different"].append({"key": k, "max_abs": float(diff.max()), "max_rel": float((diff / bf.abs().clamp_min(1e-12)).max()),
                               "at": i, "lhs": float(af.reshape(-1)[i]), "rhs": float(bf.reshape(-1)[i]),
                               "fraction": float((diff > atol + rtol * bf.abs()).float().mean())})
  rep["match"] = not (rep["only_lhs"] or rep["only_rhs"] or rep["shape_mismatch"] or rep["different"])
  return rep


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument("--lhs", required=True)
  ap.add_argument("--rhs", required=True)
  ap.add_argument("--atol", type=float, default=1e-5)
  ap.add_argument("--rtol", type=float, default=1e-3)
  ap.add_argument("--pattern", default=None)
  a = ap.parse_args(argv)
  rep = compare(load_weights(a.lhs), load_weights(a.rhs), a.atol, a.rtol, a.pattern)
  print(json.dumps(rep, indent=1))
  return 0 if rep["match"] else 1


if __name__ == "__main__":
  sys.exit(main())
