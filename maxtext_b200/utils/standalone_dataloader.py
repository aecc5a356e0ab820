"""Input-pipeline throughput without a model: `python -m maxtext_b200.utils.standalone_dataloader <yml> key=value ...`.

The role of src/maxtext/utils/standalone_dataloader.py (78 lines): iterate the configured data iterator for `steps` batches
(optionally moving each batch to the device as training does) and report batches, tokens per second and time to first batch.
"""
from __future__ import annotations

import json
import sys
import time

import torch

from ..config import pyconfig
from ..parallel import mesh as mesh_lib
from ..train import train as train_lib
from . import max_logging


def data_load_loop(config, to_device: bool = False) -> dict:
  rank, world, _ = mesh_lib.init_distributed(int(config.jax_distributed_initialization_timeout))
  mesh = mesh_lib.mesh_from_config(config, rank=rank, world=world) if world > 1 else None
  t0 = time.perf_counter()
  it = train_lib.create_data_iterator(config, mesh)
  first = next(it)
  t_first = time.perf_counter() - t0
  dev = torch.device("cuda") if (to_device and torch.cuda.is_available()) else None
  tokens, n = first["inputs"].numel(), 1
  t1 = time.perf_counter()
  for _ in range(int(config.steps) - 1):
    b = next(it)
    if dev is not None:
      b = {k: v.to(dev, non_blocking=True) for k, v in b.items() if torch.is_tensor(v)}
    tokens += b["inputs"].numel()
    n += 1
  if dev is not None:
    torch.cuda.synchronize()
  dt = time.perf_counter() - t1
  out = {"batches": n, "first_batch_seconds": round(t_first, 4), "tokens_per_second": round((tokens - first["inputs"].numel()) / max(dt, 1e-9), 1),
         "rows_per_batch": int(first["inputs"].shape[0]), "seq_len": int(first["inputs"].shape[1])}
  max_logging.log(json.dumps(out))
  return out


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  return data_load_loop(pyconfig.initialize(argv))


if __name__ == "__main__":
  main()
