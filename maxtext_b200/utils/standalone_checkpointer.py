"""Checkpoint save / restore loop without training: `python -m maxtext_b200.utils.standalone_checkpointer <yml> key=value ...`.

The role of src/maxtext/utils/standalone_checkpointer.py (161 lines): build the training state for the configured model and
mesh, then for `steps` iterations save every `checkpoint_period` steps (perturbing the parameters in between so that each
step directory differs), wait for the writes and report save / restore wall time and bytes per second.
"""
from __future__ import annotations

import json
import sys
import time

import torch

from ..config import pyconfig
from ..checkpoint import manager as ckpt_lib
from ..train import train as train_lib
from . import max_logging


def checkpoint_loop(config) -> dict:
  config, mesh, engine = train_lib.setup(config)
  engine.store.ensure_grad_buffers()
  mgr = ckpt_lib.CheckpointManager(config, engine, mesh)
  restored = mgr.restore_if_possible(None)
  start = restored or 0
  nbytes = engine.store.master.numel() * engine.store.master.element_size() * (1 + len(engine.optimizer.state_arrays()))
  saves, t_save = 0, 0.0
  for step in range(start, int(config.steps)):
    engine.store.master.add_(1e-4)           # stand-in for a train step: every checkpoint differs
    engine.store.sync_compute_from_master()
    engine.step_count = step + 1
    if mgr.should_save(step):
      t0 = time.perf_counter()
      mgr.save(step, None, force=True)
      t_save += time.perf_counter() - t0
      saves += 1
  mgr.wait_until_finished()
  t0 = time.perf_counter()
  st = engine.store
  before = {n: st.full_master(p).clone() for n, p in st.params.items()}
  st.master.zero_()
  got = mgr.restore_if_possible(None)
  t_restore = time.perf_counter() - t0
  exact = all(torch.equal(before[n], st.full_master(p)) for n, p in st.params.items())
  out = {"saves": saves, "save_seconds": round(t_save, 4), "restore_seconds": round(t_restore, 4), "restored_step": got,
         "bytes_per_rank": int(nbytes), "save_gb_per_s": round(saves * nbytes / max(t_save, 1e-9) / 1e9, 3),
         "roundtrip_exact": bool(got is not None and (not mgr.should_save(int(config.steps) - 1) or exact))}
  max_logging.log(json.dumps(out))
  return out


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  return checkpoint_loop(pyconfig.initialize(argv + ["enable_checkpointing=true"] if not any(a.startswith("enable_checkpointing=") for a in argv) else argv))


if __name__ == "__main__":
  main()
