"""Strip a full training checkpoint down to its parameters:
`python -m maxtext_b200.utils.generate_param_only_checkpoint <yml> load_full_state_path=CKPT/STEP base_output_directory=OUT run_name=NAME`.

The role of src/maxtext/utils/generate_param_only_checkpoint.py (509 lines: drop the optimizer state, optionally unroll the
scanned layer axis, write a checkpoint that decode / fine-tuning load through `load_parameters_path`). The output keeps the
source's layer layout unless `force_unroll=true`, in which case stacked `layers` arrays are written per layer.
"""
from __future__ import annotations

import os
import sys

import torch

from ..checkpoint import manager as ckpt_lib
from ..config import pyconfig
from ..train.engine import TrainEngine
from . import max_logging


def generate(config) -> str:
  src = config.load_full_state_path or config.load_parameters_path
  if not src:
    raise SystemExit("load_full_state_path=<checkpoint step directory> is required")
  engine = TrainEngine(config, None, torch.device("cpu"), init=False)
  ckpt_lib.load_params_only(src, engine)
  out_cfg = config.replace(scan_layers=False) if config.force_unroll else config
  engine.config = out_cfg
  mgr = ckpt_lib.CheckpointManager(out_cfg, engine, None)
  mgr.save_params_only(0)
  path = os.path.join(mgr.dir, "0", "items")
  max_logging.log(f"parameter-only checkpoint written to {path}")
  return path


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  return generate(pyconfig.initialize(argv + ["hardware=cpu"], num_devices=1))


if __name__ == "__main__":
  main()
