"""Search the remat policy x per-device batch that fits memory and maximises estimated throughput.

The role of src/maxtext/utils/estimator.py (616 lines: tries remat policies from cheapest recompute to full, growing the
batch until compilation reports OOM). Here every candidate is priced by `train_compile.plan` on the meta device, so a
sweep over dozens of candidates takes seconds and needs no GPU.

  python -m maxtext_b200.utils.estimator <yml> model_name=llama3-8b compile_topology=b200-8 ici_fsdp_parallelism=8
"""
from __future__ import annotations

import json
import sys

from ..config import pyconfig
from ..train import train_compile

POLICIES = ("minimal_with_context", "minimal", "save_dot_except_mlpwi", "save_dot_except_mlp", "save_qkv_proj", "save_out_proj", "full")


def search(argv, world: int | None, part: str = "b200", batches=(0.5, 1, 2, 3, 4, 6, 8, 12, 16, 24, 32), policies=POLICIES) -> list[dict]:
  rows = []
  argv = [a for a in argv if a.split("=")[0] not in ("remat_policy", "per_device_batch_size", "log_config")]
  for pol in policies:
    best = None
    for b in batches:
      try:
        cfg = pyconfig.initialize(list(argv) + [f"remat_policy={pol}", f"per_device_batch_size={b}", "log_config=false"], num_devices=world)
      except Exception:  # pylint: disable=broad-except
        continue      # e.g. a fractional batch that the mesh cannot split
      p = train_compile.plan(cfg, world or cfg.num_target_devices, part)
      if not p["fits"]:
        break
      best = dict(remat_policy=pol, per_device_batch_size=b, memory_gb=p["memory_total_gb"],
                  est_tokens_per_s_per_device=p["per_step"]["est_tokens_per_s_per_device"], est_step_s=p["per_step"]["est_step_s"])
    if best is not None:
      rows.append(best)
  rows.sort(key=lambda r: -r["est_tokens_per_s_per_device"])
  return rows


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  topo = next((a.split("=", 1)[1] for a in argv if a.startswith("compile_topology=")), "")
  part, world = train_compile.parse_topology(topo) if topo else ("b200", None)
  rows = search(argv, world, part)
  for r in rows:
    print(json.dumps(r))
  return 0 if rows else 1


if __name__ == "__main__":
  sys.exit(main())
