"""Worker for the tensor-parallel decode test: greedy-decodes a prompt under the configured mesh and writes the tokens."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
  out_path, overrides = sys.argv[1], sys.argv[2:]
  from maxtext_b200.config import pyconfig
  from maxtext_b200.inference.maxengine import MaxEngine
  from maxtext_b200.parallel import mesh as mesh_lib
  rank, world, _ = mesh_lib.init_distributed(timeout_s=120)
  cfg = pyconfig.initialize(["w", "maxtext_b200/configs/base.yml"] + overrides, num_devices=world)
  mesh = mesh_lib.mesh_from_config(cfg, rank=rank, world=world) if world > 1 else None
  eng = MaxEngine(cfg, mesh=mesh, device="cpu")
  eng.load_params()
  prompt = torch.tensor([5, 9, 2, 7, 3, 11, 4])
  prefix, first = eng.prefill(torch.nn.functional.pad(prompt, (0, 16 - prompt.numel())), prompt.numel())
  state = eng.insert(prefix, eng.init_decode_state(2), 1)
  toks = [int(first.data[0, 0])]
  for _ in range(6):
    state, res = eng.generate(state)
    toks.append(int(res.data[1, 0]))
  if rank == 0:
    with open(out_path, "w") as fh:
      json.dump({"tokens": toks, "logits": prefix.logits[0, :8].tolist()}, fh)
  if world > 1:
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()
  sys.stdout.flush()
  os._exit(0)                 # the result is on disk; skip interpreter teardown (see multirank_worker.py)


if __name__ == "__main__":
  main()
