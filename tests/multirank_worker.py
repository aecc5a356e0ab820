"""Worker for multi-rank CPU tests: runs a few train steps under gloo and writes its losses as JSON."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
  out_path, overrides = sys.argv[1], sys.argv[2:]
  from maxtext_b200.config import pyconfig
  from maxtext_b200.parallel import mesh as mesh_lib
  from maxtext_b200.train import train as T
  from maxtext_b200.train.engine import TrainEngine
  rank, world, _ = mesh_lib.init_distributed(timeout_s=120)
  cfg = pyconfig.initialize(["w", "maxtext_b200/configs/base.yml"] + overrides, num_devices=world)
  mesh = mesh_lib.mesh_from_config(cfg, rank=rank, world=world) if world > 1 else None
  from maxtext_b200.train.pipeline import make_engine
  # MAXTEXT_B200_TEST_DEVICE=cuda: the same worker on GPUs (one per rank, NCCL), used by the multi-GPU tier
  on_gpu = os.environ.get("MAXTEXT_B200_TEST_DEVICE") == "cuda"
  if on_gpu:
    # a rank that is still here after three minutes is stuck in a collective whose partner never came: leave, so that the
    # test ends with an error instead of holding the GPUs
    import threading
    t = threading.Timer(180.0, os._exit, (3,))
    t.daemon = True
    t.start()
  dev = torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu")
  eng = make_engine(cfg, mesh, dev)
  it = T.create_data_iterator(cfg, mesh)
  losses, norms = [], []
  stepper = eng
  if cfg.enable_diloco:
    from maxtext_b200.trainers.diloco import DiLoCoTrainer
    stepper = DiLoCoTrainer(eng, cfg, mesh)
  for _ in range(int(cfg.steps)):
    m = stepper.train_step(next(it))
    losses.append(float(m["learning/loss"]))
    norms.append(float(m["learning/raw_grad_norm"]))
  status = 0
  if on_gpu:
    from maxtext_b200.ops import backend
    torch.cuda.synchronize()
    status = int(backend.ext(required=True).kernel_status(True))
  if rank == 0:
    with open(out_path, "w") as fh:
      json.dump({"loss": losses, "grad_norm": norms, "kernel_status": status}, fh)
  if on_gpu:
    sys.stdout.flush()
    os._exit(0)                 # results are on disk; skip the communicator teardown
  if world > 1:
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()
  # results are on disk and the group is closed: leave without running interpreter teardown, where helper threads of a loaded
  # machine have been seen to end the process with std::terminate (exit code -6) after a correct run
  sys.stdout.flush()
  os._exit(0)


if __name__ == "__main__":
  main()
