"""Pre-training entry point: `python -m maxtext.train <config.yml> key=value ...`.

The counterpart of src/maxtext/trainers/pre_train/train.py (`main` 1143, `train_loop` 912-1069):
configuration -> distributed runtime + mesh -> model / optimizer / data -> step loop with metrics,
profiler window, periodic checkpoints and evaluation. The step itself is
`train.engine.TrainEngine.train_step`.
"""
from __future__ import annotations

import os
import sys
import time

import torch

from ..config import pyconfig
from ..parallel import mesh as mesh_lib
from ..utils import max_logging
from ..utils.metric_logger import MetricLogger
from . import engine as engine_lib


BATCH_AXES = ("diloco", "data", "fsdp", "fsdp_transpose", "expert")


def data_shard(mesh) -> tuple[int, int]:
  """(index, count) of this rank's slice of the global batch: ranks that differ only along
  sequence/tensor/stage axes read the same rows."""
  if mesh is None:
    return 0, 1
  axes = tuple(a for a in mesh.axis_names if a in BATCH_AXES)
  return mesh.axis_index(axes), mesh.axis_size(axes)


def create_data_iterator(config, mesh):
  from ..input_pipeline import interface
  return interface.create_data_iterator(config, *data_shard(mesh))


class StopTraining(Exception):
  """Raised to end the loop early and cleanly (e.g. target eval loss reached)."""


def setup(config, device=None):
  rank, world, local_rank = mesh_lib.init_distributed(int(config.jax_distributed_initialization_timeout))
  if world != config.num_target_devices:
    config = config.replace(_num_devices=world)
  mesh = mesh_lib.mesh_from_config(config, rank=rank, world=world) if world > 1 else None
  if device is None:
    use_cuda = torch.cuda.is_available() and config.hardware != "cpu"
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
  from . import pipeline as pipeline_lib
  eng = pipeline_lib.make_engine(config, mesh, device)
  return config, mesh, eng


def _default_store():
  import torch.distributed as dist
  if dist.is_available() and dist.is_initialized():
    try:
      return dist.distributed_c10d._get_default_store()  # pylint: disable=protected-access
    except Exception:  # pylint: disable=broad-except
      return None
  return None


def train_loop(config, engine=None, mesh=None, data_iterator=None, recorder=None, attempt: int = 0, preemption=None):
  from ..checkpoint import manager as ckpt_lib
  from ..utils import profiler as prof_lib, goodput, elastic
  if engine is None:
    config, mesh, engine = setup(config)
  c = config
  rank = mesh.rank if mesh is not None else 0
  recorder = recorder or goodput.create_recorder(c, rank)
  data_iterator = data_iterator or create_data_iterator(c, mesh)
  logger = MetricLogger(c, is_writer=(rank == 0))
  prof = prof_lib.Profiler(c, rank)
  ckpt = ckpt_lib.create_checkpoint_manager(c, engine, mesh) if c.enable_checkpointing and c.checkpoint_dir else None
  start_step = 0
  own_watcher = preemption is None
  preemption = preemption or elastic.PreemptionWatcher(_default_store())
  injector = elastic.FaultInjector(rank=rank, guard=elastic.peer_memory_guard(engine))
  heartbeat = None
  if c.elastic_enabled and _default_store() is not None:
    heartbeat = elastic.Heartbeat(_default_store(), rank, mesh.world if mesh is not None else 1,
                                  c.heartbeat_reporting_interval_in_seconds).start()
  if ckpt is not None:
    if attempt > 0:
      ckpt.cleanup_incomplete()
    restored = ckpt.restore_if_possible(data_iterator)
    if restored is not None:
      start_step = restored
  elif c.load_parameters_path:
    ckpt_lib.load_params_only(c.load_parameters_path, engine)
  lora_cfg = getattr(c, "lora", None) or {}
  lora_on = isinstance(lora_cfg, dict) and bool(lora_cfg.get("enable_lora"))
  if lora_on and start_step == 0:
    # adapters from an earlier run (PEFT directory); ignored when this run resumes from its own checkpoint
    adapter_dir = lora_cfg.get("lora_restore_path") or c.hf_lora_adapter_path
    if adapter_dir:
      from ..utils import lora_utils
      lora_utils.load_adapter(adapter_dir, engine.store, c)
  if lora_on and start_step == 0:
    from ..utils import nf4
    n_q = nf4.snap_store(engine.store, c)             # QLoRA: the frozen base weights take their 4-bit NormalFloat values
    if n_q and rank == 0:
      max_logging.log(f"QLoRA: {n_q} base weights rounded to nf4 (tile {lora_cfg.get('lora_tile_size') or nf4.DEFAULT_TILE})")
  engine.step_count = start_step
  is_cuda = engine.device.type == "cuda"
  stepper = engine
  if c.enable_diloco:
    from ..trainers.diloco import DiLoCoTrainer
    stepper = DiLoCoTrainer(engine, c, mesh)
  if bool(getattr(c, "use_dpo", False)):
    # preference optimisation through the same loop: batches of prompt / chosen / rejected, frozen copy of the start weights
    from ..trainers.post_train.trainers import DPODataIterator, DPOStepper
    stepper = DPOStepper(engine)
    if not (isinstance(data_iterator, DPODataIterator)):
      data_iterator = DPODataIterator(c, *data_shard(mesh))
  clean = False     # a failed attempt must not try a collective save on its way out
  try:
    for step in range(start_step, int(c.steps)):
      injector.maybe_fire(step, attempt, heartbeat)
      if heartbeat is not None:
        heartbeat.raise_if_peer_dead(c.elastic_timeout_seconds)
      prof.maybe_start(step)
      t0 = time.perf_counter()
      with recorder.span("DATA_LOADING", step):
        if int(getattr(c, "reuse_example_batch", 0) or 0) > 0 and step > start_step:
          pass                                   # performance testing: the first batch is fed again at every step
        else:
          batch = next(data_iterator)
      with recorder.span("STEP", step):
        metrics = stepper.train_step(batch)
        if is_cuda and (c.profile_cleanly or True):
          torch.cuda.synchronize()
          # a bounded device wait that ran out left incomplete tiles or gradients behind: stop before this step is logged
          # or checkpointed; the elastic supervisor treats the error as retryable
          check_kernel_status(engine.device, rank)
      dt = time.perf_counter() - t0
      logger.record(step, metrics, dt)
      if ckpt is not None:
        ckpt.maybe_save(step, data_iterator)
      if preemption.reached_preemption(step):
        if ckpt is not None and ckpt.latest_step() != step:
          ckpt.save(step, data_iterator, force=True)
        raise StopTraining(f"preemption notice at step {step}")
      if c.eval_interval > 0 and step >= c.eval_start_step and (step + 1) % c.eval_interval == 0:
        ev = run_eval(c, engine, mesh)
        if rank == 0:
          max_logging.log(f"eval step {step}: loss {ev:.4f}")
        if c.target_eval_loss > 0 and ev <= c.target_eval_loss:
          raise StopTraining(f"target eval loss {c.target_eval_loss} reached")
      prof.maybe_stop(step)
    clean = True
  except StopTraining as e:
    clean = True
    max_logging.log(f"training stopped: {e}")
  finally:
    if ckpt is not None:
      if clean and c.save_checkpoint_on_completion:
        ckpt.save(engine.step_count - 1, data_iterator, force=True)
      ckpt.wait_until_finished()
    if lora_on and clean:
      from ..utils import lora_utils
      state, acfg = lora_utils.to_peft(engine.store, c)            # collective: every rank takes part in the gathers
      if rank == 0 and c.base_output_directory:
        import json
        from safetensors.torch import save_file
        out_dir = os.path.join(c.base_output_directory, c.run_name, "lora_adapter")
        os.makedirs(out_dir, exist_ok=True)
        save_file(state, os.path.join(out_dir, "adapter_model.safetensors"))
        with open(os.path.join(out_dir, "adapter_config.json"), "w") as fh:
          json.dump(acfg, fh, indent=1)
    logger.close()
    prof.close()
    recorder.close()
    if heartbeat is not None:
      heartbeat.stop()
    if own_watcher:
      preemption.close()
  return engine, logger.history


def check_kernel_status(device, rank: int = 0, ext=None):
  """Raises CommTimeoutError when any kernel of this process recorded a timed-out wait since the last check (the status
  word is read and cleared). Called after the per-step synchronize, before logging and saving."""
  from ..ops import backend
  from ..parallel.symm import CommTimeoutError
  E = ext if ext is not None else backend.ext()
  if E is None:
    return
  st = int(E.kernel_status(True))
  if st != 0:
    what = {1: "TMA producer", 2: "MMA issuer", 3: "epilogue / softmax", 4: "peer flag"}.get(st, "unknown")
    raise CommTimeoutError(f"rank {rank} on {device}: a bounded device wait ran out (status {st}: {what}); the step's results are incomplete")


def run_eval(config, engine, mesh) -> float:
  from ..input_pipeline import interface
  has_eval_files = bool(getattr(config, "hf_eval_files", "") or getattr(config, "grain_eval_files", ""))
  # the held-out split when one is configured (hf_eval_files / grain_eval_files), else fresh batches of the training stream
  it = interface.create_data_iterator(config, *data_shard(mesh), split="eval") if has_eval_files and config.dataset_type != "synthetic" \
      else create_data_iterator(config, mesh)
  tot, w = 0.0, 0.0
  n = config.eval_steps if config.eval_steps > 0 else 1
  for _ in range(n):
    m = engine.eval_step(next(it))
    tot += float(m["evaluation/total_loss"].item())
    w += float(m["evaluation/total_weights"].item())
  return tot / max(w, 1e-8)


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  config = pyconfig.initialize(argv)
  if not config.elastic_enabled:
    return train_loop(config)
  # the whole initialise + train function is what gets retried (src/maxtext/trainers/pre_train/train.py:1111-1140)
  from ..utils import elastic
  sup = elastic.ElasticSupervisor.from_config(config, cleanup=elastic.teardown_distributed)
  return sup.run(lambda attempt, world: train_loop(config, attempt=attempt))


def cli(argv=None):
  """Entry point of `python -m ...train`: run, then close the process group and leave without interpreter teardown. With a live
  process group, helper threads of the collective backend have ended otherwise correct multi-rank runs with std::terminate
  (exit code -6) while the interpreter was shutting down; everything the run writes is flushed and closed before this point."""
  main(argv)
  sys.stdout.flush()
  sys.stderr.flush()
  import torch.distributed as dist
  if dist.is_available() and dist.is_initialized():
    try:
      dist.barrier()
      dist.destroy_process_group()
    except Exception as e:  # pylint: disable=broad-except
      max_logging.log(f"destroy_process_group: {e!r}")
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
  cli()
