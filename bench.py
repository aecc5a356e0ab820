"""Headline benchmark: Llama-3-8B pre-training throughput (tokens/s, whole job) in bf16 with fp32
master weights and AdamW, sequence 8192, per-device batch 2, remat_policy=full, FSDP over N GPUs.

  python bench.py --gpus 1 --steps 5 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      bench.py --gpus N --steps K --warmup W

Rank 0 prints one JSON line. `value` is device-timed (CUDA events, max over ranks) over exactly K
optimizer steps; `e2e` repeats the measurement through the public API including, every step, the
host->device copy of the batch from pinned memory and a device->host read of the loss.
`--impl reference` runs the unmodified reference from baseline/_ref through its own train entry point when its
JAX runtime can be imported, and reports `unavailable` with the reason otherwise. Multi-GPU runs first check, untimed,
that the fused NVLink collectives reproduce the NCCL path (`fused_vs_nccl_max_rel_err`).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PUBLISHED_TOK_S_PER_DEVICE = 7207.0   # Llama 3.1 8B, seq 8192, bf16, per device (docs/reference/models/tiering.md:16)
NOMINAL_BF16_TFLOPS = 2250.0


# Secondary configurations (BASELINE.json configs[2..4]); the headline is llama3_8b.
PRESETS = {
    "llama3_8b": dict(model="llama3-8b", seq=8192, pdbs=2.0, ep=1, tp=1, quantization="", extra=[]),
    "mixtral_ep8": dict(model="mixtral-8x7b", seq=4096, pdbs=1.0, ep=8, tp=1, quantization="", extra=[]),
    "deepseek16b_fp8_ep8": dict(model="deepseek2-16b", seq=4096, pdbs=2.0, ep=8, tp=1, quantization="fp8", extra=["fp8_block_scaling=true"]),
    # fp32 master + second moment, bf16 first moment: 14 bytes per parameter so that 70.6 B parameters fit 8 x 180 GB
    "llama70b_fsdp4_tp2": dict(model="llama3-70b", seq=4096, pdbs=1.0, ep=1, tp=2, quantization="", extra=["mu_dtype=bfloat16"]),
}


# published tokens/s/device of the reference for the model families it reports (other hardware); None where it reports none
PUBLISHED_BY_MODEL = {"mixtral-8x7b": 3899.0, "llama3-70b": 960.0}


def _vs_published(args, value, world):
  if args.layers:
    return None                                     # a reduced-depth debug run is not the published configuration
  if args.config == "llama3_8b":
    return value / (PUBLISHED_TOK_S_PER_DEVICE * world)
  per = PUBLISHED_BY_MODEL.get(args.model)
  return value / (per * world) if per else None


def _reference_overrides(args, world):
  return [f"model_name={args.model}", f"per_device_batch_size={args.pdbs}", f"max_target_length={args.seq}", "dataset_type=synthetic",
          "remat_policy=full", "enable_checkpointing=false", "hardware=gpu_multiprocess" if world > 1 else "hardware=gpu",
          f"steps={args.warmup + args.steps}", "learning_rate=3e-5", f"ici_fsdp_parallelism={world // (args.ep * args.tp)}",
          f"ici_expert_parallelism={args.ep}", f"ici_tensor_parallelism={args.tp}", "dtype=bfloat16", "weight_dtype=float32",
          "attention=cudnn_flash_te", "run_name=bench_reference", "base_output_directory=/tmp/bench_reference", "log_period=1",
          "enable_goodput_recording=false", "monitor_goodput=false", "enable_tensorboard=false"] + \
      ([f"quantization={args.quantization}"] if args.quantization else [])


def reference_arm(args):
  """Runs the unmodified reference (baseline/_ref, installed from the reference tree) through its own entry point
  `python -m maxtext.trainers.pre_train.train` with the headline overrides and reads tokens/s from its per-step log lines.
  Under torchrun every rank starts one reference process (one GPU each, JAX's own multi-process coordination on the
  torchrun rendezvous address); rank 0 prints the JSON line. Without an importable JAX it reports `unavailable`."""
  import re
  ref_dir = os.path.join(ROOT, "baseline", "_ref")
  rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))

  def unavailable(why):
    if rank == 0:
      print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}))
    return 0
  env = dict(os.environ)
  env["PYTHONPATH"] = ref_dir + os.pathsep + os.path.join(ref_dir, "src") + os.pathsep + env.get("PYTHONPATH", "")
  probe = subprocess.run([sys.executable, "-c", "import jax, flax, optax, maxtext; print(jax.__version__)"], env=env, capture_output=True, text=True)
  if probe.returncode != 0:
    last = (probe.stderr.strip().splitlines() or ["import failed"])[-1]
    return unavailable("the reference is a JAX program and its runtime (jax + jaxlib CUDA, flax, optax, orbax, grain) is neither importable "
                       f"nor in the offline wheelhouse: {last}")
  base_yml = None
  for cand in (os.path.join(ref_dir, "maxtext", "configs", "base.yml"), os.path.join(ref_dir, "src", "maxtext", "configs", "base.yml")):
    if os.path.isfile(cand):
      base_yml = cand
  if base_yml is None:
    return unavailable("baseline/_ref holds no maxtext/configs/base.yml: the reference package is not installed there")
  env.update(CUDA_VISIBLE_DEVICES=str(local), JAX_COORDINATOR_IP=os.environ.get("MASTER_ADDR", "127.0.0.1"),
             JAX_COORDINATOR_PORT=str(int(os.environ.get("MASTER_PORT", "29500")) + 7), NNODES=str(world), NODE_RANK=str(rank),
             XLA_PYTHON_CLIENT_MEM_FRACTION="0.92", TF_CPP_MIN_LOG_LEVEL="2")
  cmd = [sys.executable, "-m", "maxtext.trainers.pre_train.train", base_yml] + _reference_overrides(args, world)
  t0 = time.perf_counter()
  run = subprocess.run(cmd, env=env, capture_output=True, text=True)
  wall = time.perf_counter() - t0
  if run.returncode != 0:
    last = (run.stderr.strip().splitlines() or run.stdout.strip().splitlines() or ["failed"])[-1]
    return unavailable(f"the reference's train entry point exited {run.returncode}: {last}")
  # "completed step: 7, seconds: 1.234, TFLOP/s/device: 456.7, Tokens/s/device: 8901.2, ..."
  rows = re.findall(r"completed step: (\d+), seconds: ([0-9.]+), TFLOP/s/device: ([0-9.]+), Tokens/s/device: ([0-9.]+)", run.stdout + run.stderr)
  rows = rows[-args.steps:]
  if len(rows) < args.steps:
    return unavailable(f"the reference ran but logged {len(rows)} timed steps instead of {args.steps}")
  sec = sum(float(r[1]) for r in rows)
  gb = int(args.pdbs * world)
  value = gb * args.seq * args.steps / sec
  if rank == 0:
    print(json.dumps({"impl": "reference", "metric": "tokens/sec (whole job) Llama-3-8B FSDP bf16 seq 8192 pre-training", "value": value,
                      "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sec / args.steps,
                      "higher_is_better": True, "scaling": "weak", "vs_baseline": value / (PUBLISHED_TOK_S_PER_DEVICE * world), "dtype": "bf16",
                      "data": "synthetic", "config": {"model": args.model, "global_batch": gb, "seq_len": args.seq,
                                                      "parallelism": f"fsdp{world // (args.ep * args.tp)}", "timing": "the reference's own per-step wall clock"},
                      "model_tflops_per_sec_per_gpu": statistics.mean(float(r[2]) for r in rows),
                      "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                              "note": "the reference times whole steps of its public train loop, data pipeline included"},
                      "wall_s": wall}))
  return 0


def fused_vs_nccl_precheck(args, world, rank, dev):
  """Untimed: a 2-layer model of the benchmarked family takes two optimizer steps with this repository's fused NVLink
  collectives and again with plain NCCL, from the same initial weights and batch. Returns the largest relative difference
  over loss, gradient norm and a parameter checksum (max over ranks)."""
  import torch
  import torch.distributed as dist
  from maxtext_b200.config import pyconfig
  from maxtext_b200.input_pipeline.synthetic import SyntheticDataIterator
  from maxtext_b200.parallel import mesh as mesh_lib
  from maxtext_b200.train import train as train_lib
  from maxtext_b200.train.engine import TrainEngine
  import gc
  res = {}
  # the comparison arm's unfused paths (per-expert loops over ragged groups) may use library products: only the timed run is strict
  strict = os.environ.pop("MAXTEXT_B200_STRICT_GEMM", None)
  for mode in ("true", "false"):
    over = [f"model_name={args.model}", "per_device_batch_size=1", "max_target_length=1024", "dataset_type=synthetic", "remat_policy=full",
            "enable_checkpointing=false", "hardware=gpu", "weight_init=normal", "log_config=false", "steps=10", "learning_rate=1e-3",
            f"ici_fsdp_parallelism={world // (args.ep * args.tp)}", f"ici_expert_parallelism={args.ep}", f"ici_tensor_parallelism={args.tp}",
            "dtype=bfloat16", "weight_dtype=float32", "attention=flash", f"use_fused_comm_kernels={mode}", "base_num_decoder_layers=2",
            "override_model_config=true", "first_num_dense_layers=1"] + ([f"quantization={args.quantization}"] if args.quantization else [])
    cfg = pyconfig.initialize(["precheck", os.path.join(ROOT, "maxtext_b200", "configs", "base.yml")] + over, num_devices=world)
    mesh = mesh_lib.mesh_from_config(cfg, rank=rank, world=world)
    eng = TrainEngine(cfg, mesh, dev)
    batch = next(SyntheticDataIterator(cfg, *train_lib.data_shard(mesh)))
    vals = []
    for _ in range(2):
      m = eng.train_step(batch)
      vals += [float(m["learning/loss"]), float(m["learning/raw_grad_norm"])]
    vals.append(float(eng.store.master.double().abs().sum()))
    res[mode] = vals
    del eng, m, batch, mesh
    gc.collect()                                  # engine <-> store reference cycles: free the 2-layer model before the real one is built
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    dist.barrier()
  if strict is not None:
    os.environ["MAXTEXT_B200_STRICT_GEMM"] = strict
  rel = max(abs(a - b) / max(abs(b), 1e-12) for a, b in zip(res["true"], res["false"]))
  t = torch.tensor([rel], device=dev, dtype=torch.float64)
  dist.all_reduce(t, op=dist.ReduceOp.MAX)
  return float(t.item())


class ClockSampler:
  """Samples SM clock and throttle reasons of this rank's GPU with nvidia-smi while the timed region runs."""

  Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
       "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

  def __init__(self, gpu_index: int):
    self.gpu = gpu_index
    self.rows = []
    self.proc = None
    self.path = None

  def start(self):
    try:
      fd, self.path = tempfile.mkstemp(suffix=".csv")
      os.close(fd)
      self.fh = open(self.path, "w")
      self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                    "-i", str(self.gpu)], stdout=self.fh, stderr=subprocess.DEVNULL)
    except Exception:  # pylint: disable=broad-except
      self.proc = None

  def stop(self) -> dict:
    out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
    if self.proc is None:
      return out
    self.proc.terminate()
    try:
      self.proc.wait(timeout=5)
    except Exception:  # pylint: disable=broad-except
      self.proc.kill()
    self.fh.close()
    sm, mx, reasons = [], [], set()
    with open(self.path) as fh:
      for line in fh:
        p = [x.strip() for x in line.split(",")]
        if len(p) < 9:
          continue
        try:
          sm.append(float(p[1]))
          mx.append(float(p[2]))
        except ValueError:
          continue
        for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
          if v.lower().startswith("active"):
            reasons.add(name)
    os.unlink(self.path)
    if sm:
      out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
    return out


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=4)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--impl", default="ours")
  ap.add_argument("--config", default="llama3_8b", choices=sorted(PRESETS), help="llama3_8b is the headline; the others are BASELINE.json's "
                  "secondary configurations at their full sizes")
  ap.add_argument("--model", default="")
  ap.add_argument("--seq", type=int, default=0)
  ap.add_argument("--pdbs", type=float, default=0.0)
  ap.add_argument("--layers", type=int, default=0, help="debug only: override layer count (result is then not the headline config)")
  ap.add_argument("--no-e2e", action="store_true")
  ap.add_argument("--trace", default="", help="write a chrome trace of one extra (untimed) step to this path")
  ap.add_argument("--ep", type=int, default=0, help="expert-parallel degree (secondary benchmarks; the headline uses fsdp only)")
  ap.add_argument("--tp", type=int, default=0, help="tensor-parallel degree (secondary benchmarks)")
  ap.add_argument("--cp", type=int, default=1, help="context-parallel degree (secondary benchmarks)")
  ap.add_argument("--cp-strategy", default="ring", choices=["ring", "all_gather", "ulysses", "usp"])
  ap.add_argument("--quantization", default=None, help="'' (headline: bf16) or fp8: linear layers on the 8-bit tensor-core path (a different configuration)")
  ap.add_argument("--no-precheck", action="store_true", help="skip the untimed fused-vs-NCCL equivalence check that multi-GPU runs do first")
  ap.add_argument("--comm", default="fused", choices=["fused", "nccl"],
                  help="FSDP collectives: this repository's NVLink kernels fused with the GEMMs (default) or plain NCCL (comparison arm)")
  args = ap.parse_args()
  preset = PRESETS[args.config]
  args.model = args.model or preset["model"]
  args.seq = args.seq or preset["seq"]
  args.pdbs = args.pdbs or preset["pdbs"]
  args.ep = args.ep or preset["ep"]
  args.tp = args.tp or preset["tp"]
  args.quantization = preset["quantization"] if args.quantization is None else args.quantization
  headline = (args.model == "llama3-8b" and args.layers <= 0 and args.ep == 1 and args.tp == 1 and args.cp == 1 and args.seq == 8192 and
              args.pdbs == 2.0 and not args.quantization)
  if args.impl == "reference":
    return reference_arm(args)
  # every GEMM of the step must run on this repository's tcgen05 kernels: a shape they do not cover raises instead of
  # silently calling the library
  os.environ.setdefault("MAXTEXT_B200_STRICT_GEMM", "1")

  import torch
  import torch.distributed as dist
  from maxtext_b200.config import pyconfig
  from maxtext_b200.input_pipeline.synthetic import SyntheticDataIterator
  from maxtext_b200.ops import backend, functional as F
  from maxtext_b200.parallel import mesh as mesh_lib
  from maxtext_b200.train import train as train_lib
  from maxtext_b200.train.engine import TrainEngine
  from maxtext_b200.utils import flops

  world = int(os.environ.get("WORLD_SIZE", "1"))
  assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N>1 with torch.distributed.run"
  rank, world, local_rank = mesh_lib.init_distributed()
  dev = torch.device("cuda", torch.cuda.current_device())
  precheck = None
  if world > 1 and args.comm == "fused" and not args.no_precheck and args.cp == 1:
    precheck = fused_vs_nccl_precheck(args, world, rank, dev)
    assert precheck < 2e-2, f"fused collectives disagree with NCCL: max relative difference {precheck}"
  overrides = [f"model_name={args.model}", f"per_device_batch_size={args.pdbs}", f"max_target_length={args.seq}",
               "dataset_type=synthetic", "remat_policy=full", "enable_checkpointing=false", "hardware=gpu", "weight_init=normal",
               "log_config=false", "steps=1000", "learning_rate=3e-5", f"ici_fsdp_parallelism={world // (args.ep * args.tp * args.cp)}", f"ici_expert_parallelism={args.ep}",
               f"ici_tensor_parallelism={args.tp}", f"ici_context_parallelism={args.cp}", f"context_parallel_strategy={args.cp_strategy}", "dtype=bfloat16",
               "weight_dtype=float32", "attention=flash", f"use_fused_comm_kernels={'true' if args.comm == 'fused' else 'false'}"]
  overrides += list(preset["extra"]) if args.model == preset["model"] else []
  if args.quantization:
    overrides += [f"quantization={args.quantization}"]
  if args.layers > 0:
    overrides += [f"base_num_decoder_layers={args.layers}", "override_model_config=true"]
  cfg = pyconfig.initialize(["bench", os.path.join(ROOT, "maxtext_b200", "configs", "base.yml")] + overrides, num_devices=world)
  mesh = mesh_lib.mesh_from_config(cfg, rank=rank, world=world) if world > 1 else None
  E = backend.ext(required=True)
  eng = TrainEngine(cfg, mesh, dev)
  it = SyntheticDataIterator(cfg, *train_lib.data_shard(mesh))
  batch = next(it)   # pinned host tensors; every step copies them to the device
  fallbacks_before = int(F.gemm_fallbacks())     # the untimed comparison arm of the pre-check may have used library products

  def barrier():
    if world > 1:
      dist.barrier()
    torch.cuda.synchronize()

  for _ in range(args.warmup):
    m = eng.train_step(batch)
  barrier()
  assert E.kernel_status(True) == 0, "kernel wait timed out during warm-up"

  # ---- device-timed region
  sampler = ClockSampler(torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ else
                         int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[torch.cuda.current_device()]))
  sampler.start()
  launches0 = E.launch_count()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  barrier()
  e0.record()
  for _ in range(args.steps):
    m = eng.train_step(batch)
  e1.record()
  barrier()
  ms = e0.elapsed_time(e1)
  launches = E.launch_count() - launches0
  clocks = sampler.stop()
  loss = float(m["learning/loss"])
  t = torch.tensor([ms], device=dev)
  if world > 1:
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
  ms = float(t.item())

  # ---- end-to-end through the public API: H2D of the batch from pinned memory + D2H of the loss, every step
  e2e = None
  if not args.no_e2e:
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
      mm = eng.train_step(batch)
      _ = float(mm["learning/loss"])       # device -> host read of the step result
    barrier()
    dt = time.perf_counter() - t0
    tt = torch.tensor([dt], device=dev)
    if world > 1:
      dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    dt = float(tt.item())
    h2d = sum(v.numel() * v.element_size() for k, v in batch.items()
              if k in ("inputs", "targets", "inputs_position", "inputs_segmentation", "targets_segmentation"))
    tokens_total = cfg.global_batch_size_to_train_on * cfg.max_target_length * args.steps
    e2e = {"value": tokens_total / dt, "unit": "tokens/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": 4,
           "ms_per_step": 1e3 * dt / args.steps}
  status = E.kernel_status(True)

  if args.trace:
    # one extra, untimed step under the PyTorch profiler: a per-stream kernel timeline (chrome trace) for overlap analysis
    from torch.profiler import ProfilerActivity, profile
    barrier()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
      eng.train_step(batch)
      torch.cuda.synchronize()
    if rank == 0:
      prof.export_chrome_trace(args.trace)

  if rank == 0:
    gb = cfg.global_batch_size_to_train_on
    tokens = gb * cfg.max_target_length * args.steps
    value = tokens / (ms / 1e3)
    tflops_step, _, _ = flops.training_tflops_per_device(cfg)
    tf_s = tflops_step / (ms / 1e3 / args.steps)
    peaks = {}
    try:
      peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:  # pylint: disable=broad-except
      pass
    out = {
        "metric": "tokens/sec (whole job) Llama-3-8B FSDP bf16 seq 8192 pre-training" if headline
        else f"tokens/sec (whole job) {args.model} seq {args.seq} pre-training (secondary benchmark)", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": _vs_published(args, value, world), "dtype": "bf16" if not args.quantization else f"{args.quantization} linears, bf16 elsewhere", "data": "synthetic",
        "config": {"model": args.model + ("" if args.layers <= 0 else f"-{args.layers}layers-DEBUG"), "global_batch": gb,
                   "seq_len": cfg.max_target_length, "parallelism": f"fsdp{world // (args.ep * args.tp * args.cp)}" + (f"xep{args.ep}" if args.ep > 1 else "") + (f"xtp{args.tp}" if args.tp > 1 else "") + (f"xcp{args.cp}-{args.cp_strategy}" if args.cp > 1 else ""), "collectives": args.comm if world > 1 else "none", "remat_policy": cfg.remat_policy,
                   "optimizer": "adamw fp32 master", "l2": "inputs_larger_than_L2 (16 GB of weights streamed per step)"},
        "tokens_per_sec_per_gpu": value / world, "model_tflops_per_sec_per_gpu": tf_s,
        "mfu_of_nominal_2250": tf_s / NOMINAL_BF16_TFLOPS,
        "mfu_of_measured_cublas_sustained": tf_s / peaks["bf16_tflops_sustained"] if peaks.get("bf16_tflops_sustained") else None,
        "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"]},
        "e2e": e2e, "gpu_launches": int(launches), "final_loss": loss, "kernel_status": int(status), "impl": "ours",
        "library_gemm_fallbacks": int(F.gemm_fallbacks()) - fallbacks_before, "fused_vs_nccl_max_rel_err": precheck,
    }
    print(json.dumps(out))
  if world > 1:
    dist.destroy_process_group()
  return 0


if __name__ == "__main__":
  sys.exit(main())
