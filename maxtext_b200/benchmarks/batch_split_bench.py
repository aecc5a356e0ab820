"""Train-step time with and without the batch-split schedule on an expert-parallel MoE model.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29655 \\
      -m maxtext_b200.benchmarks.batch_split_bench [--emb 2048 --layers 4 --experts 8 --seq 2048 --batch 4 --steps 6]

A Mixtral-shaped model (random weights, synthetic data) with its experts spread over all ranks is stepped `--steps` times under
each setting after 3 warm-up steps; the step time is CUDA-event time on the launching stream, max over ranks. Every step
streams weights and activations far larger than L2 (the model holds several GB), so no explicit flush is used. Both settings use
the NCCL expert exchange so that the schedule is the only difference.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _run(cfg_args, world, rank, dev, steps):
  from maxtext_b200.config import pyconfig
  from maxtext_b200.parallel import mesh as mesh_lib
  from maxtext_b200.train import train as T
  from maxtext_b200.train.engine import TrainEngine
  cfg = pyconfig.initialize(["b", "maxtext_b200/configs/base.yml"] + cfg_args, num_devices=world)
  mesh = mesh_lib.mesh_from_config(cfg, rank=rank, world=world)
  eng = TrainEngine(cfg, mesh, dev)
  it = T.create_data_iterator(cfg, mesh)
  for _ in range(3):
    eng.train_step(next(it))
  dist.barrier()
  torch.cuda.synchronize()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(steps):
    m = eng.train_step(next(it))
  e1.record()
  torch.cuda.synchronize()
  ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
  dist.all_reduce(ms, op=dist.ReduceOp.MAX)
  loss = float(m["learning/loss"])
  del eng
  torch.cuda.empty_cache()
  return float(ms), loss


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--emb", type=int, default=2048)
  ap.add_argument("--layers", type=int, default=4)
  ap.add_argument("--experts", type=int, default=8)
  ap.add_argument("--seq", type=int, default=2048)
  ap.add_argument("--batch", type=int, default=4)
  ap.add_argument("--steps", type=int, default=6)
  a = ap.parse_args()
  from maxtext_b200.parallel import mesh as mesh_lib
  rank, world, _ = mesh_lib.init_distributed(timeout_s=120)
  dev = torch.device("cuda", torch.cuda.current_device())
  base = ["model_name=mixtral-8x7b", "override_model_config=true", f"base_emb_dim={a.emb}", f"base_num_query_heads={a.emb // 128}",
          f"base_num_kv_heads={max(1, a.emb // 512)}", "head_dim=128", f"base_mlp_dim={a.emb * 7 // 2}", f"base_moe_mlp_dim={a.emb * 7 // 2}",
          f"num_experts={a.experts}", "num_experts_per_tok=2", f"base_num_decoder_layers={a.layers}", "vocab_size=32000",
          f"max_target_length={a.seq}", f"per_device_batch_size={a.batch}", "dataset_type=synthetic", "enable_checkpointing=false", "hardware=gpu",
          "weight_init=normal", "log_config=false", "steps=100", "learning_rate=1e-4", "ici_fsdp_parallelism=1", f"ici_expert_parallelism={world}",
          "use_fused_comm_kernels=false", "remat_policy=full", "log_period=1000"]
  plain, l0 = _run(base, world, rank, dev, a.steps)
  split, l1 = _run(base + ["use_batch_split_schedule=true"], world, rank, dev, a.steps)
  if rank == 0:
    tokens = a.batch * a.seq * world
    print(json.dumps({"world": world, "shape": vars(a), "plain_ms_per_step": round(plain, 2), "split_ms_per_step": round(split, 2),
                      "plain_tokens_per_s": round(tokens / plain * 1e3), "split_tokens_per_s": round(tokens / split * 1e3),
                      "speedup": round(plain / split, 3), "final_loss": [round(l0, 4), round(l1, 4)]}))
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
