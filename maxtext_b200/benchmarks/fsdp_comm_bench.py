"""The two FSDP collectives of a training step in isolation, on one unit the size of a Llama-3-8B layer (218 M parameters):

  all-gather of the bf16 parameter shards   (copy engines `dma`, peer-load kernel `prefetch`, NCCL)
  reduce-scatter of the fp32 gradients      (peer loads, in-switch `multimem.ld_reduce`, NCCL)

  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m maxtext_b200.benchmarks.fsdp_comm_bench

Device-side timing (CUDA events on the launching stream, 3 warm-up iterations, a device barrier before each timed group),
max over ranks. Bytes that cross NVLink into a GPU: (world-1)/world * unit bytes for the gather and for the peer-load
reduce-scatter, unit bytes / world for the in-switch one; the bound is the measured 770 GB/s per direction.
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--params", type=int, default=218_112_000)
  ap.add_argument("--iters", type=int, default=10)
  a = ap.parse_args()
  from maxtext_b200.ops import backend
  from maxtext_b200.parallel import mesh as mesh_lib, symm as symm_lib
  rank, world, _ = mesh_lib.init_distributed()
  dev = torch.device("cuda", torch.cuda.current_device())
  E = backend.ext(required=True)
  chunk = -(-a.params // (world * 1024)) * 1024          # elements per rank, 4 KB aligned in both dtypes
  n = chunk * world
  sg = symm_lib.SymmGroup(None, dev)
  shard = sg.alloc(chunk, torch.bfloat16)                 # this rank's parameter shard, readable by the peers
  shard.tensor.normal_()
  grads = sg.alloc(n, torch.float32)                      # this rank's full gradient, readable by the peers
  grads.tensor.normal_()
  full = torch.empty(n, dtype=torch.bfloat16, device=dev)
  dst = torch.empty(chunk, dtype=torch.float32, device=dev)
  sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
  nccl_out = torch.empty(chunk, dtype=torch.float32, device=dev)
  torch.cuda.synchronize()
  sg.barrier(0)

  ops = {
      "ag_dma": lambda: E.gather_dma([int(p) for p in shard.ptrs], full, chunk * 2, (rank + 1) % world),
      "ag_prefetch_kernel": lambda: E.gather_segments(shard.table, full, chunk * 2, 512 * 1024 * 2, world, 32),
      "ag_nccl": lambda: dist.all_gather_into_tensor(full, shard.tensor),
      "rs_peer_loads": lambda: E.rs_sumsq(grads.table, rank * chunk, chunk, dst, False, 1.0, world, sumsq, 48),
      "rs_nccl": lambda: dist.reduce_scatter_tensor(nccl_out, grads.tensor),
  }
  if grads.mc_ptr:
    ops["rs_nvls"] = lambda: E.rs_sumsq_mc(grads.mc_ptr, rank * chunk, chunk, dst, False, 1.0, sumsq, 32)

  # the fused reductions agree with NCCL
  ops["rs_nccl"]()
  ops["rs_peer_loads"]()
  torch.cuda.synchronize()
  err = float((dst - nccl_out).abs().max() / nccl_out.abs().max())

  def timeit(fn):
    for _ in range(3):
      fn()
    torch.cuda.synchronize()
    sg.barrier(1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.iters):
      fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sg.barrier(1)
    return float(t)

  res = {k: timeit(fn) for k, fn in ops.items()}
  sg.check()
  if rank == 0:
    ag_bytes = (world - 1) / world * n * 2
    rs_bytes = {"rs_peer_loads": (world - 1) / world * n * 4, "rs_nccl": (world - 1) / world * n * 4, "rs_nvls": n * 4 / world}
    out = {"world": world, "unit_params": n, "rs_vs_nccl_rel_err": err, "kernel_status": int(E.kernel_status(False))}
    for k, ms in res.items():
      b = ag_bytes if k.startswith("ag") else rs_bytes[k]
      out[k] = {"ms": round(ms, 4), "inbound_GB": round(b / 1e9, 4), "GBps": round(b / ms / 1e6, 1), "of_770": round(b / ms / 1e6 / 770, 3)}
    print(json.dumps(out))
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
