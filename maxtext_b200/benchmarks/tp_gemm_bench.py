"""Row-parallel linear + all-reduce over a tensor-parallel group: GEMM with the reduce-scatter in its epilogue (peer-memory
reduce-add) + gather kernel, against tcgen05 GEMM followed by an NCCL all-reduce.

  python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m maxtext_b200.benchmarks.tp_gemm_bench \
      [--tokens 16384] [--cols 8192] [--depth 28672]      (depth is the un-sharded contraction size; every rank holds depth / world)

Device-side timing (CUDA events), 3 warm-up iterations, max over ranks; operands far larger than L2.
Roofline: max(FLOPs / measured GEMM peak, bytes over NVLink / 770 GB/s) with bytes = (world-1)/world * tokens * n * (4 + 2)
for the fused path (fp32 partials out, bf16 results back).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--tokens", type=int, default=16384)
  ap.add_argument("--cols", type=int, default=8192)
  ap.add_argument("--depth", type=int, default=28672)
  ap.add_argument("--iters", type=int, default=10)
  ap.add_argument("--mode", default="staged", choices=["staged", "atomic"])
  a = ap.parse_args()
  from maxtext_b200.ops import backend
  from maxtext_b200.ops import functional as F
  from maxtext_b200.parallel import mesh as mesh_lib, tp_fused
  rank, world, _ = mesh_lib.init_distributed()
  dev = torch.device("cuda", torch.cuda.current_device())
  E = backend.ext(required=True)
  kl = a.depth // world
  torch.manual_seed(rank)
  x = [(torch.randn(a.tokens, kl, device=dev) * 0.1).bfloat16() for _ in range(2)]
  w = [(torch.randn(a.cols, kl, device=dev) * 0.1).bfloat16() for _ in range(2)]
  rt = tp_fused.TPReduceRuntime(dist.group.WORLD, dev, a.tokens, a.cols, a.mode)

  def fused(i):
    return rt.all_reduce_gemm(x[i & 1], w[i & 1], True)

  def nccl(i):
    y = F.mm(x[i & 1], w[i & 1], False, True)
    dist.all_reduce(y)
    return y

  ref = nccl(0).float()
  got = fused(0).float()
  err = float((got - ref).abs().max() / ref.abs().max())

  def timeit(fn):
    for i in range(3):
      fn(i)
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.iters):
      fn(i)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)

  t_f, t_n = timeit(fused), timeit(nccl)
  flops = 2.0 * a.tokens * a.cols * kl
  link_bytes = (world - 1) / world * a.tokens * a.cols * (4 if a.mode == "staged" else 6)
  peaks = {}
  try:
    peaks = json.load(open(os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")))
  except Exception:  # pylint: disable=broad-except
    pass
  pk = float(peaks.get("bf16_tflops", 1590.0))
  roof_ms = max(flops / (pk * 1e9), link_bytes / 770e9 * 1e3)
  if rank == 0:
    print(json.dumps({"world": world, "mode": a.mode, "tokens": a.tokens, "n": a.cols, "k_local": kl, "fused_ms": round(t_f, 4), "gemm_plus_nccl_ms": round(t_n, 4),
                      "speedup": round(t_n / t_f, 3), "fused_tflops_per_gpu": round(flops / t_f / 1e9, 1), "roofline_ms": round(roof_ms, 4),
                      "fraction_of_roofline": round(roof_ms / t_f, 3), "max_rel_err_vs_nccl": err, "status": E.kernel_status(True)}))
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
