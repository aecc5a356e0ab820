"""Routed-expert FFN micro-benchmark: padded-group tcgen05 path vs the per-expert loop, forward + backward.

  python -m maxtext_b200.benchmarks.moe_bench --tokens 16384 --experts 8 --topk 2 --d 4096 --f 14336     (Mixtral-8x7B layer)

Timing: CUDA events on the launching stream, 3 warm-up iterations, an L2 flush (256 MB write) between iterations.
FLOPs counted: 3 GEMMs forward + 6 backward over tokens*topk rows (padding rows are not counted).
"""
from __future__ import annotations

import argparse
import json

import torch


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--tokens", type=int, default=16384)
  ap.add_argument("--experts", type=int, default=8)
  ap.add_argument("--topk", type=int, default=2)
  ap.add_argument("--d", type=int, default=4096)
  ap.add_argument("--f", type=int, default=14336)
  ap.add_argument("--iters", type=int, default=5)
  a = ap.parse_args()
  from maxtext_b200.ops import backend, moe_ops
  from maxtext_b200.ops import functional as F
  backend.ext(required=True)
  dev = "cuda"
  torch.manual_seed(0)

  class P:
    def __init__(self, t):
      self.data, self.main_grad, self.grad_written = t, torch.zeros(t.shape, dtype=torch.float32, device=dev), False

  w0, w1 = (P(torch.randn(a.experts, a.f, a.d, device=dev, dtype=torch.bfloat16) * 0.02) for _ in range(2))
  wo = P(torch.randn(a.experts, a.d, a.f, device=dev, dtype=torch.bfloat16) * 0.02)
  x = torch.randn(a.tokens, a.d, device=dev, dtype=torch.bfloat16, requires_grad=True)
  idx = torch.stack([torch.randperm(a.experts, device=dev)[:a.topk] for _ in range(a.tokens)])
  wts = torch.softmax(torch.randn(a.tokens, a.topk, device=dev), -1)
  g = torch.randn(a.tokens, a.d, device=dev, dtype=torch.bfloat16)
  flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

  def padded():
    for p in (w0, w1, wo):
      p.grad_written = False
    y = moe_ops.moe_ffn_padded(x, wts, idx, w0, w1, wo, a.experts, "silu")
    y.backward(g)

  def loop():
    for p in (w0, w1, wo):
      p.grad_written = False
    rows, order, sizes = moe_ops.permute(x, idx, a.experts)
    gg = moe_ops.grouped_linear(rows, w0, sizes)
    uu = moe_ops.grouped_linear(rows, w1, sizes)
    h = F.gated_act(torch.cat([gg, uu], -1), "silu")
    y = moe_ops.grouped_linear(h, wo, sizes)
    out = moe_ops.unpermute_combine(y, order, wts, a.tokens, a.topk).to(torch.bfloat16)
    out.backward(g)

  def timeit(fn):
    for _ in range(3):
      fn()
    ts = []
    for _ in range(a.iters):
      flush.zero_()
      e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      torch.cuda.synchronize()
      e0.record()
      fn()
      e1.record()
      torch.cuda.synchronize()
      ts.append(e0.elapsed_time(e1))
    return sorted(ts)[len(ts) // 2]

  flops = 9 * 2.0 * a.tokens * a.topk * a.d * a.f
  res = {}
  for name, fn in (("padded_grouped", padded), ("per_expert_loop", loop)):
    ms = timeit(fn)
    res[name] = {"ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 1)}
  print(json.dumps({"shape": vars(a), "fwd_bwd": res, "status": backend.ext().kernel_status(True)}))


if __name__ == "__main__":
  main()
