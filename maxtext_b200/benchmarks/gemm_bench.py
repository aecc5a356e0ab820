"""Times the tcgen05 GEMM against torch.matmul (cuBLAS) on the Llama-3-8B layer shapes.

  python -m maxtext_b200.benchmarks.gemm_bench [--tokens 16384] [--iters 10] [--small]

CUDA events on the launching stream, 3 warm-up launches, operands far larger than L2 in aggregate
(each shape allocates its own tensors and the loop alternates between two operand sets).
"""
from __future__ import annotations

import argparse
import json

import torch


def time_fn(fn, iters):
  for _ in range(3):
    fn(0)
  torch.cuda.synchronize()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for i in range(iters):
    fn(i)
  e1.record()
  torch.cuda.synchronize()
  return e0.elapsed_time(e1) / iters


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--tokens", type=int, default=16384)
  ap.add_argument("--iters", type=int, default=10)
  ap.add_argument("--small", action="store_true", help="one small shape only (profiling)")
  ap.add_argument("--no-cublas", action="store_true")
  ap.add_argument("--group-m", type=int, default=0, help="tuning: row blocks per tile group of the persistent walk (0 = default)")
  ap.add_argument("--raster", type=int, default=-1, help="tuning: -1 heuristic, 0 row groups, 1 column groups")
  ap.add_argument("--pair", action="store_true", help="also time the CTA-pair (cta_group::2) variant")
  ap.add_argument("--fp8", action="store_true", help="also time the 8-bit (E4M3 x E4M3) path on the forward shapes, quantisation excluded")
  args = ap.parse_args()
  from maxtext_b200.ops import backend
  E = backend.ext(required=True)
  E.gemm_set_raster(args.raster)
  if args.group_m > 0:
    E.gemm_set_group_m(args.group_m)
  T = args.tokens
  D, F, QKV = 4096, 14336, 6144
  shapes = [("qkv fwd", T, QKV, D, False, True, torch.bfloat16), ("mlp up fwd", T, 2 * F, D, False, True, torch.bfloat16),
            ("mlp down fwd", T, D, F, False, True, torch.bfloat16), ("mlp up dX", T, D, 2 * F, False, False, torch.bfloat16),
            ("mlp down dX", T, F, D, False, False, torch.bfloat16), ("mlp up dW", 2 * F, D, T, True, False, torch.float32),
            ("mlp down dW", D, F, T, True, False, torch.float32)]
  if args.small:
    shapes = [("small", 8192, 8192, 4096, False, True, torch.bfloat16)]   # 256 MB of operands: larger than L2, small enough to profile
  rows = []
  for name, M, N, K, ta, tb, odt in shapes:
    sets = []
    for _ in range(2):
      a = torch.randn((K, M) if ta else (M, K), device="cuda").bfloat16()
      b = torch.randn((N, K) if tb else (K, N), device="cuda").bfloat16()
      sets.append((a, b))
    out = torch.empty(M, N, device="cuda", dtype=odt)
    E.gemm_use_pair(False)            # this row is the single-CTA kernel; --pair adds the CTA-pair kernel the framework uses by default
    ms = time_fn(lambda i: E.gemm(sets[i & 1][0], sets[i & 1][1], out, ta, tb, False), args.iters)
    E.gemm_use_pair(True)
    row = {"shape": name, "M": M, "N": N, "K": K, "ta": ta, "tb": tb, "out": str(odt).split(".")[-1], "ms": ms,
           "tflops": 2.0 * M * N * K / ms / 1e9}
    if not args.no_cublas:
      def cb(i):
        a, b = sets[i & 1]
        r = torch.mm(a.t() if ta else a, b.t() if tb else b)
        if odt == torch.float32:
          out.copy_(r)
      ms2 = time_fn(cb, args.iters)
      row.update(cublas_ms=ms2, cublas_tflops=2.0 * M * N * K / ms2 / 1e9, ratio=ms2 / ms)
    if args.pair and N % 128 == 0:
      msp = time_fn(lambda i: E.gemm_pair(sets[i & 1][0], sets[i & 1][1], out, ta, tb, False), args.iters)
      row.update(pair_ms=msp, pair_tflops=2.0 * M * N * K / msp / 1e9)
    if args.fp8 and not ta and tb and odt == torch.bfloat16:
      q = [(E.quantize_fp8(a, 0, True, False), E.quantize_fp8(b, 0, True, False)) for a, b in sets]
      ms8 = time_fn(lambda i: E.gemm_fp8(q[i & 1][0][0], q[i & 1][1][0], out, 0, 0, q[i & 1][0][2], q[i & 1][1][2], False), args.iters)
      row.update(fp8_ms=ms8, fp8_tflops=2.0 * M * N * K / ms8 / 1e9)
      ref = torch.mm(sets[1][0].float()[:256], sets[1][1].float().t())
      E.gemm_fp8(q[1][0][0], q[1][1][0], out, 0, 0, q[1][0][2], q[1][1][2], False)
      row.update(fp8_rel_err=float((out[:256].float() - ref).abs().max() / ref.abs().max()))
      # block-scaled form (1 x 128 activation, 128 x 128 weight scales): the product alone, then with both quantisations
      qb = [(E.quant_fp8_rows(a), E.quant_fp8_blocks(b, True, False)) for a, b in sets]
      msb = time_fn(lambda i: E.gemm_fp8_block(qb[i & 1][0][0], qb[i & 1][0][1], qb[i & 1][1][0], qb[i & 1][1][2], False, out, None, None),
                    args.iters)
      msq = time_fn(lambda i: (E.quant_fp8_rows(sets[i & 1][0]), E.quant_fp8_blocks(sets[i & 1][1], True, False)), args.iters)
      E.gemm_fp8_block(qb[1][0][0], qb[1][0][1], qb[1][1][0], qb[1][1][2], False, out, None, None)
      row.update(fp8_block_ms=msb, fp8_block_tflops=2.0 * M * N * K / msb / 1e9, fp8_block_quant_ms=msq,
                 fp8_block_rel_err=float((out[:256].float() - ref).abs().max() / ref.abs().max()))
    rows.append(row)
    print(json.dumps(row), flush=True)
    del sets, out
  st = E.kernel_status(True)
  print(json.dumps({"kernel_status": st}))


if __name__ == "__main__":
  main()
