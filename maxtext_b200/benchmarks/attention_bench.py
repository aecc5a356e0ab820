"""Times the tcgen05 flash attention (forward and backward) at the Llama-3-8B shape and, for context,
the library attention PyTorch dispatches to.

  python -m maxtext_b200.benchmarks.attention_bench [--batch 2] [--seq 8192] [--small]

FLOPs are counted as 4*B*S^2*Hq*D/2 forward (causal half) and 2.5x that backward, the accounting used by
the reference's TFLOPs formula. CUDA events, 3 warm-up launches.
"""
from __future__ import annotations

import argparse
import json

import torch


def timeit(fn, iters):
  for _ in range(3):
    fn()
  torch.cuda.synchronize()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(iters):
    fn()
  e1.record()
  torch.cuda.synchronize()
  return e0.elapsed_time(e1) / iters


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--batch", type=int, default=2)
  ap.add_argument("--seq", type=int, default=8192)
  ap.add_argument("--hq", type=int, default=32)
  ap.add_argument("--hkv", type=int, default=8)
  ap.add_argument("--dim", type=int, default=128)
  ap.add_argument("--dim-v", type=int, default=0, help="head dim of V / O when it differs (multi-head latent attention: --dim 192 --dim-v 128)")
  ap.add_argument("--iters", type=int, default=10)
  ap.add_argument("--small", action="store_true")
  ap.add_argument("--no-lib", action="store_true")
  a = ap.parse_args()
  if a.small:
    a.batch, a.seq, a.hq, a.hkv, a.iters = 2, 4096, 32, 8, 3     # 160 MB of q, k, v, out: larger than L2, small enough to profile
  from maxtext_b200.ops import backend
  E = backend.ext(required=True)
  B, S, Hq, Hkv, D = a.batch, a.seq, a.hq, a.hkv, a.dim
  Dv = a.dim_v or D
  if Dv == D:
    qkv = (0.3 * torch.randn(B, S, Hq + 2 * Hkv, D, device="cuda")).bfloat16()
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    dqkv = torch.empty_like(qkv)
    dq, dk, dv = dqkv[:, :, :Hq], dqkv[:, :, Hq:Hq + Hkv], dqkv[:, :, Hq + Hkv:]
  else:
    q = (0.3 * torch.randn(B, S, Hq, D, device="cuda")).bfloat16()
    k = (0.3 * torch.randn(B, S, Hkv, D, device="cuda")).bfloat16()
    v = (0.3 * torch.randn(B, S, Hkv, Dv, device="cuda")).bfloat16()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    a.no_lib = True
  out = torch.empty(B, S, Hq, Dv, device="cuda", dtype=torch.bfloat16)
  lse = torch.empty(B, Hq, S, device="cuda")
  dout = torch.randn_like(out)
  fwd_flops = 2.0 * B * S * S * Hq * (D + Dv) / 2
  ms_f = timeit(lambda: E.flash_fwd(q, k, v, out, lse, None, None, None, None, None, 1.0, 0.0, True, 0, 0, 0), a.iters)
  ms_b = timeit(lambda: E.flash_bwd(dout, q, k, v, out, lse, dq, dk, dv, None, None, None, None, 1.0, 0.0, True, 0, 0, 0), a.iters)
  row = {"B": B, "S": S, "Hq": Hq, "Hkv": Hkv, "D": D, "Dv": Dv, "fwd_ms": ms_f, "fwd_tflops": fwd_flops / ms_f / 1e9, "bwd_ms": ms_b,
         "bwd_tflops": 2.5 * fwd_flops / ms_b / 1e9, "kernel_status": E.kernel_status(True)}
  if not a.no_lib:
    qh, kh, vh = (t.transpose(1, 2).contiguous().requires_grad_(True) for t in (q, k, v))
    sd = lambda: torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=True, scale=1.0, enable_gqa=True)  # noqa: E731
    with torch.no_grad():
      ms_lf = timeit(sd, a.iters)
    o = sd()
    do = torch.randn_like(o)
    ms_lb = timeit(lambda: torch.autograd.grad(o, (qh, kh, vh), do, retain_graph=True), a.iters)
    row.update(lib_fwd_ms=ms_lf, lib_fwd_tflops=fwd_flops / ms_lf / 1e9, lib_bwd_ms=ms_lb, lib_bwd_tflops=2.5 * fwd_flops / ms_lb / 1e9)
  print(json.dumps(row))


if __name__ == "__main__":
  main()
