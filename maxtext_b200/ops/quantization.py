"""FP8 training path for linear layers (config `quantization=fp8`).

The reference wires quantised dot_generals through providers (src/maxtext/layers/quantizations.py: `Fp8Quantization`,
`NANOOFp8Quantization`; per-tensor scaling, E4M3 for activations and weights, E5M2 for gradients). Here every product of a
linear layer runs on the 8-bit tensor-core path (tcgen05 kind::f8f6f4, fp32 accumulation in tensor memory):

  y  = Q(x) Q(W)^T          E4M3 x E4M3
  dx = Q(dy) Q(W^T)^T       E5M2 x E4M3
  dW = Q(dy^T) Q(x^T)^T     E5M2 x E4M3, accumulated in fp32 straight into the gradient store

Scales are per tensor from the tensor's own absolute maximum ("current scaling"), computed and consumed on the device; the
quantise kernel emits the row-major and the transposed copy in one pass because the 8-bit path takes K-major operands only.
"""
from __future__ import annotations

import torch

from . import backend

E4M3, E5M2 = 0, 1
_MODE = ""


def set_mode(mode: str):
  """'' (bf16), 'fp8' (all three products in 8 bit). Set once by the engine from config.quantization."""
  global _MODE
  _MODE = "fp8" if mode in ("fp8", "fp8_full", "fp8_gpu", "nanoo_fp8", "fp8_nanoo") else ""


def mode() -> str:
  return _MODE


def supported(x2: torch.Tensor, w: torch.Tensor) -> bool:
  return (_MODE == "fp8" and backend.use_cuda_kernels(x2) and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
          and x2.shape[0] % 128 == 0 and x2.shape[1] % 128 == 0 and w.shape[0] % 128 == 0 and w.is_contiguous()
          and hasattr(backend.ext(), "gemm_fp8"))


def linear_fwd(x2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
  E = backend.ext()
  xq, _, sx = E.quantize_fp8(x2, E4M3, True, False)
  wq, _, sw = E.quantize_fp8(w, E4M3, True, False)
  y = torch.empty(x2.shape[0], w.shape[0], dtype=torch.bfloat16, device=x2.device)
  E.gemm_fp8(xq, wq, y, E4M3, E4M3, sx, sw, False)
  return y


def linear_bwd(dy2: torch.Tensor, x2: torch.Tensor, w: torch.Tensor, need_dx: bool, grad_out: torch.Tensor | None, accumulate: bool):
  """Returns dx (bf16) or None; writes dW into grad_out [out, in] fp32 when given."""
  E = backend.ext()
  dyq, dyt, sdy = E.quantize_fp8(dy2, E5M2, need_dx, grad_out is not None)
  dx = None
  if need_dx:
    _, wt, sw = E.quantize_fp8(w, E4M3, False, True)             # W^T [in, out]: the contraction runs over `out`
    dx = torch.empty(dy2.shape[0], w.shape[1], dtype=torch.bfloat16, device=dy2.device)
    E.gemm_fp8(dyq, wt, dx, E5M2, E4M3, sdy, sw, False)
  if grad_out is not None:
    _, xt, sx = E.quantize_fp8(x2, E4M3, False, True)            # x^T [in, tokens]
    E.gemm_fp8(dyt, xt, grad_out, E5M2, E4M3, sdy, sx, accumulate)
  return dx
