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
_HISTORY_LEN = 0          # 0: current scaling; n > 0: delayed scaling over the last n amax values (the reference uses 1024)
_HISTORY: dict = {}       # (owner id, role) -> [ring tensor [n], write position]


def set_mode(mode: str):
  """'' (bf16), 'fp8' (all three products in 8 bit), 'int8' (forward and input-gradient products on int8 operands).
  Set once by the engine from config.quantization."""
  global _MODE
  _MODE = "fp8" if mode in ("fp8", "fp8_full", "fp8_gpu", "nanoo_fp8", "fp8_nanoo") else "int8" if mode in ("int8", "intmp") else ""


def mode() -> str:
  return _MODE


def set_delayed_scaling(history_len: int):
  """Delayed scaling (src/maxtext/layers/quantizations.py:333-391 `Fp8Einsum`: amax history, scale from its maximum): the
  scale used for a tensor comes from the amax values seen in earlier steps, so quantisation does not wait for a reduction
  over the tensor it is about to cast. History lives on the device; 0 returns to current scaling."""
  global _HISTORY_LEN
  _HISTORY_LEN = int(history_len)
  _HISTORY.clear()


def _quantize(x2, fmt, want_q, want_t, key=None):
  E = backend.ext()
  if _HISTORY_LEN <= 0 or key is None:
    return E.quantize_fp8(x2, fmt, want_q, want_t)
  ent = _HISTORY.get(key)
  if ent is None:
    q, qt, deq, amax = E.quantize_fp8_with(x2, fmt, want_q, want_t, None)       # first sight of this tensor: its own amax
    ring = amax.repeat(_HISTORY_LEN)
    _HISTORY[key] = [ring, 0]
    return q, qt, deq
  ring, pos = ent
  q, qt, deq, amax = E.quantize_fp8_with(x2, fmt, want_q, want_t, ring.max().reshape(1))
  ring[pos % _HISTORY_LEN] = amax[0]
  ent[1] = pos + 1
  return q, qt, deq


def supported(x2: torch.Tensor, w: torch.Tensor) -> bool:
  return (_MODE == "fp8" and backend.use_cuda_kernels(x2) and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
          and x2.shape[0] % 128 == 0 and x2.shape[1] % 128 == 0 and w.shape[0] % 128 == 0 and w.is_contiguous()
          and hasattr(backend.ext(), "gemm_fp8"))


def linear_fwd(x2: torch.Tensor, w: torch.Tensor, owner=None, keep_for_bwd: bool = False):
  """`owner` (the parameter object) keys the amax histories when delayed scaling is on. With keep_for_bwd the same quantise
  pass also writes the transposed copies the backward products need; they are returned as (y, saved) so that the backward
  does not read x and W again."""
  E = backend.ext()
  k = id(owner) if owner is not None else None
  xq, xt, sx = _quantize(x2, E4M3, True, keep_for_bwd, (k, "x") if k else None)
  wq, wt, sw = _quantize(w, E4M3, True, keep_for_bwd, (k, "w") if k else None)
  y = torch.empty(x2.shape[0], w.shape[0], dtype=torch.bfloat16, device=x2.device)
  E.gemm_fp8(xq, wq, y, E4M3, E4M3, sx, sw, False)
  if keep_for_bwd:
    return y, (xt, sx, wt, sw)
  return y


def linear_bwd(dy2: torch.Tensor, x2: torch.Tensor, w: torch.Tensor, need_dx: bool, grad_out: torch.Tensor | None, accumulate: bool,
               owner=None, saved=None):
  """Returns dx (bf16) or None; writes dW into grad_out [out, in] fp32 when given. `saved` = the transposed 8-bit copies of
  x and W that linear_fwd(keep_for_bwd=True) produced."""
  E = backend.ext()
  k = id(owner) if owner is not None else None
  dyq, dyt, sdy = _quantize(dy2, E5M2, need_dx, grad_out is not None, (k, "dy") if k else None)
  dx = None
  if saved is not None:
    xt, sx, wt, sw = saved
    if need_dx:
      dx = torch.empty(dy2.shape[0], w.shape[1], dtype=torch.bfloat16, device=dy2.device)
      E.gemm_fp8(dyq, wt, dx, E5M2, E4M3, sdy, sw, False)
    if grad_out is not None:
      E.gemm_fp8(dyt, xt, grad_out, E5M2, E4M3, sdy, sx, accumulate)
    return dx
  if need_dx:
    _, wt, sw = _quantize(w, E4M3, False, True, (k, "w") if k else None)             # W^T [in, out]: the contraction runs over `out`
    dx = torch.empty(dy2.shape[0], w.shape[1], dtype=torch.bfloat16, device=dy2.device)
    E.gemm_fp8(dyq, wt, dx, E5M2, E4M3, sdy, sw, False)
  if grad_out is not None:
    _, xt, sx = _quantize(x2, E4M3, False, True, (k, "x") if k else None)            # x^T [in, tokens]
    E.gemm_fp8(dyt, xt, grad_out, E5M2, E4M3, sdy, sx, accumulate)
  return dx


# ------------------------------------------------------------------------------------------------------------- int8
# `quantization=int8` (src/maxtext/layers/quantizations.py:144-224 `AqtQuantization`, AQT config_v3 with fwd_bits = 8,
# dlhs_bits = 8, drhs_bits = None): the forward product and the input-gradient product take symmetric int8 operands with one
# scale per contraction-free channel (per token for activations and gradients, per output or input feature for the
# weight); the weight-gradient product stays in the compute dtype. Rounding is to nearest; gradients pass straight through
# the rounding. The integer product itself is a library call on the GPU (`torch._int_mm`) and an exact float emulation
# elsewhere; there is no tcgen05 kind::i8 kernel in this repository yet.
def int8_on() -> bool:
  return _MODE == "int8"


def _q8(t: torch.Tensor, dim: int):
  """Symmetric int8 along `dim` (the contraction dim): returns (int8 values, fp32 scale with `dim` kept as size 1)."""
  amax = t.abs().amax(dim=dim, keepdim=True).float().clamp_(min=1e-12)
  scale = amax / 127.0
  return torch.clamp(torch.round(t.float() / scale), -127, 127).to(torch.int8), scale


def _imm(a8: torch.Tensor, b8t: torch.Tensor) -> torch.Tensor:
  """a8 [M, K] x b8t [N, K]^T -> fp32 [M, N] holding the exact integer products."""
  M, K = a8.shape
  N = b8t.shape[0]
  if a8.is_cuda and M > 16 and K % 8 == 0 and N % 8 == 0:
    return torch._int_mm(a8, b8t.t()).float()   # pylint: disable=protected-access
  return a8.float() @ b8t.float().t()          # |sum| <= K * 127^2: exact in fp32 up to K = 1040, rounded beyond


def int8_linear_fwd(x2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
  xq, sx = _q8(x2, 1)          # per token
  wq, sw = _q8(w, 1)           # per output feature
  return (_imm(xq, wq) * sx * sw.t()).to(x2.dtype)


def int8_linear_dx(dy2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
  gq, sg = _q8(dy2, 1)         # per token
  wq, sw = _q8(w, 0)           # per input feature (the contraction now runs over the output features)
  return (_imm(gq, wq.t().contiguous()) * sg * sw).to(dy2.dtype)


# ------------------------------------------------------------------------------------------------------- block-scaled fp8
# `quantization=fp8` with `fp8_block_scaling=true`: E4M3 operands with one fp32 scale per 1 x 128 block of the contraction
# dimension for activations / gradients and one per 128 x 128 block for weights (the recipe of DeepSeek-V3 style training;
# the reference reaches block-scaled formats through src/maxtext/layers/quantizations.py:1022-1043 and quantises around the
# expert collectives in src/maxtext/models/deepseek_batchsplit_fp8.py:42-98). The forward and the input-gradient products
# run on `csrc/gemm_fp8_block_sm100.cu`; the weight-gradient product stays in bf16 with fp32 accumulation into the store.
_BLOCK = False


def set_block_scaling(on: bool):
  global _BLOCK
  _BLOCK = bool(on)


def block_on() -> bool:
  return _MODE == "fp8" and _BLOCK


def block_supported(x2: torch.Tensor, w: torch.Tensor) -> bool:
  return (block_on() and backend.use_cuda_kernels(x2) and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 2
          and x2.shape[1] % 16 == 0 and w.shape[0] % 16 == 0 and w.is_contiguous() and hasattr(backend.ext(), "gemm_fp8_block"))


def block_linear_fwd(x2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
  """y = x W^T: x quantised 1 x 128 along `in`, W [out, in] in 128 x 128 blocks."""
  E = backend.ext()
  xq, sx = E.quant_fp8_rows(x2)
  wq, _, sw = E.quant_fp8_blocks(w, True, False)
  y = torch.empty(x2.shape[0], w.shape[0], dtype=torch.bfloat16, device=x2.device)
  E.gemm_fp8_block(xq, sx, wq, sw, False, y, None, None)
  return y


def block_linear_dx(dy2: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
  """dx = dy W: dy quantised 1 x 128 along `out`; the operand is the transposed 8-bit copy of W with the same block scales."""
  E = backend.ext()
  gq, sg = E.quant_fp8_rows(dy2)
  _, wt, sw = E.quant_fp8_blocks(w, False, True)            # wt [1, in, out]; sw [1, out/128, in/128] is read transposed
  dx = torch.empty(dy2.shape[0], w.shape[1], dtype=torch.bfloat16, device=dy2.device)
  E.gemm_fp8_block(gq, sg, wt, sw, True, dx, None, None)
  return dx


def block_grouped_fwd(rows: torch.Tensor, w: torch.Tensor, offs, blk_expert, out: torch.Tensor):
  """out = rows W_e^T over padded expert groups (W [E, out, in])."""
  E = backend.ext()
  rq, sr = E.quant_fp8_rows(rows)
  wq, _, sw = E.quant_fp8_blocks(w, True, False)
  E.gemm_fp8_block(rq, sr, wq, sw, False, out, offs, blk_expert)
  return out


def block_grouped_dx(dy: torch.Tensor, w: torch.Tensor, offs, blk_expert, out: torch.Tensor):
  """out = dy W_e over padded expert groups."""
  E = backend.ext()
  gq, sg = E.quant_fp8_rows(dy)
  _, wt, sw = E.quant_fp8_blocks(w, False, True)
  E.gemm_fp8_block(gq, sg, wt, sw, True, out, offs, blk_expert)
  return out
