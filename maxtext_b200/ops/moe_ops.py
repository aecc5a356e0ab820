"""MoE data-movement and grouped-GEMM ops with explicit backward passes.

permute / unpermute_combine reproduce the dropless token permutation of
src/maxtext/layers/moe.py:872-1063 (stable sort by expert id, k copies per token, weighted sum on the
way back); grouped_linear is the grouped matmul that the reference gets from megablox / ragged_dot
(src/maxtext/kernels/megablox/ops.py:46-137): rows grouped by expert times a per-expert matrix, with
the transposed grouped product for the weight gradient written into the fp32 gradient store.
"""
from __future__ import annotations

import torch

from . import backend
from . import functional as F


class _PermuteFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, src_row, T):
    ctx.save_for_backward(src_row)
    ctx.T = T
    return x.index_select(0, src_row)

  @staticmethod
  def backward(ctx, dy):
    (src_row,) = ctx.saved_tensors
    dx = torch.zeros(ctx.T, dy.shape[1], dtype=torch.float32, device=dy.device)
    dx.index_add_(0, src_row, dy.float())
    return dx.to(dy.dtype), None, None


def permute(x2: torch.Tensor, expert_idx: torch.Tensor, num_experts: int):
  """x2 [T, D], expert_idx [T, k] -> (rows [T*k, D] sorted by expert, order [T*k], group sizes [E])."""
  T, k = expert_idx.shape
  flat = expert_idx.reshape(-1)
  order = torch.argsort(flat, stable=True)
  sizes = torch.bincount(flat, minlength=num_experts)
  src_row = torch.div(order, k, rounding_mode="floor")
  rows = _PermuteFn.apply(x2, src_row, T) if torch.is_grad_enabled() else x2.index_select(0, src_row)
  return rows, order, sizes


def unpermute_combine(y: torch.Tensor, order: torch.Tensor, weights: torch.Tensor, T: int, k: int, fp32_sum: bool = True):
  """Inverse permutation + weighted sum over the k experts of each token."""
  inv = torch.empty_like(order)
  inv[order] = torch.arange(order.numel(), device=order.device)
  yk = y.index_select(0, inv).view(T, k, -1)
  w = weights.to(torch.float32 if fp32_sum else y.dtype)
  if fp32_sum:
    return (yk.float() * w.unsqueeze(-1)).sum(1)
  return (yk * w.unsqueeze(-1)).sum(1)


def _grouped_mm(x, w, sizes_host, tb: bool, out=None):
  """x rows grouped by expert; w [E, N, K] if tb (y = x @ w[e].T) else [E, K, N] (y = x @ w[e])."""
  n_out = w.shape[1] if tb else w.shape[2]
  if out is None:
    out = torch.empty(x.shape[0], n_out, dtype=x.dtype, device=x.device)
  s = 0
  for e, n in enumerate(sizes_host):
    if n:
      F.mm(x[s:s + n], w[e], False, tb, out=out[s:s + n])
    s += n
  if s < x.shape[0]:
    out[s:].zero_()
  return out


class _GroupedLinearFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, w, pv, sizes):
    ctx.pv = pv
    sizes_host = sizes.tolist()
    ctx.sizes_host = sizes_host
    ctx.save_for_backward(x, w)
    return grouped_mm_fwd(x, w, sizes, sizes_host)

  @staticmethod
  def backward(ctx, dy):
    x, w = ctx.saved_tensors
    pv, sizes_host = ctx.pv, ctx.sizes_host
    dy = dy.contiguous()
    dx = _grouped_mm(dy, w, sizes_host, tb=False)
    if pv is not None and pv.main_grad is not None:
      g = pv.main_grad.view(w.shape)
      s = 0
      for e, n in enumerate(sizes_host):
        if n:
          F.mm(dy[s:s + n], x[s:s + n], True, False, out=g[e], accumulate=pv.grad_written)
        elif not pv.grad_written:
          g[e].zero_()
        s += n
      pv.grad_written = True
    return dx, None, None, None


def grouped_mm_fwd(x, w, sizes, sizes_host=None):
  if backend.use_cuda_kernels(x):
    E = backend.ext()
    if hasattr(E, "grouped_gemm_nt") and x.dtype == torch.bfloat16 and E.grouped_gemm_supported(x, w):
      out = torch.empty(x.shape[0], w.shape[1], dtype=x.dtype, device=x.device)
      E.grouped_gemm_nt(x, w, sizes.to(torch.int32), out)
      return out
  return _grouped_mm(x, w, sizes_host if sizes_host is not None else sizes.tolist(), tb=True)


def grouped_linear(x: torch.Tensor, p, sizes: torch.Tensor) -> torch.Tensor:
  """y[r] = x[r] @ W[e(r)].T with W = p.data [E, out, in] and rows grouped by expert."""
  if not torch.is_grad_enabled():
    return grouped_mm_fwd(x, p.data, sizes)
  return _GroupedLinearFn.apply(x, p.data, p, sizes)
