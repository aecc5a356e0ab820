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
from . import quantization as _quant
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


# ======================================================================================== padded-group GPU path
class GroupPlan:
  """Device-side description of one token->expert assignment in the padded row layout (no host synchronisation).

  Every expert's rows are padded to a multiple of 128 so that each GEMM tile belongs to one expert; `rows_max` is the
  static upper bound n + E * 127 rounded to 128 that sizes every buffer."""

  def __init__(self, expert_idx: torch.Tensor, num_experts: int):
    E_ = backend.ext()
    T, k = expert_idx.shape
    n = T * k
    self.T, self.k, self.E, self.n = T, k, num_experts, n
    self.rows_max = -(-(n + num_experts * 127) // 128) * 128
    dev = expert_idx.device
    i32 = dict(dtype=torch.int32, device=dev)
    self.sizes = torch.empty(num_experts, **i32)
    self.offs = torch.empty(num_experts + 1, **i32)
    self.blk_expert = torch.empty(self.rows_max // 128, **i32)
    self.dest = torch.empty(n, **i32)
    self.row_pair = torch.empty(self.rows_max, **i32)
    E_.moe_sort(expert_idx.reshape(-1).to(torch.int32).contiguous(), num_experts, self.sizes, self.offs, self.blk_expert, self.dest,
                self.row_pair)


def padded_path_supported(x2: torch.Tensor, d_model: int, d_ff: int, num_experts: int) -> bool:
  if not backend.use_cuda_kernels(x2) or x2.dtype != torch.bfloat16:
    return False
  E_ = backend.ext()
  return hasattr(E_, "grouped_gemm") and d_model % 128 == 0 and d_ff % 128 == 0 and num_experts <= 512


class _GatherRowsFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x2, plan):
    ctx.plan = plan
    rows = torch.empty(plan.rows_max, x2.shape[1], dtype=x2.dtype, device=x2.device)
    backend.ext().moe_gather(x2.contiguous(), plan.row_pair, plan.offs, plan.k, rows)
    return rows

  @staticmethod
  def backward(ctx, drows):
    plan = ctx.plan
    dx = torch.empty(plan.T, drows.shape[1], dtype=drows.dtype, device=drows.device)
    backend.ext().moe_combine(drows.contiguous(), plan.dest, None, plan.k, dx)      # each token sums its k rows, fixed order
    return dx, None


class _CombineFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, y, weights, plan):
    ctx.plan = plan
    w = weights.float().contiguous()
    ctx.save_for_backward(y, w)
    ctx.w_dtype = weights.dtype
    out = torch.empty(plan.T, y.shape[1], dtype=y.dtype, device=y.device)
    backend.ext().moe_combine(y, plan.dest, w.reshape(-1), plan.k, out)
    return out

  @staticmethod
  def backward(ctx, dout):
    y, w = ctx.saved_tensors
    plan = ctx.plan
    dy = torch.empty_like(y)
    dw = torch.empty_like(w)
    backend.ext().moe_combine_bwd(dout.contiguous(), y, plan.row_pair, plan.offs, w.reshape(-1), plan.k, dy, dw.view(-1))
    return dy, dw.to(ctx.w_dtype), None


def _dw_into(pv, dy, x, plan, shape):
  """dW[e] = dy_e^T x_e straight into the fp32 gradient store of parameter `pv` (accumulating if it already holds a gradient)."""
  E_ = backend.ext()
  if pv is not None and pv.main_grad is not None:
    E_.grouped_gemm(3, dy, x, pv.main_grad.view(shape), plan.offs, plan.blk_expert, bool(pv.grad_written))
    pv.grad_written = True
    return None
  g = torch.empty(shape, dtype=torch.float32, device=dy.device)
  E_.grouped_gemm(3, dy, x, g, plan.offs, plan.blk_expert, False)
  return g


class _ExpertsFFNFn(torch.autograd.Function):
  """h = act(rows W0_e^T) * (rows W1_e^T); y = h Wo_e^T over padded expert groups; every product is one grouped tcgen05 GEMM."""

  @staticmethod
  def forward(ctx, rows, w0, w1, wo, p0, p1, po, plan, act):
    E_ = backend.ext()
    Fdim = w0.shape[1]
    gu = torch.empty(plan.rows_max, 2 * Fdim, dtype=rows.dtype, device=rows.device)
    f8 = _quant.block_on() and Fdim % 16 == 0 and rows.shape[1] % 16 == 0      # block-scaled 8-bit forward / input-gradient products
    ctx.f8 = f8
    h = torch.empty(plan.rows_max, Fdim, dtype=rows.dtype, device=rows.device)
    y = torch.empty(plan.rows_max, wo.shape[1], dtype=rows.dtype, device=rows.device)
    if f8:
      E8 = backend.ext()
      rq, sr = E8.quant_fp8_rows(rows)                                         # one quantisation of the rows feeds both up-projections
      for w_, dst in ((w0, gu[:, :Fdim]), (w1, gu[:, Fdim:])):
        wq, _, sw = E8.quant_fp8_blocks(w_, True, False)
        E8.gemm_fp8_block(rq, sr, wq, sw, False, dst, plan.offs, plan.blk_expert)
      E_.gated_act_fwd(gu, h, F._ACT_CODE[act])
      _quant.block_grouped_fwd(h, wo, plan.offs, plan.blk_expert, y)
    else:
      E_.grouped_gemm(1, rows, w0, gu[:, :Fdim], plan.offs, plan.blk_expert, False)
      E_.grouped_gemm(1, rows, w1, gu[:, Fdim:], plan.offs, plan.blk_expert, False)
      E_.gated_act_fwd(gu, h, F._ACT_CODE[act])
      E_.grouped_gemm(1, h, wo, y, plan.offs, plan.blk_expert, False)
    ctx.save_for_backward(rows, gu, w0, w1, wo)
    ctx.misc = (p0, p1, po, plan, act)
    return y

  @staticmethod
  def backward(ctx, dy):
    E_ = backend.ext()
    rows, gu, w0, w1, wo = ctx.saved_tensors
    p0, p1, po, plan, act = ctx.misc
    Fdim = w0.shape[1]
    dy = dy.contiguous()
    h = torch.empty(plan.rows_max, Fdim, dtype=rows.dtype, device=rows.device)
    E_.gated_act_fwd(gu, h, F._ACT_CODE[act])                     # recomputed: cheaper than keeping it
    g_o = _dw_into(po, dy, h, plan, wo.shape)
    f8 = getattr(ctx, "f8", False)
    dh = h                                                          # reuse the buffer
    if f8:
      _quant.block_grouped_dx(dy, wo, plan.offs, plan.blk_expert, dh)
    else:
      E_.grouped_gemm(2, dy, wo, dh, plan.offs, plan.blk_expert, False)
    dgu = torch.empty_like(gu)
    E_.gated_act_bwd(dh, gu, dgu, F._ACT_CODE[act])
    d0, d1 = dgu[:, :Fdim], dgu[:, Fdim:]
    g_0 = _dw_into(p0, d0, rows, plan, w0.shape)
    g_1 = _dw_into(p1, d1, rows, plan, w1.shape)
    drows = torch.empty_like(rows)
    tmp = torch.empty_like(rows)
    if f8:
      _quant.block_grouped_dx(d0, w0, plan.offs, plan.blk_expert, drows)
      _quant.block_grouped_dx(d1, w1, plan.offs, plan.blk_expert, tmp)
    else:
      E_.grouped_gemm(2, d0, w0, drows, plan.offs, plan.blk_expert, False)
      E_.grouped_gemm(2, d1, w1, tmp, plan.offs, plan.blk_expert, False)
    drows.add_(tmp)
    return drows, g_0, g_1, g_o, None, None, None, None, None


def moe_ffn_padded(x2, weights, expert_idx, p_wi0, p_wi1, p_wo, num_experts: int, act: str):
  """Whole routed-expert computation for one rank's experts: sort -> gather -> grouped FFN -> weighted combine."""
  plan = GroupPlan(expert_idx, num_experts)
  grad = torch.is_grad_enabled()
  w0, w1, wo = p_wi0.data, p_wi1.data, p_wo.data
  if grad:
    rows = _GatherRowsFn.apply(x2, plan)
    y = _ExpertsFFNFn.apply(rows, w0, w1, wo, p_wi0, p_wi1, p_wo, plan, act)
    return _CombineFn.apply(y, weights, plan)
  rows = _GatherRowsFn.forward(F._Dummy(), x2, plan)
  y = _ExpertsFFNFn.forward(F._Dummy(), rows, w0, w1, wo, None, None, None, plan, act)
  return _CombineFn.forward(F._Dummy(), y, weights, plan)


# =============================================================================== router (softmax / sigmoid + top-k in one launch)
class _RouterFn(torch.autograd.Function):
  """Scores, top-k indices and routing weights of the MoE router from one kernel (`csrc/router_sm100.cu`); the gradient of
  these few [T, E] / [T, k] tensors is assembled here from the saved outputs."""

  @staticmethod
  def forward(ctx, logits, bias, k, mode, sigmoid_scores, raw_weights, scaling):
    idx, wts, probs, counts = backend.ext().router_topk(logits.contiguous(), bias, int(k), int(mode), bool(sigmoid_scores), bool(raw_weights),
                                                        float(scaling))
    ctx.save_for_backward(idx, wts, probs)
    ctx.cfg = (int(mode), bool(sigmoid_scores), bool(raw_weights), float(scaling), logits.dtype)
    ctx.mark_non_differentiable(idx, counts)
    return idx, wts, probs, counts

  @staticmethod
  def backward(ctx, _didx, dwts, dprobs, _dcounts):
    idx, wts, probs = ctx.saved_tensors
    mode, sig, raw, scaling, dtype = ctx.cfg
    li = idx.long()
    dscore = dprobs.clone() if dprobs is not None else torch.zeros_like(probs)       # gradient w.r.t. the scores (mode 1) / probs
    dlogits = torch.zeros_like(probs)
    if dwts is not None:
      if mode == 1:
        sel = probs.gather(1, li)
        if sig:
          tot = sel.sum(-1, keepdim=True) + 1e-20
          w = sel / tot                                                              # wts / scaling
          g = dwts * scaling
          dsel = (g - (g * w).sum(-1, keepdim=True)) / tot
        else:
          dsel = dwts * scaling
        dscore.scatter_add_(1, li, dsel)
      elif raw:
        dlogits.scatter_add_(1, li, dwts)
      else:
        dv = wts * (dwts - (dwts * wts).sum(-1, keepdim=True))                        # softmax over the k selected logits
        dlogits.scatter_add_(1, li, dv)
    if mode == 1 and sig:
      dlogits += dscore * probs * (1.0 - probs)
    else:
      dlogits += probs * (dscore - (dscore * probs).sum(-1, keepdim=True))            # softmax over all experts
    return dlogits.to(dtype), None, None, None, None, None, None


def router_topk(logits: torch.Tensor, bias, k: int, mode: int = 0, sigmoid_scores: bool = False, raw_weights: bool = False,
                scaling: float = 1.0):
  """(idx [T,k] int64, wts [T,k] fp32, probs [T,E] fp32, counts [E] int32) on a GPU; see `_RouterFn`."""
  b = bias.detach().float().contiguous() if bias is not None else None
  if torch.is_grad_enabled() and logits.requires_grad:
    idx, wts, probs, counts = _RouterFn.apply(logits, b, k, mode, sigmoid_scores, raw_weights, scaling)
  else:
    idx, wts, probs, counts = backend.ext().router_topk(logits.contiguous(), b, int(k), int(mode), bool(sigmoid_scores), bool(raw_weights),
                                                        float(scaling))
  return idx.long(), wts, probs, counts


def router_kernel_ok(logits: torch.Tensor, E: int, k: int) -> bool:
  return backend.use_cuda_kernels(logits) and logits.dtype in (torch.float32, torch.bfloat16) and E <= 512 and k <= 32 and k <= E
