"""Differentiable building blocks that write weight gradients straight into the parameter store.

Every op takes `Param` handles (see `parallel.param_store`) instead of autograd leaves: the backward
of a linear layer launches the dW GEMM with the fp32 `main_grad` view as its output (beta = 1 when a
gradient is already there), so no bf16 weight-gradient tensor is ever materialised and gradient
accumulation is free. On a GPU each op launches the hand-written sm_100a kernels of `csrc/`; on CPU
it evaluates the PyTorch definition in `ops.reference` (the numerical oracle of the kernel tests).
"""
from __future__ import annotations

import math
import os

import torch

from . import backend
from . import quantization as _quant, reference as ref

_GEMM_IMPL = os.environ.get("MAXTEXT_B200_GEMM", "tcgen05")   # "tcgen05" (product) | "cublas" (A/B comparison only)
_ATTN_IMPL = os.environ.get("MAXTEXT_B200_ATTN", "auto")


# =============================================================================== GEMM
_GEMM_FALLBACKS = 0
_ATTN_FALLBACKS = 0


def attention_fallbacks() -> int:
  """How many attention forward / backward calls on a GPU were evaluated by PyTorch ops instead of the flash kernels."""
  return _ATTN_FALLBACKS


def gemm_fallbacks() -> int:
  """How many matrix products on a GPU went to the library because the tcgen05 kernels do not cover their shape."""
  return _GEMM_FALLBACKS


def _small_m_wins(M, N, K) -> bool:
  """Shapes on which the weight-streaming kernel measured faster than the library's small-M kernels on a B200 (4096 x 4096
  weights at M <= 32: 11.4 - 15.3 us against 15.6 - 17.1 us). Its mma.sync inner loop runs out of issue rate above M = 32, and
  on wider or deeper weights the library's kernels are ahead, so those go to the library (and are counted as fallbacks).
  MAXTEXT_B200_SMALL_M=all / none overrides the rule."""
  mode = os.environ.get("MAXTEXT_B200_SMALL_M", "")
  if mode == "none" or M > 64:
    return False
  if mode == "all":
    return True
  return M <= 32 and N <= 4096 and K <= 4096


def _gemm_supported(M, N, K, a, b):
  return a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and K % 8 == 0 and N % 8 == 0 and K >= 16


def mm(a: torch.Tensor, b: torch.Tensor, ta: bool, tb: bool, out: torch.Tensor | None = None,
       accumulate: bool = False, out_dtype: torch.dtype | None = None) -> torch.Tensor:
  """out (+)= op(a) @ op(b) with op(a) = a.T if ta, op(b) = b.T if tb; fp32 accumulation.

  The three layouts used by training are nt (forward x @ W.T), nn (dX = dY @ W) and tn
  (dW = dY.T @ X). `out` may be fp32 (gradient accumulators) or the compute dtype.
  """
  M = a.shape[1] if ta else a.shape[0]
  K = a.shape[0] if ta else a.shape[1]
  N = b.shape[0] if tb else b.shape[1]
  if out is None:
    out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
    accumulate = False
  if a.is_cuda:
    E = backend.ext(required=True)
    if (_GEMM_IMPL == "tcgen05" and not ta and tb and not accumulate and out.dtype == torch.bfloat16 and _small_m_wins(M, N, K)
        and E.gemm_small_m_supported(a, b, out)):
      E.gemm_small_m(a, b, out)            # decode-sized products stream the weight once (csrc/gemm_small_m.cu)
      return out
    if _GEMM_IMPL == "tcgen05" and _gemm_supported(M, N, K, a, b) and E.gemm_supported(a, b, out, ta, tb):
      E.gemm(a, b, out, ta, tb, accumulate)
      return out
    if _GEMM_IMPL == "tcgen05":
      global _GEMM_FALLBACKS
      _GEMM_FALLBACKS += 1
      if os.environ.get("MAXTEXT_B200_STRICT_GEMM") == "1":
        raise RuntimeError(f"tcgen05 GEMM does not cover M={M} N={N} K={K} {a.dtype} (strides {a.stride()}, {b.stride()})")
  opa, opb = (a.t() if ta else a), (b.t() if tb else b)
  if accumulate:
    if out.dtype == a.dtype:
      out.addmm_(opa, opb)
    else:
      out.add_(torch.mm(opa, opb).to(out.dtype)) if a.is_cuda else out.add_(torch.mm(opa.float(), opb.float()).to(out.dtype))
  else:
    if out.dtype == a.dtype:
      torch.mm(opa, opb, out=out)
    elif a.is_cuda:
      out.copy_(torch.mm(opa, opb))
    else:
      out.copy_(torch.mm(opa.float(), opb.float()))
  return out


class _LinearFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, w, pv, saved_out, bias, precomputed=None, tp_reduce_dx=None):
    ctx.pv = pv
    ctx.tp_reduce_dx = tp_reduce_dx
    x2 = x
    ctx.save_for_backward(x2, w)
    ctx.has_bias = bias is not None
    ctx.fp8 = False
    if precomputed is not None:
      return precomputed
    if saved_out is not None:
      # a copy: callers may transform the projection in place (rotary embedding on the packed q|k|v)
      return saved_out.reshape(-1, w.shape[0]).clone()
    ctx.fp8b = _quant.block_supported(x2, w)
    ctx.fp8 = not ctx.fp8b and _quant.supported(x2, w)
    ctx.fp8_saved = None
    ctx.int8 = _quant.int8_on()
    if ctx.fp8b:
      y = _quant.block_linear_fwd(x2, w)
    elif ctx.int8:
      y = _quant.int8_linear_fwd(x2, w)
    elif ctx.fp8:
      y, ctx.fp8_saved = _quant.linear_fwd(x2, w, pv, keep_for_bwd=True)     # this forward will be differentiated: quantise once for both passes
    else:
      y = mm(x2, w, False, True)
    if bias is not None:
      y = y + bias.to(y.dtype)
    return y

  @staticmethod
  def backward(ctx, dy):
    x2, w = ctx.saved_tensors
    pv = ctx.pv
    dy2 = dy.reshape(-1, dy.shape[-1])
    if not dy2.is_contiguous():
      dy2 = dy2.contiguous()
    if getattr(ctx, "fp8", False) and ctx.tp_reduce_dx is None and _quant.supported(dy2, w):
      go = pv.main_grad.view(w.shape) if (pv is not None and pv.main_grad is not None and not getattr(pv, "frozen", False)) else None
      dx = _quant.linear_bwd(dy2, x2, w, bool(ctx.needs_input_grad[0]), go, bool(pv.grad_written) if go is not None else False, pv,
                             getattr(ctx, "fp8_saved", None))
      ctx.fp8_saved = None
      if go is not None:
        pv.grad_written = True
      dbias = dy2.float().sum(0) if ctx.has_bias else None
      return dx, None, None, None, dbias, None, None
    if not ctx.needs_input_grad[0]:
      dx = None
    elif getattr(ctx, "fp8b", False) and ctx.tp_reduce_dx is None and _quant.block_supported(dy2, w):
      dx = _quant.block_linear_dx(dy2, w)
    elif getattr(ctx, "int8", False) and ctx.tp_reduce_dx is None:
      dx = _quant.int8_linear_dx(dy2, w)
    elif ctx.tp_reduce_dx is not None:
      dx = ctx.tp_reduce_dx.all_reduce_gemm(dy2, w, False)      # column-parallel input gradient: summed over the TP ranks in the GEMM
    else:
      dx = mm(dy2, w, False, False)
    if pv is not None and pv.main_grad is not None and not getattr(pv, "frozen", False):
      mm(dy2, x2, True, False, out=pv.main_grad.view(w.shape), accumulate=pv.grad_written)
      pv.grad_written = True
    dbias = dy2.float().sum(0) if ctx.has_bias else None
    return dx, None, None, None, dbias, None, None


def linear(x: torch.Tensor, p, saved_out: torch.Tensor | None = None, bias=None, tp_reduce=None, tp_reduce_dx=None) -> torch.Tensor:
  """y = x @ W.T for W = p.data stored [out, in]. `saved_out` short-cuts the forward GEMM when a remat
  policy kept this projection's output. `tp_reduce` (a parallel.tp_fused runtime) sums the product over the
  tensor-parallel ranks inside the GEMM (row-parallel layers); `tp_reduce_dx` does the same for the input gradient
  (column-parallel layers)."""
  b = bias.leaf() if bias is not None else None
  x2 = x.reshape(-1, x.shape[-1])
  if not x2.is_contiguous():
    x2 = x2.contiguous()
  # FSDP: when the unit's all-gather is still pending, this GEMM performs it inside its own launch
  pre = None
  pend = p.pending_unit() if hasattr(p, "pending_unit") else None
  if tp_reduce is not None and saved_out is None and b is None:
    pre = tp_reduce.all_reduce_gemm(x2, p.data, True)
  elif pend is not None and saved_out is None and b is None:
    pre = pend.store.ag_linear(pend, p, x2)
  lo = getattr(p, "lora", None)
  if not torch.is_grad_enabled():
    if saved_out is not None:
      return saved_out
    y = (pre if pre is not None else _quant.block_linear_fwd(x2, p.data) if _quant.block_supported(x2, p.data) else
         _quant.int8_linear_fwd(x2, p.data) if _quant.int8_on() else
         (_quant.linear_fwd(x2, p.data, p) if _quant.supported(x2, p.data) else mm(x2, p.data, False, True)))
    if lo is not None:
      y = y + _lora_delta(x2, lo).to(y.dtype)
    y = y.view(*x.shape[:-1], p.shape[0])
    return y + b.to(y.dtype) if b is not None else y
  y = _LinearFn.apply(x2, p.data, p, saved_out, b, pre, tp_reduce_dx)
  if lo is not None:
    d = _lora_delta(x2, lo).to(y.dtype)
    # a kept output already contains the adapter's contribution: add only its gradient path
    y = y + (d - d.detach() if saved_out is not None else d)
  return y.view(*x.shape[:-1], p.shape[0])


def _lora_delta(x2: torch.Tensor, lo) -> torch.Tensor:
  """scale * (x A^T) B^T for a low-rank adapter (A [r, in], B [out, r]); both products go through `linear`, so the
  adapters' gradients land in their fp32 accumulators like any other weight's."""
  a, b, scale = lo
  return linear(linear(x2, a), b) * scale


# =============================================================================== RMSNorm
class _RMSNormFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, scale, pv, eps, offset):
    ctx.pv, ctx.eps, ctx.offset = pv, eps, offset
    if backend.use_cuda_kernels(x) and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
      E = backend.ext()
      x2 = x.reshape(-1, x.shape[-1])
      if not x2.is_contiguous():
        x2 = x2.contiguous()
      y = torch.empty_like(x2)
      rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
      E.rmsnorm_fwd(x2, scale, float(eps), float(offset), y, rstd)
      ctx.save_for_backward(x2, scale, rstd)
      ctx.cuda = True
      return y
    ctx.cuda = False
    ctx.save_for_backward(x, scale)
    return ref.rmsnorm(x, scale, eps, offset)

  @staticmethod
  def backward(ctx, dy):
    pv = ctx.pv
    if ctx.cuda:
      x2, scale, rstd = ctx.saved_tensors
      E = backend.ext()
      dy2 = dy.reshape(x2.shape)
      if not dy2.is_contiguous():
        dy2 = dy2.contiguous()
      dx = torch.empty_like(x2)
      want_ds = scale is not None and pv is not None and pv.main_grad is not None
      if want_ds and not pv.grad_written:
        pv.main_grad.zero_()
        pv.grad_written = True
      E.rmsnorm_bwd(dy2, x2, scale, rstd, float(ctx.offset), dx, pv.main_grad if want_ds else None)
      return dx, None, None, None, None
    x, scale = ctx.saved_tensors
    dx, ds = ref.rmsnorm_bwd(dy, x, scale, ctx.eps, ctx.offset)
    if ds is not None and pv is not None and pv.main_grad is not None:
      pv.accumulate_grad(ds)
    return dx, None, None, None, None


def rmsnorm(x: torch.Tensor, p, eps: float, offset: float = 0.0) -> torch.Tensor:
  scale = p.data if p is not None else None
  if not torch.is_grad_enabled():
    if backend.use_cuda_kernels(x) and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
      x2 = x.reshape(-1, x.shape[-1])
      x2 = x2 if x2.is_contiguous() else x2.contiguous()
      y = torch.empty_like(x2)
      backend.ext().rmsnorm_fwd(x2, scale, float(eps), float(offset), y, None)
      return y.view(x.shape)
    return ref.rmsnorm(x, scale, eps, offset)
  x2 = x.reshape(-1, x.shape[-1])
  if not x2.is_contiguous():
    x2 = x2.contiguous()
  return _RMSNormFn.apply(x2, scale, p, eps, offset).view(x.shape)


# =============================================================================== gated activation
_ACT_CODE = {"silu": 0, "swish": 0, "gelu": 1, "relu": 2, "linear": 3}


class _GatedActFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, gu, act):
    ctx.act = act
    ctx.save_for_backward(gu)
    if backend.use_cuda_kernels(gu) and gu.dtype == torch.bfloat16 and act in _ACT_CODE and gu.shape[-1] % 16 == 0:
      g2 = gu.reshape(-1, gu.shape[-1])
      out = torch.empty(g2.shape[0], g2.shape[1] // 2, dtype=gu.dtype, device=gu.device)
      backend.ext().gated_act_fwd(g2, out, _ACT_CODE[act])
      return out
    return ref.gated_act(gu, act)

  @staticmethod
  def backward(ctx, dy):
    (gu,) = ctx.saved_tensors
    if backend.use_cuda_kernels(gu) and gu.dtype == torch.bfloat16 and ctx.act in _ACT_CODE and gu.shape[-1] % 16 == 0:
      g2 = gu.reshape(-1, gu.shape[-1])
      dy2 = dy.reshape(-1, dy.shape[-1])
      dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
      dgu = torch.empty_like(g2)
      backend.ext().gated_act_bwd(dy2, g2, dgu, _ACT_CODE[ctx.act])
      return dgu, None
    return ref.gated_act_bwd(dy, gu, ctx.act), None


def gated_act(gate_up: torch.Tensor, act: str = "silu") -> torch.Tensor:
  """act(gate) * up for an input laid out [..., gate | up]."""
  g2 = gate_up.reshape(-1, gate_up.shape[-1])
  if not g2.is_contiguous():
    g2 = g2.contiguous()
  if not torch.is_grad_enabled():
    out = _GatedActFn.forward(_Dummy(), g2, act)
  else:
    out = _GatedActFn.apply(g2, act)
  return out.view(*gate_up.shape[:-1], gate_up.shape[-1] // 2)


class _Dummy:
  """Stand-in ctx so Function.forward bodies can be reused under no_grad."""
  def save_for_backward(self, *a):
    pass

  def mark_dirty(self, *a):
    pass


# =============================================================================== rope (+ packed attention)
def rope_packed_(qkv: torch.Tensor, positions: torch.Tensor, inv_ts: torch.Tensor, n_rot_heads: int,
                 interleaved: bool, inverse: bool = False, rotary_dim: int | None = None):
  """Rotate, in place, the first `n_rot_heads` heads of a packed [B,S,H,Dh] tensor."""
  B, S, H, Dh = qkv.shape
  if backend.use_cuda_kernels(qkv) and qkv.dtype == torch.bfloat16 and qkv.is_contiguous():
    backend.ext().rope_inplace(qkv.view(B * S, H, Dh), positions.reshape(-1).to(torch.int32), inv_ts, n_rot_heads,
                               bool(interleaved), bool(inverse), int(rotary_dim or Dh))
    return qkv
  part = ref.apply_rope(qkv[:, :, :n_rot_heads], positions, inv_ts, interleaved, rotary_dim, inverse)
  qkv[:, :, :n_rot_heads].copy_(part)
  return qkv


def _sdpa_reference(q, k, v, mask_args, scale, soft_cap):
  m = ref.attention_mask(**mask_args)
  return ref.attention(q, k, v, m, scale, soft_cap, return_lse=True)


class _PackedAttnFn(torch.autograd.Function):
  """rope + causal/segment/sliding flash attention over a packed [B,S,Hq+2Hkv,Dh] projection."""

  @staticmethod
  def forward(ctx, qkv, positions, segment_ids, inv_ts, hq, hkv, interleaved, scale, soft_cap, window, use_rope):
    B, S, H, Dh = qkv.shape
    qkv = qkv.contiguous()
    if use_rope:
      rope_packed_(qkv, positions, inv_ts, hq + hkv, interleaved)
    q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hkv], qkv[:, :, hq + hkv:]
    out, lse = attention_fwd(q, k, v, positions, segment_ids, scale, soft_cap, window)
    ctx.save_for_backward(qkv, out, lse, positions, segment_ids, inv_ts)
    ctx.cfg = (hq, hkv, interleaved, scale, soft_cap, window, use_rope)
    return out

  @staticmethod
  def backward(ctx, dout):
    qkv, out, lse, positions, segment_ids, inv_ts = ctx.saved_tensors
    hq, hkv, interleaved, scale, soft_cap, window, use_rope = ctx.cfg
    q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hkv], qkv[:, :, hq + hkv:]
    dqkv = torch.empty_like(qkv)
    attention_bwd(dout.contiguous(), q, k, v, out, lse, positions, segment_ids, scale, soft_cap, window,
                  dqkv[:, :, :hq], dqkv[:, :, hq:hq + hkv], dqkv[:, :, hq + hkv:])
    if use_rope:
      rope_packed_(dqkv, positions, inv_ts, hq + hkv, interleaved, inverse=True)
    return (dqkv,) + (None,) * 10


def packed_attention(qkv, positions, segment_ids, inv_ts, hq, hkv, interleaved=False, scale=1.0, soft_cap=0.0,
                     window=0, use_rope=True):
  if not torch.is_grad_enabled():
    return _PackedAttnFn.forward(_Dummy(), qkv, positions, segment_ids, inv_ts, hq, hkv, interleaved, scale, soft_cap,
                                 window, use_rope)
  return _PackedAttnFn.apply(qkv, positions, segment_ids, inv_ts, hq, hkv, interleaved, scale, soft_cap, window, use_rope)


def _flash_ok(q, k, v, soft_cap):
  return q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == v.shape[-1] and q.shape[-1] in (64, 128) and not soft_cap


def _i32(t):
  return None if t is None else t.to(torch.int32).contiguous()


def attention_fwd(q, k, v, positions, segment_ids, scale, soft_cap, window, causal=True, kv_positions=None,
                  kv_segment_ids=None, chunk=0, sinks=None):
  """Returns (out [B,Sq,Hq,Dv], lse [B,Hq,Sq] fp32). Strided q/k/v views are accepted.

  On a GPU this is the tcgen05 flash kernel for every mask form the models use: causal or not, sliding window, chunked
  attention, segment ids, logit soft-cap, per-head sink logits, Dqk != Dv (MLA), any sequence length, and keys that are
  a block of a longer sequence (`kv_positions` / `kv_segment_ids`, context parallelism). `positions` are only consulted
  when the mask cannot be derived from token indices: with kv_positions, or chunked attention over packed rows."""
  if backend.use_cuda_kernels(q):
    E = backend.ext()
    if q.dtype == torch.bfloat16 and _ATTN_IMPL != "sdpa" and E.flash_fwd_supported(q, k, v):
      out = torch.empty(q.shape[0], q.shape[1], q.shape[2], v.shape[-1], dtype=q.dtype, device=q.device)
      lse = torch.empty(q.shape[0], q.shape[2], q.shape[1], dtype=torch.float32, device=q.device)
      seg_q = _i32(segment_ids)
      seg_k = _i32(kv_segment_ids) if kv_segment_ids is not None else seg_q
      if seg_q is None:
        seg_k = None
      by_arrays = kv_positions is not None or (chunk and segment_ids is not None)
      pos_q = _i32(positions) if by_arrays else None
      pos_k = _i32(kv_positions if kv_positions is not None else positions) if by_arrays else None
      sk = sinks.detach().float().contiguous() if sinks is not None else None
      E.flash_fwd(q, k, v, out, lse, seg_q, seg_k, pos_q, pos_k, sk, float(scale), float(soft_cap or 0.0), bool(causal), int(window or 0),
                  int(chunk or 0), int(k.shape[1] - q.shape[1]) if not by_arrays else 0)
      return out, lse
  mask_args = dict(q_pos=positions, kv_pos=kv_positions if kv_positions is not None else positions, q_seg=segment_ids,
                   kv_seg=kv_segment_ids if kv_segment_ids is not None else segment_ids, causal=causal,
                   sliding_window=window, chunk=chunk)
  if q.is_cuda:
    global _ATTN_FALLBACKS
    _ATTN_FALLBACKS += 1
    if _ATTN_IMPL == "sdpa" and segment_ids is None and not window and not soft_cap and causal and kv_positions is None and not chunk \
        and sinks is None:
      # comparison arm only (library attention); the product path is the flash kernel above
      o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                           is_causal=True, scale=scale, enable_gqa=q.shape[2] != k.shape[2])
      return o.transpose(1, 2).contiguous(), None
    return _attention_chunked(q, k, v, mask_args, scale, soft_cap, sinks=sinks)
  m = ref.attention_mask(**mask_args)
  return ref.attention(q, k, v, m, scale, soft_cap, sinks=sinks, return_lse=True)


def _attention_chunked(q, k, v, mask_args, scale, soft_cap, chunk=1024, sinks=None):
  """Memory-bounded evaluation of the reference attention on GPU (query chunks)."""
  outs, lses = [], []
  Sq = q.shape[1]
  for s in range(0, Sq, chunk):
    ma = dict(mask_args)
    ma["q_pos"] = mask_args["q_pos"][:, s:s + chunk]
    if ma.get("q_seg") is not None:
      ma["q_seg"] = mask_args["q_seg"][:, s:s + chunk]
    o, l = ref.attention(q[:, s:s + chunk], k, v, ref.attention_mask(**ma), scale, soft_cap, sinks=sinks, return_lse=True)
    outs.append(o)
    lses.append(l)
  return torch.cat(outs, 1), torch.cat(lses, 2)


def attention_bwd(dout, q, k, v, out, lse, positions, segment_ids, scale, soft_cap, window, dq, dk, dv, causal=True,
                  kv_positions=None, kv_segment_ids=None, chunk=0, sinks=None):
  """Gradients of attention given the forward's `out` and `lse`. With kv_positions the keys are a block of a longer
  (context-parallel) sequence: `out`/`lse` are then the merged global results and the returned dq/dk/dv are this
  block's exact contributions. Returns the gradient of the sink logits (or None)."""
  dsinks = None
  if sinks is not None and lse is not None:
    # d loss / d sink_h = -sum_{b,q} p_sink * delta, with p_sink = exp(sink - lse) and delta = rowsum(dO * O)
    delta = (dout.float() * out.float()).sum(-1).permute(0, 2, 1)                 # [B, Hq, Sq]
    dsinks = -(torch.exp(sinks.detach().float()[None, :, None] - lse) * delta).sum((0, 2)).to(sinks.dtype)
  if backend.use_cuda_kernels(q) and lse is not None and q.dtype == torch.bfloat16:
    E = backend.ext()
    if E.flash_bwd_supported(q, k, v) and E.flash_fwd_supported(dq, dk, dv):
      seg_q = _i32(segment_ids)
      seg_k = _i32(kv_segment_ids) if kv_segment_ids is not None else seg_q
      if seg_q is None:
        seg_k = None
      by_arrays = kv_positions is not None or (chunk and segment_ids is not None)
      pos_q = _i32(positions) if by_arrays else None
      pos_k = _i32(kv_positions if kv_positions is not None else positions) if by_arrays else None
      E.flash_bwd(dout if dout.is_contiguous() else dout.contiguous(), q, k, v, out if out.is_contiguous() else out.contiguous(), lse, dq, dk, dv,
                  seg_q, seg_k, pos_q, pos_k, float(scale), float(soft_cap or 0.0), bool(causal), int(window or 0), int(chunk or 0),
                  int(k.shape[1] - q.shape[1]) if not by_arrays else 0)
      return dsinks
  kpos = kv_positions if kv_positions is not None else positions
  kseg = kv_segment_ids if kv_segment_ids is not None else segment_ids
  if q.is_cuda:
    global _ATTN_FALLBACKS
    _ATTN_FALLBACKS += 1
  if lse is None:
    # comparison arm (library attention): differentiate the library call
    with torch.enable_grad():
      ql, kl, vl = (t.detach().requires_grad_(True) for t in (q, k, v))
      o = torch.nn.functional.scaled_dot_product_attention(ql.transpose(1, 2), kl.transpose(1, 2), vl.transpose(1, 2),
                                                           is_causal=True, scale=scale, enable_gqa=q.shape[2] != k.shape[2])
      gq, gk, gv = torch.autograd.grad(o, (ql, kl, vl), dout.transpose(1, 2))
    dq.copy_(gq)
    dk.copy_(gk)
    dv.copy_(gv)
    return dsinks
  # reference: recompute probabilities from lse, chunked over queries
  B, Sq, Hq, D = q.shape
  Hkv = k.shape[2]
  g = Hq // Hkv
  kf, vf = k.float(), v.float()
  dkf = torch.zeros(B, k.shape[1], Hkv, D, dtype=torch.float32, device=q.device)
  dvf = torch.zeros(B, v.shape[1], Hkv, v.shape[-1], dtype=torch.float32, device=q.device)
  step = 1024 if q.is_cuda else Sq
  for s in range(0, Sq, step):
    e = min(Sq, s + step)
    qf = q[:, s:e].float().reshape(B, e - s, Hkv, g, D)
    mask = ref.attention_mask(positions[:, s:e], kpos, segment_ids[:, s:e] if segment_ids is not None else None,
                              kseg, causal, window, chunk)
    raw = torch.einsum("bqhgd,bkhd->bhgqk", qf, kf) * scale
    if soft_cap and soft_cap > 0:
      t = torch.tanh(raw / soft_cap)
      logits = t * soft_cap
    else:
      logits = raw
    l = lse[:, :, s:e].reshape(B, Hkv, g, e - s)
    p = torch.exp(logits - l[..., None]).masked_fill(~mask[:, :, None], 0.0)
    do = dout[:, s:e].float().reshape(B, e - s, Hkv, g, -1)
    o = out[:, s:e].float().reshape(B, e - s, Hkv, g, -1)
    dvf += torch.einsum("bhgqk,bqhgd->bkhd", p, do)
    dp = torch.einsum("bqhgd,bkhd->bhgqk", do, vf)
    delta = (do * o).sum(-1).permute(0, 2, 3, 1)  # b h g q
    ds = p * (dp - delta[..., None])
    if soft_cap and soft_cap > 0:
      ds = ds * (1 - t * t)
    ds = ds * scale
    dq[:, s:e].copy_(torch.einsum("bhgqk,bkhd->bqhgd", ds, kf).reshape(B, e - s, Hq, D).to(dq.dtype))
    dkf += torch.einsum("bhgqk,bqhgd->bkhd", ds, qf)
  dk.copy_(dkf.to(dk.dtype))
  dv.copy_(dvf.to(dv.dtype))
  return dsinks


class _AttnFn(torch.autograd.Function):
  """Attention over separate q/k/v tensors (used when q/k need per-head norms or differ in width)."""

  @staticmethod
  def forward(ctx, q, k, v, positions, segment_ids, scale, soft_cap, window, causal, kv_positions=None, kv_segment_ids=None, chunk=0,
              sinks=None):
    out, lse = attention_fwd(q, k, v, positions, segment_ids, scale, soft_cap, window, causal, kv_positions, kv_segment_ids, chunk, sinks)
    ctx.save_for_backward(q, k, v, out, lse, positions, segment_ids, kv_positions, kv_segment_ids, sinks)
    ctx.cfg = (scale, soft_cap, window, causal, chunk)
    return out

  @staticmethod
  def backward(ctx, dout):
    q, k, v, out, lse, positions, segment_ids, kpos, kseg, sinks = ctx.saved_tensors
    scale, soft_cap, window, causal, chunk = ctx.cfg
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dsinks = attention_bwd(dout.contiguous(), q, k, v, out, lse, positions, segment_ids, scale, soft_cap, window, dq, dk, dv, causal, kpos,
                           kseg, chunk, sinks)
    return dq, dk, dv, None, None, None, None, None, None, None, None, None, dsinks


def attention(q, k, v, positions, segment_ids, scale=1.0, soft_cap=0.0, window=0, causal=True, kv_positions=None, kv_segment_ids=None,
              chunk=0, sinks=None):
  """kv_positions / kv_segment_ids describe keys that are not the queries' own tokens (context parallelism); `chunk` restricts
  attention to blocks of that many positions; `sinks` [Hq] are per-head logits that only enter the softmax denominator."""
  if not torch.is_grad_enabled():
    return attention_fwd(q, k, v, positions, segment_ids, scale, soft_cap, window, causal, kv_positions, kv_segment_ids, chunk, sinks)[0]
  return _AttnFn.apply(q, k, v, positions, segment_ids, scale, soft_cap, window, causal, kv_positions, kv_segment_ids, chunk, sinks)


class _RopeFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, positions, inv_ts, interleaved, rotary_dim):
    ctx.save_for_backward(positions, inv_ts)
    ctx.cfg = (interleaved, rotary_dim)
    y = x.contiguous().clone()
    return rope_packed_(y, positions, inv_ts, y.shape[2], interleaved, False, rotary_dim)

  @staticmethod
  def backward(ctx, dy):
    positions, inv_ts = ctx.saved_tensors
    interleaved, rotary_dim = ctx.cfg
    dx = dy.contiguous().clone()
    return rope_packed_(dx, positions, inv_ts, dx.shape[2], interleaved, True, rotary_dim), None, None, None, None


def rope(x, positions, inv_ts, interleaved=False, rotary_dim=None):
  """Out-of-place rotary embedding of x [B,S,H,Dh]."""
  if not torch.is_grad_enabled():
    return rope_packed_(x.contiguous().clone(), positions, inv_ts, x.shape[2], interleaved, False, rotary_dim)
  return _RopeFn.apply(x, positions, inv_ts, interleaved, rotary_dim)


# =============================================================================== embedding
def embedding_lookup(tokens, table):
  if backend.use_cuda_kernels(table) and table.dtype == torch.bfloat16 and table.shape[1] % 8 == 0:
    out = torch.empty(*tokens.shape, table.shape[1], dtype=table.dtype, device=table.device)
    backend.ext().embedding_fwd(tokens.reshape(-1).to(torch.int32), table, out.view(-1, table.shape[1]))
    return out
  return table[tokens.long()]


def embedding_scatter_add(tokens, dy, grad_table):
  d2 = dy.reshape(-1, dy.shape[-1])
  if backend.use_cuda_kernels(d2) and d2.dtype == torch.bfloat16 and grad_table.dtype == torch.float32 and d2.shape[1] % 8 == 0:
    backend.ext().embedding_bwd(tokens.reshape(-1).to(torch.int32), d2.contiguous(), grad_table)
    return
  grad_table.index_add_(0, tokens.reshape(-1).long(), d2.to(grad_table.dtype))


def embedding(tokens: torch.Tensor, p) -> torch.Tensor:
  """Row gather from the [V, D] table. Its backward (a scatter-add into the fp32 gradient) only fires
  when the output requires grad, i.e. when it is called on a detached leaf by the engine."""
  if not torch.is_grad_enabled():
    return embedding_lookup(tokens, p.data)
  dummy = torch.zeros((), device=p.data.device, requires_grad=True)
  return _EmbedGradFn.apply(dummy, tokens, p.data, p)


class _EmbedGradFn(torch.autograd.Function):
  """Embedding whose autograd edge hangs off a dummy scalar so that backward is always invoked."""

  @staticmethod
  def forward(ctx, dummy, tokens, table, pv):
    ctx.pv = pv
    ctx.save_for_backward(tokens)
    return embedding_lookup(tokens, table)

  @staticmethod
  def backward(ctx, dy):
    (tokens,) = ctx.saved_tensors
    pv = ctx.pv
    if pv is not None and pv.main_grad is not None:
      if not pv.grad_written:
        pv.main_grad.zero_()
        pv.grad_written = True
      embedding_scatter_add(tokens, dy, pv.main_grad)
    return None, None, None, None


# =============================================================================== fused output head + loss
def fused_head_loss(h: torch.Tensor, head, targets: torch.Tensor, weights: torch.Tensor, z_loss: float = 0.0,
                    soft_cap: float = 0.0, chunk_tokens: int = 2048, logit_scale: float = 1.0, compute_grads: bool = True,
                    transposed_head: bool = False):
  """Output projection + cross entropy (+ z-loss) without materialising [tokens, vocab] in fp32.

  Tokens are processed in chunks: logits chunk = h_c @ W.T (compute dtype), loss and d(logits) are
  produced in place by one kernel, then dH_c = dlogits @ W and dW += dlogits.T @ h_c go straight into
  the gradient store. Because the loss is the last node of the graph the backward can run inside the
  forward; gradients are those of sum_t weights_t * loss_t (normalisation is applied with the global
  gradient scale in the optimizer). This plays the role of the reference's vocabulary tiling
  (src/maxtext/utils/vocabulary_tiling.py:280-496) and custom-VJP cross entropy
  (src/maxtext/utils/max_utils.py:626-716).

  head: Param with data [V, D] (or [D, V] -> transposed_head for tied embeddings is [V, D] already).
  Returns (loss_sum fp32 scalar, z_sum scalar, dh or None).
  """
  T, D = h.shape
  W = head.data
  loss_sum = torch.zeros((), dtype=torch.float32, device=h.device)
  z_sum = torch.zeros((), dtype=torch.float32, device=h.device)
  dh = torch.empty_like(h) if compute_grads else None
  use_k = backend.use_cuda_kernels(h) and h.dtype == torch.bfloat16 and not soft_cap
  for s in range(0, T, chunk_tokens):
    e = min(T, s + chunk_tokens)
    hc = h[s:e]
    logits = mm(hc, W, False, True)
    if logit_scale != 1.0:
      logits.mul_(logit_scale)
    tg, wt = targets[s:e], weights[s:e]
    if use_k:
      E = backend.ext()
      lt = torch.empty(e - s, dtype=torch.float32, device=h.device)
      zt = torch.empty(e - s, dtype=torch.float32, device=h.device)
      E.xent_fwd_bwd(logits, tg.to(torch.int32), wt.float(), float(z_loss), lt, zt, bool(compute_grads))
      loss_sum += (lt * wt).sum()
      z_sum += (zt * wt).sum()
      dlogits = logits
    else:
      lg = logits.float()
      if soft_cap and soft_cap > 0:
        capped = torch.tanh(lg / soft_cap) * soft_cap
      else:
        capped = lg
      lt, zt = ref.cross_entropy(capped, tg, z_loss)
      loss_sum += (lt * wt).sum()
      z_sum += (zt * wt).sum()
      if compute_grads:
        dl = ref.cross_entropy_dlogits(capped, tg, wt, z_loss)
        if soft_cap and soft_cap > 0:
          dl = dl * (1 - (capped / soft_cap) ** 2)
        dlogits = dl.to(h.dtype)
    if compute_grads:
      if logit_scale != 1.0:
        dlogits.mul_(logit_scale)
      mm(dlogits, W, False, False, out=dh[s:e])
      if head.main_grad is not None:
        mm(dlogits, hc, True, False, out=head.main_grad.view(W.shape), accumulate=head.grad_written)
        head.grad_written = True
    del logits
  return loss_sum, z_sum, dh


def head_logits(h: torch.Tensor, head, soft_cap: float = 0.0, logit_scale: float = 1.0) -> torch.Tensor:
  """Full fp32 logits (inference / evaluation of small batches)."""
  lg = mm(h.reshape(-1, h.shape[-1]), head.data, False, True).float().view(*h.shape[:-1], head.data.shape[0])
  if logit_scale != 1.0:
    lg = lg * logit_scale
  if soft_cap and soft_cap > 0:
    lg = torch.tanh(lg / soft_cap) * soft_cap
  return lg


# =============================================================================== optimizer kernels
def sum_of_squares(flat: torch.Tensor) -> torch.Tensor:
  if backend.use_cuda_kernels(flat) and flat.dtype == torch.float32 and flat.is_contiguous():
    out = torch.zeros(1, dtype=torch.float32, device=flat.device)
    backend.ext().sumsq(flat, out)
    return out[0]
  return flat.float().pow(2).sum()


def adamw_flat(master, grad, m, v, shadow, lr, b1, b2, eps, eps_root, wd, step, grad_scale: torch.Tensor, pax: bool = False):
  """Single-launch AdamW over a flat shard. `grad_scale` is a 1-element device tensor (clip factor x
  1/total_weights) so no host synchronisation is needed. `shadow` (compute dtype) may alias master.

  `pax` selects the praxis form (src/maxtext/optimizers/optimizers.py:289-310): the bias correction is folded into
  step-dependent decays, so the moments themselves are the corrected estimates and no division follows."""
  bc1, bc2 = 1.0 - b1 ** step, 1.0 - b2 ** step
  if pax:
    b1 = b1 * (1.0 - b1 ** (step - 1)) / bc1
    b2 = b2 * (1.0 - b2 ** (step - 1)) / bc2
    bc1 = bc2 = 1.0
  if backend.use_cuda_kernels(master) and master.dtype == torch.float32 and grad.dtype == torch.float32 \
      and v.dtype == torch.float32 and m.dtype in (torch.float32, torch.bfloat16) and master.numel() % 4 == 0 \
      and master.data_ptr() % 16 == 0:
    sh = shadow if (shadow is not None and shadow.data_ptr() != master.data_ptr()) else None
    backend.ext().adamw(master, grad, m, v, sh, float(lr), float(b1), float(b2), float(eps), float(eps_root), float(wd),
                        float(bc1), float(bc2), grad_scale)
    return
  g = grad.float() * grad_scale.float()
  mf = m.float().mul_(b1).add_(g, alpha=1 - b1)
  v.mul_(b2).addcmul_(g, g, value=1 - b2)
  m.copy_(mf)
  u = (mf / bc1) / (torch.sqrt(v / bc2 + eps_root) + eps)
  pf = master.float()
  pf.add_(u + wd * pf, alpha=-lr)
  master.copy_(pf)
  if shadow is not None and shadow.data_ptr() != master.data_ptr():
    shadow.copy_(master)
