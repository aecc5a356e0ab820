"""Expert parallelism over NVLink peer memory: dispatch rows to the ranks that own their experts, run the grouped expert FFN
there, bring the results back -- all with this repository's kernels writing to / reading from the peers' symmetric buffers.

Replaces the variable-size all-to-all of the reference (ragged_all_to_all, src/maxtext/layers/moe.py:1202-1361) and the
host round trip for split sizes that an NCCL all_to_all_single needs: counts travel as a tiny put, every index is derived
on the device (csrc/moe_ep_sm100.cu), and the only cross-rank synchronisation is four epoch flags per exchange.

Buffer discipline (one pair of symmetric buffers per EP group, shared by all layers):
  A (inbound rows): written by peers' push kernels between flag 2 of one exchange and the next; the owner clones it before
    it signals flag 3, and no peer can start the next push before it has seen that flag.
  B (outbound rows): written by the owner before flag 3, read by peers' pull kernels before they signal flag 4; the owner
    does not touch it again until it has seen flag 4 from everyone.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import backend, moe_ops
from ..ops import functional as F
from ..parallel import symm as symm_lib

_RUNTIMES: dict = {}


class _RecvPlan:
  """Layout of the rows this rank received (what the grouped GEMM needs) plus where this rank's own pairs went."""

  def __init__(self, rt, n):
    i32 = dict(dtype=torch.int32, device=rt.device)
    self.rows_max = rt.cap
    self.offs = torch.empty(rt.el + 1, **i32)
    self.blk_expert = torch.empty(rt.cap // 128, **i32)
    self.valid = torch.empty(rt.el, **i32)
    self.send_base = torch.empty(rt.E, **i32)
    self.pair_owner = torch.empty(n, **i32)
    self.pair_row = torch.empty(n, **i32)


class _IdentityPlan:
  """Plan-shaped view of rows that already sit in pair order (row j = pair j)."""

  def __init__(self, T, k, device):
    n = T * k
    self.T, self.k, self.n, self.rows_max = T, k, n, n
    self.dest = torch.arange(n, dtype=torch.int32, device=device)
    self.row_pair = self.dest
    self.offs = torch.tensor([0, n], dtype=torch.int32, device=device)


class EPRuntime:
  def __init__(self, group, device, num_experts: int, d_model: int, pairs: int, factor: float):
    self.symm = symm_lib.SymmGroup(group, device)
    self.group, self.device = group, device
    self.ep, self.rank = self.symm.world, self.symm.rank
    self.E, self.el, self.D = num_experts, num_experts // self.ep, d_model
    worst = self.ep * pairs
    want = min(worst, int(factor * pairs + 0.5)) + self.el * 127
    self.cap = -(-want // 128) * 128
    self.counts = self.symm.alloc(self.ep * self.E, torch.int32, zero=True)
    self.buf_a = self.symm.alloc(self.cap * d_model, torch.bfloat16)
    self.buf_b = self.symm.alloc(self.cap * d_model, torch.bfloat16)
    self.a2d = self.buf_a.tensor.view(self.cap, d_model)
    self.b2d = self.buf_b.tensor.view(self.cap, d_model)
    dist.barrier(group=group)

  # ---- the two directions
  def push_rows(self, src, src_div, lp, rp, idx32):
    """Pair rows -> owners' buffer A; returns a private copy of what this rank received (padding rows zeroed)."""
    E_ = backend.ext()
    E_.ep_push(src, src_div, idx32, lp.dest, lp.offs, rp.send_base, self.el, self.cap, self.buf_a.table, rp.pair_owner, rp.pair_row)
    self.symm.signal(2)
    self.symm.wait(2)
    E_.ep_zero_pads(self.a2d, rp.offs, rp.valid)
    return self.a2d.clone()

  def pull_rows(self, rows, rp, n):
    """Owner-side rows -> buffer B -> every rank pulls the rows of its own pairs (pair order)."""
    E_ = backend.ext()
    self.b2d.copy_(rows)
    self.symm.signal(3)
    self.symm.wait(3)
    out = torch.empty(n, self.D, dtype=torch.bfloat16, device=self.device)
    E_.ep_pull(self.buf_b.table, rp.pair_owner, rp.pair_row, self.cap, out)
    self.symm.signal(4)
    self.symm.wait(4)
    return out


def runtime(group, device, num_experts, d_model, pairs, factor, slot: int = 0) -> EPRuntime:
  """`slot` separates exchanges that may be in flight at the same time (the micro-batches of the batch-split schedule run
  on different streams): each slot owns its buffers and its epoch flags."""
  key = (id(group), num_experts, d_model, pairs, slot)
  if key not in _RUNTIMES:
    _RUNTIMES[key] = EPRuntime(group, device, num_experts, d_model, pairs, factor)
  return _RUNTIMES[key]


class _DispatchFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x2, rt, lp, rp, idx32):
    E_ = backend.ext()
    E_.ep_put_counts(lp.sizes, rt.rank, rt.counts.table)
    rt.symm.signal(1)
    rt.symm.wait(1)
    E_.ep_index(rt.counts.tensor, rt.ep, rt.rank, rp.offs, rp.blk_expert, rp.valid, rp.send_base)
    ctx.misc = (rt, lp, rp)
    return rt.push_rows(x2.contiguous(), lp.k, lp, rp, idx32)

  @staticmethod
  def backward(ctx, drows):
    rt, lp, rp = ctx.misc
    d_pairs = rt.pull_rows(drows, rp, lp.n)
    dx = torch.empty(lp.T, rt.D, dtype=drows.dtype, device=drows.device)
    backend.ext().moe_combine(d_pairs, _ident(lp).dest, None, lp.k, dx)
    return dx, None, None, None, None


class _ReturnFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, y, rt, lp, rp, idx32):
    ctx.misc = (rt, lp, rp, idx32)
    return rt.pull_rows(y, rp, lp.n)

  @staticmethod
  def backward(ctx, dy_pairs):
    rt, lp, rp, idx32 = ctx.misc
    return rt.push_rows(dy_pairs.contiguous(), 1, lp, rp, idx32), None, None, None, None


def _ident(lp):
  if getattr(lp, "_ident", None) is None:
    lp._ident = _IdentityPlan(lp.T, lp.k, lp.dest.device)
  return lp._ident


def supported(x2, moe, ctx) -> bool:
  c = moe.c
  if getattr(ctx, "split_active", False) and os.environ.get("MAXTEXT_B200_SPLIT_FUSED_EP") != "1":
    # two micro-batches of a split layer exchange at the same time on two streams. Each slot has its own buffers and flags
    # (`runtime(slot=)`), but that combination has not run on GPUs yet: the exchange goes through the NCCL path, whose calls
    # are issued in the same order on every rank
    return False
  return (bool(getattr(c, "use_fused_comm_kernels", False)) and x2.dtype == torch.bfloat16 and moe.act in F._ACT_CODE
          and moe_ops.padded_path_supported(x2, x2.shape[1], moe.wi_0.data.shape[1], moe.E) and symm_lib.available())


def expert_parallel_ffn(x2, wts, idx, moe, ctx):
  """x2 [T, D] -> [T, D]: routed experts spread over the `expert` mesh axis."""
  T, k = idx.shape
  rt = runtime(ctx.ep_group, x2.device, moe.E, x2.shape[1], T * k, float(getattr(moe.c, "ep_buffer_factor", 2.0)), int(ctx.micro_slot) % 2)
  lp = moe_ops.GroupPlan(idx, moe.E)                 # this rank's pairs sorted by GLOBAL expert
  rp = _RecvPlan(rt, T * k)
  idx32 = idx.reshape(-1).to(torch.int32).contiguous()
  grad = torch.is_grad_enabled()
  D_ = F._Dummy()
  w0, w1, wo = moe.wi_0.data, moe.wi_1.data, moe.wo.data
  if grad:
    rows = _DispatchFn.apply(x2, rt, lp, rp, idx32)
    y = moe_ops._ExpertsFFNFn.apply(rows, w0, w1, wo, moe.wi_0, moe.wi_1, moe.wo, rp, moe.act)
    y_pairs = _ReturnFn.apply(y, rt, lp, rp, idx32)
    return moe_ops._CombineFn.apply(y_pairs, wts, _ident(lp))
  rows = _DispatchFn.forward(D_, x2, rt, lp, rp, idx32)
  y = moe_ops._ExpertsFFNFn.forward(D_, rows, w0, w1, wo, None, None, None, rp, moe.act)
  y_pairs = _ReturnFn.forward(D_, y, rt, lp, rp, idx32)
  return moe_ops._CombineFn.forward(D_, y_pairs, wts, _ident(lp))
