"""Tensor-sequence parallelism (Megatron "sequence parallel"; the reference's `tensor_sequence` mesh axis,
src/maxtext/configs/base.yml:580,597: `activation_norm_length` -> `tensor_sequence`).

With plain tensor parallelism the residual stream, the norms and the checkpoints kept for recomputation are replicated
on every tensor rank. Here they are split along the sequence instead: a block gathers its normalised input over the
tensor ranks right before the column-parallel projections and reduce-scatters the row-parallel output, so the two
all-reduces of a block become an all-gather plus a reduce-scatter (the same bytes) while everything between blocks is
1 / tp of the size. All tensors are [B, S, ...] and are split along dim 1 in rank order.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _ag(x, group):
  x = x.contiguous()
  n = dist.get_world_size(group)
  if n == 1:
    return x
  out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
  dist.all_gather_into_tensor(out, x, group=group)          # rank-major along dim 0
  return torch.cat(list(out.view((n,) + tuple(x.shape)).unbind(0)), dim=1)


def _rs(x, group):
  n = dist.get_world_size(group)
  if n == 1:
    return x
  parts = torch.cat([c.contiguous() for c in x.chunk(n, dim=1)], dim=0)      # rank-major along dim 0
  out = torch.empty((x.shape[0], x.shape[1] // n) + tuple(x.shape[2:]), dtype=x.dtype, device=x.device)
  dist.reduce_scatter_tensor(out, parts, group=group)
  return out


def _local(x, group):
  n, r = dist.get_world_size(group), dist.get_rank(group)
  return x.chunk(n, dim=1)[r].contiguous()


class _GatherSeq(torch.autograd.Function):
  """all-gather forward; the consumers produce partial input gradients, so backward reduce-scatters them."""
  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return _ag(x, group)

  @staticmethod
  def backward(ctx, dy):
    return _rs(dy, ctx.group), None


class _ReduceScatterSeq(torch.autograd.Function):
  """reduce-scatter forward (sum of the ranks' partial outputs, each keeps its part of the sequence); all-gather backward."""
  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return _rs(x, group)

  @staticmethod
  def backward(ctx, dy):
    return _ag(dy, ctx.group), None


class _SliceSeq(torch.autograd.Function):
  """keep this rank's part of a tensor that every rank holds whole; every rank needs the whole gradient back."""
  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return _local(x, group)

  @staticmethod
  def backward(ctx, dy):
    return _ag(dy, ctx.group), None


class _GatherSeqWhole(torch.autograd.Function):
  """all-gather forward for consumers that hand back the whole, already summed input gradient on every rank: backward
  keeps this rank's part."""
  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return _ag(x, group)

  @staticmethod
  def backward(ctx, dy):
    return _local(dy, ctx.group), None


def gather(x, group):
  return _GatherSeq.apply(x, group) if torch.is_grad_enabled() else _ag(x, group)


def reduce_scatter(x, group):
  return _ReduceScatterSeq.apply(x, group) if torch.is_grad_enabled() else _rs(x, group)


def slice_local(x, group):
  return _SliceSeq.apply(x, group) if torch.is_grad_enabled() else _local(x, group)


def gather_whole(x, group):
  return _GatherSeqWhole.apply(x, group) if torch.is_grad_enabled() else _ag(x, group)


# plain (non-differentiable) forms used by the engine at the ends of the layer stack
all_gather_seq = _ag
local_seq = _local
