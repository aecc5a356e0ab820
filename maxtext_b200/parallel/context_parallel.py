"""Context parallelism: the sequence is split over the `context` (and `context_usp_ulysses`) mesh axes.

Strategies (context_parallel_strategy, src/maxtext/configs/types.py:4004-4147; src/maxtext/layers/attention_op.py:1389-1546):
  all_gather : keys/values are all-gathered along the sequence, every rank attends its own queries to all keys.
  ulysses    : all-to-all swaps the split from sequence to heads; each rank runs ordinary full-sequence attention on
               heads/cp heads -- on an NVSwitch node this is the cheapest form (the square causal flash kernel is used
               unchanged and every GPU talks to every peer at full bandwidth).
  ring       : key/value blocks travel around the ring, partial results are merged with their log-sum-exp; the backward
               pass sends the blocks round again together with their gradient accumulators.
  usp        : ulysses inside the `context_usp_ulysses` group, ring across the `context` group.
Load balancing (context_parallel_load_balance, src/maxtext/utils/max_utils.py reorder_sequence / train_utils.py:305-331):
the sequence is cut into 2*cp chunks and rank r holds chunks r and 2*cp-1-r, so causal work is even. Masks are always
computed from the original token positions, which travel with the data, so any order is legal.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


# --------------------------------------------------------------------------------------------- sequence layout
def balanced_order(cp: int) -> list[int]:
  """Chunk ids (of 2*cp) in the order the ranks hold them: [0, 2cp-1, 1, 2cp-2, ...]."""
  out = []
  for r in range(cp):
    out += [r, 2 * cp - 1 - r]
  return out


def reorder_sequence(x: torch.Tensor, cp: int, dim: int = 1, to_contiguous: bool = False) -> torch.Tensor:
  """Natural order -> load-balanced order (or back with to_contiguous=True) along `dim`."""
  n = x.shape[dim]
  assert n % (2 * cp) == 0, f"sequence {n} must divide by 2*cp={2 * cp}"
  chunks = x.split(n // (2 * cp), dim=dim)
  order = balanced_order(cp)
  if to_contiguous:
    inv = [0] * len(order)
    for i, c in enumerate(order):
      inv[c] = i
    order = inv
  return torch.cat([chunks[c] for c in order], dim=dim)


def shard_sequence(x: torch.Tensor, rank: int, cp: int, load_balance: bool, dim: int = 1) -> torch.Tensor:
  """This rank's slice of a [B, S, ...] tensor."""
  if cp == 1:
    return x
  if load_balance:
    x = reorder_sequence(x, cp, dim)
  n = x.shape[dim] // cp
  return x.narrow(dim, rank * n, n).contiguous()


def shard_batch(batch: dict, rank: int, cp: int, load_balance: bool) -> dict:
  """Sequence-slice every [B, S] entry; positions are materialised first so that they keep the original indices."""
  if cp == 1:
    return batch
  out = dict(batch)
  B, S = batch["inputs"].shape
  if out.get("inputs_position") is None:
    out["inputs_position"] = torch.arange(S, dtype=torch.int32, device=batch["inputs"].device)[None].expand(B, S)
  for k, v in out.items():
    if torch.is_tensor(v) and v.dim() >= 2 and v.shape[1] == S:
      out[k] = shard_sequence(v, rank, cp, load_balance)
  return out


# --------------------------------------------------------------------------------------------- differentiable collectives
class _AllGatherSeq(torch.autograd.Function):
  """[B, s, ...] -> [B, cp*s, ...] (rank-major); backward reduce-scatters the gradient."""

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    cp = dist.get_world_size(group)
    parts = [torch.empty_like(x) for _ in range(cp)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=1)

  @staticmethod
  def backward(ctx, g):
    cp = dist.get_world_size(ctx.group)
    parts = [p.contiguous() for p in g.chunk(cp, dim=1)]
    out = torch.empty_like(parts[0])
    dist.reduce_scatter(out, parts, group=ctx.group)
    return out, None


def all_gather_seq(x, group):
  if x.requires_grad and torch.is_grad_enabled():
    return _AllGatherSeq.apply(x, group)
  cp = dist.get_world_size(group)
  parts = [torch.empty_like(x) for _ in range(cp)]
  dist.all_gather(parts, x.contiguous(), group=group)
  return torch.cat(parts, dim=1)


def _a2a(x, group, split_dim, cat_dim):
  cp = dist.get_world_size(group)
  send = torch.stack(x.chunk(cp, dim=split_dim))          # [cp, ...]: slab i goes to rank i
  recv = torch.empty_like(send)
  dist.all_to_all_single(recv, send, group=group)
  return torch.cat(list(recv.unbind(0)), dim=cat_dim)


class _SeqToHeads(torch.autograd.Function):
  """[B, s, H, D] (sequence split) -> [B, cp*s, H/cp, D] (head split); the backward is the inverse exchange."""

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return _a2a(x, group, 2, 1)

  @staticmethod
  def backward(ctx, g):
    return _a2a(g, ctx.group, 1, 2), None


class _HeadsToSeq(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return _a2a(x, group, 1, 2)

  @staticmethod
  def backward(ctx, g):
    return _a2a(g, ctx.group, 2, 1), None


def seq_to_heads(x, group):
  return _SeqToHeads.apply(x, group) if (x.requires_grad and torch.is_grad_enabled()) else _a2a(x, group, 2, 1)


def heads_to_seq(x, group):
  return _HeadsToSeq.apply(x, group) if (x.requires_grad and torch.is_grad_enabled()) else _a2a(x, group, 1, 2)


def _gather_ints(x, group):
  if x is None:
    return None
  cp = dist.get_world_size(group)
  parts = [torch.empty_like(x) for _ in range(cp)]
  dist.all_gather(parts, x.contiguous(), group=group)
  return torch.cat(parts, dim=1)


# --------------------------------------------------------------------------------------------- strategies
def _attn(q, k, v, pos, seg, kw, kpos=None, kseg=None):
  from ..ops import functional as F
  return F.attention(q, k, v, pos, seg, kw.get("scale", 1.0), kw.get("soft_cap", 0.0), kw.get("window", 0), True, kpos, kseg)


def attend_all_gather(q, k, v, pos, seg, group, **kw):
  kf, vf = all_gather_seq(k, group), all_gather_seq(v, group)
  return _attn(q, kf, vf, pos, seg, kw, _gather_ints(pos, group), _gather_ints(seg, group))


def _expand_kv_heads(k, v, hq: int, cp: int):
  """Repeat key/value heads until they divide by cp (grouped-query models with fewer kv heads than ranks)."""
  hkv = k.shape[2]
  if hkv % cp == 0:
    return k, v
  import math
  r = cp // math.gcd(hkv, cp)
  assert hq % (hkv * r) == 0, f"cannot split {hq} query / {hkv} kv heads over {cp} ranks"
  return k.repeat_interleave(r, dim=2), v.repeat_interleave(r, dim=2)


def attend_ulysses(q, k, v, pos, seg, group, load_balance=True, inner=None, **kw):
  """`inner(q, k, v, pos, seg)` replaces the local attention (usp runs ring attention there)."""
  cp = dist.get_world_size(group)
  k, v = _expand_kv_heads(k, v, q.shape[2], cp)
  qf, kf, vf = seq_to_heads(q, group), seq_to_heads(k, group), seq_to_heads(v, group)
  pf, sf = _gather_ints(pos, group), _gather_ints(seg, group)
  natural = load_balance and inner is None
  if natural:        # the square causal kernel masks by index: restore the original token order
    qf, kf, vf = (reorder_sequence(t, cp, 1, True) for t in (qf, kf, vf))
    pf = reorder_sequence(pf, cp, 1, True)
    sf = reorder_sequence(sf, cp, 1, True) if sf is not None else None
  out = inner(qf, kf, vf, pf, sf) if inner is not None else _attn(qf, kf, vf, pf, sf, kw)
  if natural:
    out = reorder_sequence(out, cp, 1)
  return heads_to_seq(out, group)


def _merge(out, lse, o_i, lse_i):
  """Combine two partial softmax results over disjoint key sets. out [B,S,H,D], lse [B,H,S]."""
  if out is None:
    return o_i.float(), lse_i
  tot = torch.logaddexp(lse, lse_i)
  wa = torch.exp(lse - tot).transpose(1, 2).unsqueeze(-1)
  wb = torch.exp(lse_i - tot).transpose(1, 2).unsqueeze(-1)
  return out * wa + o_i.float() * wb, tot


def _ring_exchange(tensors, group):
  """Send every tensor to the next rank of the ring and receive the previous rank's; returns the received list."""
  cp, r = dist.get_world_size(group), dist.get_rank(group)
  nxt, prv = dist.get_global_rank(group, (r + 1) % cp), dist.get_global_rank(group, (r - 1) % cp)
  recv = [torch.empty_like(t) for t in tensors]
  ops = []
  for t, b in zip(tensors, recv):
    ops.append(dist.P2POp(dist.isend, t.contiguous(), nxt, group))
    ops.append(dist.P2POp(dist.irecv, b, prv, group))
  return recv, dist.batch_isend_irecv(ops)


class _RingAttention(torch.autograd.Function):
  @staticmethod
  def forward(ctx, q, k, v, pos, seg, group, scale, soft_cap, window):
    from ..ops import functional as F
    cp = dist.get_world_size(group)
    has_seg = seg is not None
    blk = [k.contiguous(), v.contiguous(), pos.contiguous()] + ([seg.contiguous()] if has_seg else [])
    out = lse = None
    for step in range(cp):
      nxt_blk, reqs = _ring_exchange(blk, group) if step < cp - 1 else (None, [])     # overlaps the attention below
      o_i, l_i = F.attention_fwd(q, blk[0], blk[1], pos, seg, scale, soft_cap, window, True, blk[2], blk[3] if has_seg else None)
      out, lse = _merge(out, lse, o_i, l_i)
      for w in reqs:
        w.wait()
      if nxt_blk is not None:
        blk = nxt_blk
    out = out.to(q.dtype)
    ctx.save_for_backward(q, k, v, out, lse, pos, seg)
    ctx.cfg = (group, scale, soft_cap, window)
    return out

  @staticmethod
  def backward(ctx, dout):
    from ..ops import functional as F
    q, k, v, out, lse, pos, seg = ctx.saved_tensors
    group, scale, soft_cap, window = ctx.cfg
    cp = dist.get_world_size(group)
    has_seg = seg is not None
    dout = dout.contiguous()
    dq = torch.zeros_like(q, dtype=torch.float32)
    # the block and its gradient accumulators travel together; after cp hops they are home again
    blk = [k.contiguous(), v.contiguous(), pos.contiguous()] + ([seg.contiguous()] if has_seg else [])
    dk_acc = torch.zeros_like(k, dtype=torch.float32)
    dv_acc = torch.zeros_like(v, dtype=torch.float32)
    for step in range(cp):
      dq_i, dk_i, dv_i = torch.empty_like(q), torch.empty_like(blk[0]), torch.empty_like(blk[1])
      F.attention_bwd(dout, q, blk[0], blk[1], out, lse, pos, seg, scale, soft_cap, window, dq_i, dk_i, dv_i, True,
                      blk[2], blk[3] if has_seg else None)
      dq += dq_i.float()
      dk_acc += dk_i.float()
      dv_acc += dv_i.float()
      moved, reqs = _ring_exchange(blk + [dk_acc, dv_acc], group)
      for w in reqs:
        w.wait()
      blk, dk_acc, dv_acc = moved[:-2], moved[-2], moved[-1]
    return dq.to(q.dtype), dk_acc.to(k.dtype), dv_acc.to(v.dtype), None, None, None, None, None, None


def attend_ring(q, k, v, pos, seg, group, **kw):
  return _RingAttention.apply(q, k, v, pos, seg, group, kw.get("scale", 1.0), kw.get("soft_cap", 0.0), kw.get("window", 0))


def context_attention(q, k, v, pos, seg, ctx, scale=1.0, soft_cap=0.0, window=0):
  """Dispatch on config.context_parallel_strategy; `ctx` is the LayerCtx (cp_group, usp_group, config)."""
  c = ctx.config
  kw = dict(scale=scale, soft_cap=soft_cap, window=window)
  strat = c.context_parallel_strategy
  lb = bool(c.context_parallel_load_balance)
  if strat == "all_gather":
    return attend_all_gather(q, k, v, pos, seg, ctx.cp_group, **kw)
  if strat == "ulysses":
    return attend_ulysses(q, k, v, pos, seg, ctx.cp_group, load_balance=lb, **kw)
  if strat == "ring":
    return attend_ring(q, k, v, pos, seg, ctx.cp_group, **kw)
  if strat == "usp":
    ring_g, uly_g = ctx.cp_group, ctx.usp_group
    if uly_g is None:
      return attend_ring(q, k, v, pos, seg, ring_g, **kw)
    inner = (lambda a, b, d, p, s: attend_ring(a, b, d, p, s, ring_g, **kw)) if ring_g is not None else None
    return attend_ulysses(q, k, v, pos, seg, uly_g, load_balance=False if inner else lb, inner=inner, **kw)
  raise ValueError(f"unknown context_parallel_strategy {strat}")
