"""Routed mixture-of-experts: router, dropless permutation, grouped expert FFN, expert parallelism.

Semantics follow src/maxtext/layers/moe.py: gate 247-392, top-k 717-765 (softmax over the selected
logits for Mixtral-style blocks; DeepSeek uses pre-scored values, optionally group-limited and
bias-corrected 775-838), dropless permutation 872-1002 (stable sort by expert id) and combine
1004-1063, load-balance loss 2662-2687, shared experts 3259-3371. Expert parallelism moves rows with
a variable-size all-to-all whose split sizes come from an exchanged count matrix (1202-1361);
`ops.moe_ops` provides the kernels (router top-k, counting-sort permutation, grouped GEMM).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..ops import functional as F
from ..ops import moe_ops
from .blocks import Builder, FusedParam, MLP, Norm, tp_enter, tp_exit


class _AllToAllRows(torch.autograd.Function):
  @staticmethod
  def forward(ctx, rows, send_sizes, recv_sizes, group):
    ctx.group, ctx.send, ctx.recv = group, send_sizes, recv_sizes
    out = rows.new_empty((sum(recv_sizes),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), recv_sizes, send_sizes, group=group)
    return out

  @staticmethod
  def backward(ctx, dy):
    dx = dy.new_empty((sum(ctx.send),) + tuple(dy.shape[1:]))
    dist.all_to_all_single(dx, dy.contiguous(), ctx.send, ctx.recv, group=ctx.group)
    return dx, None, None, None


class _AllGatherRows(torch.autograd.Function):
  """[t, ...] -> [ep * t, ...] (rank-major); the backward reduce-scatters."""

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    out = x.new_empty((dist.get_world_size(group) * x.shape[0],) + tuple(x.shape[1:]))
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out

  @staticmethod
  def backward(ctx, g):
    n = dist.get_world_size(ctx.group)
    out = g.new_empty((g.shape[0] // n,) + tuple(g.shape[1:]))
    dist.reduce_scatter_tensor(out, g.contiguous(), group=ctx.group)
    return out, None


class _ReduceScatterRows(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    n = dist.get_world_size(group)
    out = x.new_empty((x.shape[0] // n,) + tuple(x.shape[1:]))
    dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
    return out

  @staticmethod
  def backward(ctx, g):
    out = g.new_empty((dist.get_world_size(ctx.group) * g.shape[0],) + tuple(g.shape[1:]))
    dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
    return out, None


class _AllReduceMean(torch.autograd.Function):
  """Mean over a group of equally weighted partial means; every rank uses the result in an identical loss term, so the
  gradient of a rank's part is the mean of the ranks' output gradients."""
  @staticmethod
  def forward(ctx, x, group, n):
    ctx.group, ctx.n = group, n
    y = x.contiguous().clone()
    dist.all_reduce(y, group=group)
    return y / n

  @staticmethod
  def backward(ctx, dy):
    g = dy.contiguous().clone()
    dist.all_reduce(g, group=ctx.group)
    return g / ctx.n, None, None


class RoutedMoE:
  def __init__(self, b: Builder, config, name="MoeBlock_0", deepseek_style=False, style: str = "", hash_routing: bool = False):
    """style: "llama4" (raw top-k logits, sigmoid score applied to the expert input, unit combine weights;
    src/maxtext/layers/moe.py:752,902-906,1051-1053) or "gpt_oss" (router bias on the logits, per-expert biases and the
    clamped x * sigmoid(1.702 x) * (up + 1) activation; moe.py:617-637,841-853,2239-2242)."""
    c = config
    self.c = c
    self.style = style
    self.E, self.k = c.num_experts, c.num_experts_per_tok
    self.deepseek = deepseek_style
    mb = b.sub(name)
    d, f = c.emb_dim, c.moe_mlp_dim
    self.gate = mb.sub("gate").linear("kernel", (d,), (self.E,), ("embed", None))
    self.gate_bias = mb.sub("gate").vector("bias", self.E, (None,), init="zeros") if c.routed_bias else None
    self.wi_0 = mb.experts("wi_0", self.E, d, f, ("exp", "embed_moe", "mlp_moe"), tp="col")
    self.wi_1 = mb.experts("wi_1", self.E, d, f, ("exp", "embed_moe", "mlp_moe"), tp="col")
    self.wo = mb.experts("wo", self.E, f, d, ("exp", "mlp_moe", "embed_moe"), tp="row")
    self.act = c.mlp_activations[0]
    self.e_local = self.E // b.ep_size
    self.b0 = self.b1 = self.bo = None
    if c.mlp_bias:
      self.b0 = mb.table("wi_0_bias", (self.E, f), ("exp", "activation_mlp"), init="zeros")
      self.b1 = mb.table("wi_1_bias", (self.E, f), ("exp", "activation_mlp"), init="zeros")
      self.bo = mb.table("wo_bias", (self.E, d), ("exp", "activation_embed"), init="zeros")
    # gemma4 (src/maxtext/layers/moe.py:639-645,744-763): combine weights are the soft-max probabilities of the chosen experts,
    # renormalised, times a learned scale per expert
    self.per_expert_scale = mb.vector("per_expert_scale", self.E, ("exp",), init="ones") if style == "gemma4" else None
    # DeepSeek-V4 prefix layers (src/maxtext/layers/moe.py:442-455,729-739): experts are chosen by a fixed table indexed with the
    # TOKEN ID ([vocab, k], stored as floats in the checkpoint, never trained); the router only supplies the combine weights
    self.tid2eid = None
    if hash_routing:
      self.tid2eid = mb.table("tid2eid", (c.vocab_size, self.k), (None, None), init="zeros")
      self.tid2eid.pdef.frozen = True

  # ---- routing
  def route(self, x2, B, S, ctx=None, gate_inputs=None):
    c = self.c
    src = x2 if gate_inputs is None else gate_inputs
    xg = src.float() if c.float32_gate_logits else src
    w = self.gate.leaf()
    logits = torch.nn.functional.linear(xg, w.to(xg.dtype))
    if self.style == "gemma4":
      probs = torch.softmax(logits.float(), -1)
      idx = logits.topk(self.k, dim=-1).indices
      wts = probs.gather(-1, idx)
      if c.norm_topk_prob:
        wts = wts / wts.sum(-1, keepdim=True)
      wts = wts * self.per_expert_scale.leaf().float()[idx]
      return wts, idx, self._aux(probs, idx, B, S, ctx)
    grouped = self.deepseek and c.n_routing_groups > 0 and c.topk_routing_group > 0
    func = (c.routed_score_func or "softmax") if self.deepseek else "softmax"
    if (self.tid2eid is None and moe_ops.router_kernel_ok(logits, self.E, self.k) and not grouped and func in ("softmax", "sigmoid")
        and not bool(getattr(c, "use_random_routing", False))):
      # one launch: scores, top-k, routing weights (csrc/router_sm100.cu); the bias only steers the selection and is not trained
      bias = self.gate_bias.leaf() if self.gate_bias is not None else None
      if self.deepseek:
        idx, wts, probs, _ = moe_ops.router_topk(logits, bias, self.k, 1, func == "sigmoid", False, float(c.routed_scaling_factor))
      else:
        lg = logits + bias.to(logits.dtype) if bias is not None else logits      # here the bias is part of the logits (and trained)
        idx, wts, probs, _ = moe_ops.router_topk(lg, None, self.k, 0, False, self.style == "llama4", 1.0)
        if c.norm_topk_prob:
          wts = wts / wts.sum(-1, keepdim=True)
    elif self.deepseek:
      lf = logits.float()
      # src/maxtext/layers/linears.py:40-56: the gate's score function; DeepSeek-V4 uses sqrt(softplus(logit))
      scores = torch.softmax(lf, -1) if func == "softmax" else torch.sigmoid(lf) if func == "sigmoid" else \
          torch.sqrt(torch.nn.functional.softplus(lf)) if func == "sqrtsoftplus" else lf
      sel = scores + self.gate_bias.leaf().float() if self.gate_bias is not None else scores
      if self.tid2eid is not None:
        if ctx is None or ctx.tokens is None:
          raise ValueError("hash routing needs the token ids of the batch")
        sel = None
      if sel is not None and c.n_routing_groups > 0 and c.topk_routing_group > 0:
        G = c.n_routing_groups
        grp = sel.view(-1, G, self.E // G)
        gscore = grp.topk(2, dim=-1).values.sum(-1) if self.gate_bias is not None else grp.max(-1).values
        gidx = gscore.topk(c.topk_routing_group, dim=-1).indices
        gmask = torch.zeros_like(gscore).scatter_(1, gidx, 1.0).bool()
        sel = sel.masked_fill(~gmask[:, :, None].expand_as(grp).reshape(sel.shape), float("-inf"))
      if sel is None:
        idx = self.tid2eid.data.detach()[ctx.tokens.reshape(-1).long()].long().clamp_(0, self.E - 1)
      else:
        idx = sel.topk(self.k, dim=-1).indices
      wts = scores.gather(-1, idx)
      if func in ("sigmoid", "sqrtsoftplus"):
        wts = wts / (wts.sum(-1, keepdim=True) + 1e-20)
      wts = wts * c.routed_scaling_factor
      probs = scores
    else:
      if self.gate_bias is not None:
        logits = logits + self.gate_bias.leaf().to(logits.dtype)
      vals, idx = logits.topk(self.k, dim=-1)
      wts = vals.float() if self.style == "llama4" else torch.softmax(vals.float(), -1)
      if c.norm_topk_prob:
        wts = wts / wts.sum(-1, keepdim=True)
      probs = torch.softmax(logits.float(), -1)
    if bool(getattr(c, "use_random_routing", False)) and not self.deepseek:
      # debugging aid (src/maxtext/layers/moe.py `random_routing`): uniformly random experts, weights from their logits
      idx = torch.rand(logits.shape, device=logits.device).topk(self.k, dim=-1).indices
      vals = logits.gather(-1, idx)
      wts = vals.float() if self.style == "llama4" else torch.softmax(vals.float(), -1)
    cf = float(getattr(c, "capacity_factor", -1.0) or -1.0)
    if cf > 0:
      # token dropping (moe.py `generate_masks`): per sequence, assignments are counted per expert in (token, choice)
      # order and those beyond the expert's capacity get weight zero
      cap = int(max(math.ceil(S * self.k / self.E) * cf, cf))
      onehot_k = torch.nn.functional.one_hot(idx.view(B, S * self.k), self.E)                  # [B, S*k, E]
      rank_in_expert = (onehot_k.cumsum(1) * onehot_k).sum(-1)                                # 1-based arrival order
      wts = wts * (rank_in_expert <= cap).view(B * S, self.k).to(wts.dtype)
    return wts, idx, self._aux(probs, idx, B, S, ctx)

  def _aux(self, probs, idx, B, S, ctx):
    c = self.c
    aux = None
    if c.load_balance_loss_weight > 0:
      onehot = torch.zeros(B * S, self.E, dtype=torch.float32, device=probs.device).scatter_add_(
          1, idx, torch.ones_like(idx, dtype=torch.float32))
      density = onehot.view(B, S, self.E).mean(1)
      density_prob = probs.view(B, S, self.E).mean(1)
      if ctx is not None and ctx.cp_size > 1:
        # context parallelism: the two means run over the whole sequence, of which this rank holds a part
        cp_axes = ("context", "context_usp_ulysses")
        g = ctx.mesh.group(cp_axes) if ctx.mesh is not None else ctx.cp_group
        density = _AllReduceMean.apply(density, g, ctx.cp_size)
        density_prob = _AllReduceMean.apply(density_prob, g, ctx.cp_size)
      aux = (density * density_prob).mean() * (self.E ** 2) * c.load_balance_loss_weight
    return aux

  # ---- expert FFN on rows grouped by (local) expert
  def experts_ffn(self, rows, sizes):
    g = moe_ops.grouped_linear(rows, self.wi_0, sizes)
    u = moe_ops.grouped_linear(rows, self.wi_1, sizes)
    row_e = None
    if self.b0 is not None:
      row_e = torch.repeat_interleave(torch.arange(sizes.numel(), device=rows.device), sizes.long(), output_size=rows.shape[0])
      g = g + self.b0.leaf()[row_e].to(g.dtype)
      u = u + self.b1.leaf()[row_e].to(u.dtype)
    if self.style == "gpt_oss":
      lim = float(self.c.mlp_activations_limit)
      gf, uf = g.float().clamp(max=lim), u.float().clamp(-lim, lim)
      h = (gf * torch.sigmoid(1.702 * gf) * (uf + 1.0)).to(rows.dtype)
    else:
      h = F.gated_act(torch.cat([g, u], dim=-1), self.act)
    y = moe_ops.grouped_linear(h, self.wo, sizes)
    if self.bo is not None:
      y = y + self.bo.leaf()[row_e].to(y.dtype)
    return y

  def _ring_of_experts(self, x2, B, S, ctx):
    """`use_ring_of_experts` (src/maxtext/layers/moe.py:1700-1716): instead of moving routed rows, every expert shard
    receives ALL tokens (all-gather over the expert axis), routes them itself, runs only its own experts on the rows that
    chose them, and the partial outputs are reduce-scattered back. No variable-size exchange, at the price of gathering
    the activations."""
    ep, el = ctx.ep_size, self.e_local
    rank = dist.get_rank(ctx.ep_group)
    xg = _AllGatherRows.apply(x2, ctx.ep_group) if torch.is_grad_enabled() else _AllGatherRows.forward(F._Dummy(), x2, ctx.ep_group)
    wts, idx, aux = self.route(xg, B * ep, S)
    if aux is not None:
      ctx.aux_losses.append(("moe_lb_loss", aux))
    mine = (idx // el) == rank
    idx_l = torch.where(mine, idx - rank * el, torch.full_like(idx, el))      # group `el` collects the rows of other shards
    wts_l = torch.where(mine, wts, torch.zeros_like(wts))
    rows, order, sizes = moe_ops.permute(xg, idx_l, el + 1)
    n_mine = int(sizes[:el].sum().item())
    y_mine = self.experts_ffn(rows[:n_mine], sizes[:el])
    y = torch.cat([y_mine, y_mine.new_zeros(rows.shape[0] - n_mine, y_mine.shape[1])], 0)
    out = moe_ops.unpermute_combine(y, order, wts_l, xg.shape[0], self.k, fp32_sum=self.c.float32_weight_sum).to(x2.dtype)
    red = _ReduceScatterRows.apply(out, ctx.ep_group) if torch.is_grad_enabled() else _ReduceScatterRows.forward(F._Dummy(), out, ctx.ep_group)
    return red

  def __call__(self, x, ctx, gate_inputs=None):
    if ctx.sp and ctx.tp_size > 1:
      assert gate_inputs is None, "a separate router input is not implemented under tensor-sequence parallelism"
      # sequence-parallel residual stream: routing needs every token, so the block runs the plain tensor-parallel form on
      # the gathered sequence (which returns complete outputs and complete input gradients on every rank) and keeps its part
      from ..parallel import sequence_parallel as sp
      ctx.sp = False
      try:
        out = self(sp.gather_whole(x, ctx.tp_group), ctx)
      finally:
        ctx.sp = True
      return sp.slice_local(out, ctx.tp_group)
    B, S, D = x.shape
    x2 = x.reshape(B * S, D)
    if ctx.ep_size > 1 and self.c.use_ring_of_experts and self.style != "llama4":
      out = self._ring_of_experts(x2, B, S, ctx)
      if ctx.tp_size > 1:
        out = tp_exit(out, ctx)
      return out.view(B, S, D)
    wts, idx, aux = self.route(x2, B, S, ctx, gate_inputs.reshape(B * S, D) if gate_inputs is not None else None)
    if aux is not None:
      ctx.aux_losses.append(("moe_lb_loss", aux))
    if (self.gate_bias is not None and self.deepseek and self.c.routed_bias_update_rate > 0 and ctx.expert_counts is not None
        and ctx.mode == "train" and not ctx.recompute):
      cnt = torch.bincount(idx.reshape(-1), minlength=self.E).float()
      ctx.expert_counts[self] = ctx.expert_counts[self] + cnt if self in ctx.expert_counts else cnt
    if self.style == "llama4":
      assert self.k == 1, "llama4 routing scales the expert input by its single score"
      x2 = (x2.float() * torch.sigmoid(wts)).to(x2.dtype)
      wts = torch.ones_like(wts)
    if ctx.tp_size > 1:
      # the experts' hidden dim is split over the tensor ranks: what flows back into the tokens and into the combine weights
      # is a partial sum on every rank (the router itself runs replicated and stays outside). The fused paths combine before
      # the all-reduce of the output, the generic path after it, where the combine already sees complete expert outputs.
      x2, wts_fused = tp_enter(x2, ctx), tp_enter(wts, ctx)
    else:
      wts_fused = wts
    plain_ffn = self.b0 is None and self.style != "gpt_oss"
    if plain_ffn and ctx.ep_size == 1 and self.act in F._ACT_CODE and moe_ops.padded_path_supported(x2, D, self.wi_0.data.shape[1], self.E):
      # GPU path: device-side stable sort into 128-row-padded expert groups, grouped tcgen05 GEMMs, no host synchronisation
      out = moe_ops.moe_ffn_padded(x2, wts_fused, idx, self.wi_0, self.wi_1, self.wo, self.E, self.act)
      if ctx.tp_size > 1:
        out = tp_exit(out, ctx)
      return out.view(B, S, D)
    if plain_ffn and ctx.ep_size > 1 and x2.is_cuda:
      from . import moe_ep
      if moe_ep.supported(x2, self, ctx):
        # dispatch / return through the peers' symmetric buffers (this repository's kernels); the NCCL path below is the fallback
        out = moe_ep.expert_parallel_ffn(x2, wts_fused, idx, self, ctx)
        if ctx.tp_size > 1:
          out = tp_exit(out, ctx)
        return out.view(B, S, D)
    rows, order, sizes = moe_ops.permute(x2, idx, self.E)          # rows sorted by global expert id
    y = self._expert_parallel(rows, sizes, ctx) if ctx.ep_size > 1 else self.experts_ffn(rows, sizes)
    if ctx.tp_size > 1:
      y = tp_exit(y, ctx)           # the experts' hidden dim is split over the tensor ranks: sum the partial outputs
    out = moe_ops.unpermute_combine(y, order, wts, B * S, self.k, fp32_sum=self.c.float32_weight_sum)
    return out.view(B, S, D).to(x.dtype)

  def _expert_parallel(self, rows, sizes, ctx):
    """NCCL reference path: counts exchange -> a2a dispatch -> local regroup -> FFN -> reverse."""
    ep, el = ctx.ep_size, self.e_local
    counts = sizes.view(ep, el)                                  # rows this rank sends to (dest rank, its expert)
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts.contiguous(), group=ctx.ep_group)   # [src rank, my expert]
    send_sizes = counts.sum(1).tolist()
    recv_sizes = recv_counts.sum(1).tolist()
    recv = _AllToAllRows.apply(rows, send_sizes, recv_sizes, ctx.ep_group)         # grouped by src rank, then expert
    # regroup by local expert
    src_expert = torch.repeat_interleave(torch.arange(el, device=rows.device).repeat(ep), recv_counts.reshape(-1))
    local_order = torch.argsort(src_expert, stable=True)
    local_sizes = recv_counts.sum(0)
    grouped = recv[local_order]
    y = self.experts_ffn(grouped, local_sizes)
    inv = torch.empty_like(local_order)
    inv[local_order] = torch.arange(local_order.numel(), device=rows.device)
    y = y[inv]
    return _AllToAllRows.apply(y, recv_sizes, send_sizes, ctx.ep_group)


class Gemma4MoE:
  """Feed-forward block of the Gemma-4 MoE models (src/maxtext/models/gemma4.py:57-147): the dense MLP ("shared expert", width
  mlp_dim) reads the pre-normed input; the routed experts read their own RMS norm of the un-normed residual stream; the router
  reads a scale-free RMS norm of it times emb_dim^-1/2 times a learned per-channel scale; each branch has its own output norm."""

  def __init__(self, b: Builder, config, name="mlp"):
    c = config
    mb = b.sub(name)
    eps = c.normalization_layer_epsilon
    self.routed = RoutedMoE(mb.sub("moe_block"), c, "MoeBlock_0", deepseek_style=False, style="gemma4")
    self.shared = MLP(mb.sub("moe_block"), c, "shared_experts", hidden=max(1, int(c.shared_experts)) * c.mlp_dim)
    self.router_scale = mb.vector("pre_forward_scale_2", c.emb_dim, ("embed",), init="ones")
    self.pre2 = Norm(mb, "pre_feedforward_layernorm_2", c.emb_dim, eps)
    self.post1 = Norm(mb, "post_feedforward_layernorm_1", c.emb_dim, eps)
    self.post2 = Norm(mb, "post_feedforward_layernorm_2", c.emb_dim, eps)
    self.eps, self.root = eps, c.emb_dim ** -0.5

  def __call__(self, x, ctx, original):
    shared = self.post1(self.shared(x, ctx))
    of = original.float()
    gate_in = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + self.eps) * self.root * self.router_scale.leaf().float()
    routed = self.post2(self.routed(self.pre2(original), ctx, gate_inputs=gate_in if self.routed.c.float32_gate_logits else gate_in.to(x.dtype)))
    return routed + shared


class RoutedAndSharedMoE:
  """Routed experts plus always-on shared experts (src/maxtext/layers/moe.py:3259-3371)."""

  def __init__(self, b: Builder, config, name="DeepSeekMoeBlock_0", style: str = "", hash_routing: bool = False):
    mb = b.sub(name)
    self.shared_gate = None
    if style == "qwen3_next":
      # src/maxtext/models/qwen3.py:1107-1193: softmax top-k router, one shared expert whose output is scaled per token by
      # sigmoid(x . w_gate)
      self.routed = RoutedMoE(mb, config, "routed_experts", deepseek_style=False, style="")
      self.shared = MLP(mb, config, "shared_expert", hidden=config.moe_mlp_dim)
      self.shared_gate = mb.sub("shared_expert_gate").linear("kernel", (config.emb_dim,), (1,), ("embed", None))
      return
    self.routed = RoutedMoE(mb, config, "MoeBlock_0", deepseek_style=(style == ""), style=style, hash_routing=hash_routing)
    self.shared = MLP(mb, config, "shared_experts", hidden=config.shared_experts * config.moe_mlp_dim) \
        if config.shared_experts > 0 else None

  def __call__(self, x, ctx):
    y = self.routed(x, ctx)
    if self.shared is not None:
      sh = self.shared(x, ctx)
      if self.shared_gate is not None:
        gate = torch.nn.functional.linear(x.float(), self.shared_gate.leaf().float())
        sh = (sh.float() * torch.sigmoid(gate)).to(sh.dtype)
      y = y + sh
    return y
