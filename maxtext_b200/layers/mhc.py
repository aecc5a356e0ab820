"""Manifold-constrained hyper-connections (src/maxtext/layers/mhc.py:78-365) and the stream-collapsing head of DeepSeek-V4
(src/maxtext/layers/mhc.py:368-436).

With `mhc_expansion_rate = k > 1` the residual stream carries k copies of the model width, [B, S, k, D]. Around every
branch (attention or feed-forward) one RMS-normalised read of the flattened stream produces three small maps per token:

  pre  [k]     sigmoid gate that mixes the k streams into the branch input
  post [k]     2 * sigmoid gate that writes the branch output back into each stream
  res  [k, k]  doubly-stochastic matrix that mixes the streams among themselves: Sinkhorn iterations on a softmax, or
               (`enable_mhc_lite`) a softmax-weighted sum of the k! permutation matrices

All three come from ONE product of the normalised stream with the concatenated [pre | post | res] matrix; the rest is
per-token arithmetic on k or k*k numbers, done in fp32.
"""
from __future__ import annotations

import itertools
import math

import torch

from ..ops import functional as F
from . import blocks as L


def permutation_matrices(k: int, device=None) -> torch.Tensor:
  """All k! permutation matrices, [k!, k, k], in lexicographic order of the permutations."""
  perms = torch.tensor(list(itertools.permutations(range(k))), dtype=torch.long, device=device)
  return torch.eye(k, device=device)[perms]


def sinkhorn(t: torch.Tensor, iters: int = 20) -> torch.Tensor:
  """Rows and columns of softmax(t) alternately normalised to sum to one (fp32)."""
  eps = 1e-6
  t = torch.softmax(t.float(), dim=-1) + eps
  t = t / (t.sum(-2, keepdim=True) + eps)
  for _ in range(iters - 1):
    t = t / (t.sum(-1, keepdim=True) + eps)
    t = t / (t.sum(-2, keepdim=True) + eps)
  return t


def expand_streams(x: torch.Tensor, k: int) -> torch.Tensor:
  """[B, S, D] -> [B, S, k, D]: every stream starts as a copy of the embedding."""
  return x.unsqueeze(2).expand(-1, -1, k, -1).contiguous()


def reduce_streams(x: torch.Tensor) -> torch.Tensor:
  """[B, S, k, D] -> [B, S, D]: plain sum over the streams."""
  return x.sum(2, dtype=x.dtype)


class HyperConnection:
  """The wrapper of one branch. Parameter names and shapes follow the reference module (norm over k*D, three scalar scales
  initialised to 0.01, [k*D, k] / [k*D, k*k or k!] matrices, zero biases)."""

  def __init__(self, b: L.Builder, config, name: str, dim: int):
    c = config
    self.k = int(c.mhc_expansion_rate)
    self.dim = dim
    self.lite = bool(c.enable_mhc_lite)
    self.iters = int(c.sinkhorn_iterations)
    k = self.k
    sb = b.sub(name)
    self.norm = L.Norm(sb, "mhc_norm", k * dim, c.normalization_layer_epsilon)
    scalar = lambda n: sb._add(n, shape=(1,), ref_shape=(1,), logical_axes=(None,), kind="same", init="const", init_scale=0.01)  # noqa: E731
    self.res_alpha_scale, self.pre_alpha_scale, self.post_alpha_scale = scalar("res_alpha_scale"), scalar("pre_alpha_scale"), scalar("post_alpha_scale")
    n_res = math.factorial(k) if self.lite else k * k
    ax = ("activation_embed", None)
    self.res_alpha = sb.linear("res_alpha", (k * dim,), (n_res,), ax, init="fan_in_normal")
    self.pre_alpha = sb.linear("pre_alpha", (k * dim,), (k,), ax, init="fan_in_normal")
    self.post_alpha = sb.linear("post_alpha", (k * dim,), (k,), ax, init="fan_in_normal")
    res_shape = (n_res,) if self.lite else (k, k)
    self.res_beta = sb._add("res_beta", shape=res_shape, ref_shape=res_shape, logical_axes=(None,) * len(res_shape), kind="same", init="zeros")
    self.pre_beta = sb.vector("pre_beta", k, axes=(None,), init="zeros")
    self.post_beta = sb.vector("post_beta", k, axes=(None,), init="zeros")
    self._perms = None

  def maps(self, x: torch.Tensor):
    """x [B, S, k, D] -> (pre [B,S,k], post [B,S,k], res [B,S,k,k]) in fp32."""
    B, S, k, D = x.shape
    nx = self.norm(x.reshape(B, S, k * D))
    # the three projections read the same normalised stream: one product against [pre | post | res]
    w = torch.cat([self.pre_alpha.leaf(), self.post_alpha.leaf(), self.res_alpha.leaf()], 0)          # [k + k + n_res, k*D]
    h = torch.matmul(nx, w.t().to(nx.dtype)).float()
    h_pre, h_post, h_res = h[..., :k], h[..., k:2 * k], h[..., 2 * k:]
    pre = torch.sigmoid(self.pre_alpha_scale.leaf().float() * h_pre + self.pre_beta.leaf().float()) + 1e-6
    post = 2.0 * torch.sigmoid(self.post_alpha_scale.leaf().float() * h_post + self.post_beta.leaf().float())
    rs = self.res_alpha_scale.leaf().float()
    if self.lite:
      if self._perms is None or self._perms.device != x.device:
        self._perms = permutation_matrices(k, x.device)
      wts = torch.softmax(rs * h_res + self.res_beta.leaf().float(), dim=-1)
      res = torch.einsum("bsn,nkm->bskm", wts, self._perms)
    else:
      res = sinkhorn(rs * h_res.reshape(B, S, k, k) + self.res_beta.leaf().float(), self.iters)
    return pre, post, res

  def __call__(self, norm_fn, branch_fn, x: torch.Tensor) -> torch.Tensor:
    """x [B, S, k, D] -> [B, S, k, D]; `branch_fn` maps the normalised [B, S, D] branch input to the branch output."""
    pre, post, res = self.maps(x)
    xf = x.float()
    inp = torch.einsum("bsk,bskd->bsd", pre, xf).to(x.dtype)
    out = branch_fn(norm_fn(inp) if norm_fn is not None else inp)
    post_out = out.float().unsqueeze(2) * post.unsqueeze(3)
    res_out = torch.einsum("bskm,bskd->bsmd", res, xf)
    return (res_out + post_out).to(x.dtype)


class HyperHead:
  """Final collapse of the k streams (DeepSeek-V4): scale-free RMS statistic of the flattened stream, a [k*D, k] projection,
  sigmoid gates, weighted sum of the streams."""

  def __init__(self, b: L.Builder, config, name: str = "hyper_head"):
    c = config
    self.k, self.dim, self.eps = int(c.mhc_expansion_rate), int(c.emb_dim), 1e-6
    sb = b.sub(name)
    self.hc_fn = sb.linear("hc_fn", (self.k * self.dim,), (self.k,), ("activation_embed", None), init="fan_in_normal")
    self.hc_base = sb.vector("hc_base", self.k, axes=(None,), init="zeros")
    self.hc_scale = sb._add("hc_scale", shape=(1,), ref_shape=(1,), logical_axes=(None,), kind="same", init="const", init_scale=0.01)

  def __call__(self, x: torch.Tensor) -> torch.Tensor:
    B, S, k, D = x.shape
    flat = x.reshape(B, S, k * D).float()
    flat = flat * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + self.eps)
    mixes = torch.matmul(flat, self.hc_fn.leaf().float().t())
    pre = torch.sigmoid(mixes * self.hc_scale.leaf().float() + self.hc_base.leaf().float()) + self.eps
    return (pre.unsqueeze(-1) * x.float()).sum(2).to(x.dtype)
