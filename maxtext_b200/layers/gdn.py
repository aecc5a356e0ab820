"""Gated delta network: the linear-attention layer of Qwen3-Next (src/maxtext/models/qwen3.py:62-1015).

Per value head the layer keeps a matrix state S [Dk, Dv] and, per token t,

  S <- exp(g_t) S                        (decay, g_t = -exp(A_log) softplus(a_t + dt_bias) <= 0)
  S <- S + k_t (beta_t (v_t - S^T k_t))^T   (delta rule: overwrite what the key currently retrieves)
  o_t = S^T q_t

with q, k L2-normalised, q scaled by Dk^-1/2, and q | k | v first passed through a depthwise causal convolution and
SiLU. Training and prefill evaluate the recurrence chunk by chunk so that almost all of the work is matrix products:
inside a chunk of C tokens the dependence of the written values on each other is a unit lower triangular system
(solved once per chunk), and only the [Dk, Dv] state crosses chunk borders. Decode applies the three lines above to
the cached state.
"""
from __future__ import annotations

import torch
import torch.nn.functional as tF

from ..ops import functional as F
from .blocks import Builder


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
  return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def gated_delta_recurrent(q, k, v, g, beta, state=None):
  """Token-by-token evaluation (the definition; used for decode and as the oracle of the chunked form).

  q, k [B,T,H,Dk]; v [B,T,H,Dv]; g, beta [B,T,H]; state [B,H,Dk,Dv] or None. fp32 inside. Returns (o [B,T,H,Dv], state)."""
  B, T, H, Dk = q.shape
  Dv = v.shape[-1]
  qf, kf, vf = l2norm(q.float()) * Dk ** -0.5, l2norm(k.float()), v.float()
  S = torch.zeros(B, H, Dk, Dv, dtype=torch.float32, device=q.device) if state is None else state.float()
  outs = []
  for t in range(T):
    S = S * torch.exp(g[:, t].float())[:, :, None, None]
    kt = kf[:, t]
    read = torch.einsum("bhkv,bhk->bhv", S, kt)
    delta = (vf[:, t] - read) * beta[:, t].float()[:, :, None]
    S = S + kt[..., None] * delta[:, :, None, :]
    outs.append(torch.einsum("bhkv,bhk->bhv", S, qf[:, t]))
  return torch.stack(outs, 1), S


def gated_delta_chunked(q, k, v, g, beta, chunk: int = 64, state=None):
  """The same function with O(T/C) sequential steps. Shapes as in `gated_delta_recurrent`."""
  B, T, H, Dk = q.shape
  Dv = v.shape[-1]
  C = int(chunk)
  pad = (-T) % C
  qf = (l2norm(q.float()) * Dk ** -0.5).transpose(1, 2)          # [B,H,T,Dk]
  kf = l2norm(k.float()).transpose(1, 2)
  vf = v.float().transpose(1, 2)
  gf = g.float().transpose(1, 2)                                 # [B,H,T]
  bf = beta.float().transpose(1, 2)
  if pad:                                                        # zero keys / values and zero log-decay leave the state unchanged
    qf, kf, vf = tF.pad(qf, (0, 0, 0, pad)), tF.pad(kf, (0, 0, 0, pad)), tF.pad(vf, (0, 0, 0, pad))
    gf, bf = tF.pad(gf, (0, pad)), tF.pad(bf, (0, pad))
  N = (T + pad) // C
  qc, kc, vc = qf.view(B, H, N, C, Dk), kf.view(B, H, N, C, Dk), vf.view(B, H, N, C, Dv)
  gc = gf.view(B, H, N, C).cumsum(-1)                            # log-decay from the chunk start up to and including token i
  bc = bf.view(B, H, N, C)
  kb, vb = kc * bc[..., None], vc * bc[..., None]
  low = torch.tril(torch.ones(C, C, dtype=torch.bool, device=q.device))
  strict = torch.tril(torch.ones(C, C, dtype=torch.bool, device=q.device), -1)
  # decay from token j (after its write) to token i, for j <= i; masked before exp so that no inf * 0 appears
  diff = (gc[..., :, None] - gc[..., None, :]).masked_fill(~low, 0.0)
  decay = torch.exp(diff) * low
  # (I + L) w = rhs, L[i,j] = beta_i k_i.k_j decay_ij for j < i: token i's write depends on the earlier writes of its chunk
  Lmat = (kb @ kc.transpose(-1, -2)) * decay * strict
  eye = torch.eye(C, dtype=torch.float32, device=q.device)
  Tinv = torch.linalg.solve_triangular(eye + Lmat, eye.expand_as(Lmat), upper=False)
  u = Tinv @ vb                                                  # writes if the incoming state were zero
  w = Tinv @ (kb * torch.exp(gc)[..., None])                     # how much of the incoming state each write removes
  qk = (qc @ kc.transpose(-1, -2)) * decay                       # lower triangular incl. the diagonal
  S = torch.zeros(B, H, Dk, Dv, dtype=torch.float32, device=q.device) if state is None else state.float()
  outs = []
  for n in range(N):
    v_new = u[:, :, n] - w[:, :, n] @ S                          # [B,H,C,Dv]
    o = (qc[:, :, n] * torch.exp(gc[:, :, n])[..., None]) @ S + qk[:, :, n] @ v_new
    glast = gc[:, :, n, -1]
    S = S * torch.exp(glast)[..., None, None] + (kc[:, :, n] * torch.exp(glast[..., None] - gc[:, :, n])[..., None]).transpose(-1, -2) @ v_new
    outs.append(o)
  o = torch.stack(outs, 2).view(B, H, N * C, Dv)[:, :, :T]
  return o.transpose(1, 2), S


class GDNState:
  """Decode-time state of one gated-delta layer for `slots` sequences: the last K-1 convolution inputs and S."""

  def __init__(self, slots, conv_dim, kernel, heads, dk, dv, device):
    self.conv = torch.zeros(slots, kernel - 1, conv_dim, dtype=torch.float32, device=device)
    self.rec = torch.zeros(slots, heads, dk, dv, dtype=torch.float32, device=device)
    self.slot_ids = None
    self.lengths = None

  def bind(self, slot_ids, lengths):
    self.slot_ids, self.lengths = slot_ids, lengths


class GatedDeltaNet:
  """Parameters follow the reference tree: in_proj_qkvz / in_proj_ba / conv1d / A_log / dt_bias / norm/rms_norm / out_proj.

  `in_proj_qkvz` packs, per key head, [q (Dk) | k (Dk) | v (r Dv) | z (r Dv)] with r value heads per key head, and
  `in_proj_ba` packs per key head [b (r) | a (r)]."""

  def __init__(self, b: Builder, config, name="attention"):
    c = config
    assert b.tp_size == 1, "the gated delta network is not split over the tensor axis"
    self.c = c
    self.hk, self.hv = int(c.gdn_num_key_heads), int(c.gdn_num_value_heads)
    self.dk, self.dv = int(c.gdn_key_head_dim), int(c.gdn_value_head_dim)
    self.r = self.hv // self.hk
    self.K = int(c.gdn_conv_kernel_dim)
    self.chunk = int(c.gdn_chunk_size)
    self.key_dim, self.value_dim = self.hk * self.dk, self.hv * self.dv
    self.conv_dim = 2 * self.key_dim + self.value_dim
    d = c.emb_dim
    ab = b.sub(*name.split("/"))
    self.in_qkvz = ab.sub("in_proj_qkvz").linear("kernel", (d,), (2 * self.key_dim + 2 * self.value_dim,), ("embed", "gdn_head"))
    self.in_ba = ab.sub("in_proj_ba").linear("kernel", (d,), (2 * self.hv,), ("embed", "gdn_head"))
    # depthwise filter, reference layout [kernel, 1, channels]
    self.conv = ab.sub("conv1d").table("kernel", (self.K, 1, self.conv_dim), (None, None, "gdn_head"), init="fan_in_normal")
    self.A_log = ab.vector("A_log", self.hv, (None,), init="log_uniform_16")
    self.dt_bias = ab.vector("dt_bias", self.hv, (None,), init="ones")
    self.norm = ab.sub("norm", "rms_norm").vector("scale", self.dv, ("norm",))
    self.out = ab.sub("out_proj").linear("kernel", (self.value_dim,), (d,), ("gdn_head", "embed"))

  def __call__(self, x, ctx):
    B, S, _ = x.shape
    hk, r, dk, dv = self.hk, self.r, self.dk, self.dv
    qkvz = F.linear(x, self.in_qkvz).view(B, S, hk, 2 * dk + 2 * r * dv)
    ba = F.linear(x, self.in_ba).view(B, S, hk, 2 * r)
    q, k, v, z = torch.split(qkvz, [dk, dk, r * dv, r * dv], dim=-1)
    bb, aa = ba[..., :r].reshape(B, S, self.hv), ba[..., r:].reshape(B, S, self.hv)
    z = z.reshape(B, S, self.hv, dv)
    mixed = torch.cat([q.reshape(B, S, -1), k.reshape(B, S, -1), v.reshape(B, S, -1)], dim=-1).float()   # [B,S,conv_dim]
    st = ctx.cache if isinstance(ctx.cache, GDNState) else None
    if st is not None:
      hist = st.conv[st.slot_ids]                                                                      # [B,K-1,conv_dim]
    else:
      hist = torch.zeros(B, self.K - 1, self.conv_dim, dtype=torch.float32, device=x.device)
    seq = torch.cat([hist, mixed], dim=1)
    wconv = self.conv.leaf().float().view(self.K, self.conv_dim)
    conv = sum(seq[:, j:j + S] * wconv[j] for j in range(self.K))
    conv = tF.silu(conv)
    if st is not None:
      st.conv[st.slot_ids] = seq[:, -(self.K - 1):]
    q, k, v = torch.split(conv, [self.key_dim, self.key_dim, self.value_dim], dim=-1)
    q, k, v = q.view(B, S, hk, dk), k.view(B, S, hk, dk), v.view(B, S, self.hv, dv)
    if r > 1:
      q, k = q.repeat_interleave(r, dim=2), k.repeat_interleave(r, dim=2)
    beta = torch.sigmoid(bb.float())
    g = -torch.exp(self.A_log.leaf().float()) * tF.softplus(aa.float() + self.dt_bias.leaf().float())
    s0 = st.rec[st.slot_ids] if st is not None else None
    if S == 1:
      o, s1 = gated_delta_recurrent(q, k, v, g, beta, s0)
    else:
      o, s1 = gated_delta_chunked(q, k, v, g, beta, self.chunk, s0)
    if st is not None:
      st.rec[st.slot_ids] = s1
    # RMS norm over the value head dim, learned scale, then the SiLU gate
    eps = self.c.normalization_layer_epsilon
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * self.norm.leaf().float()
    o = (o * tF.silu(z.float())).to(x.dtype)
    return F.linear(o.reshape(B, S, self.value_dim), self.out)
