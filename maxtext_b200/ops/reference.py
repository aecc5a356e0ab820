"""Plain-PyTorch definitions of every hot op.

These are the numerical oracles for the CUDA kernels in `csrc/` and the implementation used on CPU
(tests, the fp32 tiny-model configuration). Shapes follow the kernels' conventions:
activations are `[tokens, features]` or `[batch, seq, heads, head_dim]`, linear weights are stored
`[out, in]` (K-major for the forward GEMM).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# ----------------------------------------------------------------------------- norms
def rmsnorm(x: torch.Tensor, scale: torch.Tensor | None, eps: float, offset: float = 0.0) -> torch.Tensor:
  """y = (x_f32 * rsqrt(mean(x_f32^2) + eps)).to(dtype) * (scale.to(dtype) + offset)
  (src/maxtext/layers/normalizations.py:75-96: the scale multiply happens in the compute dtype)."""
  xf = x.float()
  y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
  if scale is None:
    return y
  return y * (scale.to(x.dtype) + offset)


def rmsnorm_bwd(dy, x, scale, eps, offset=0.0):
  xf, dyf = x.float(), dy.float()
  rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
  xhat = xf * rstd
  g = dyf * (scale.float() + offset) if scale is not None else dyf
  dx = rstd * (g - xhat * (g * xhat).mean(-1, keepdim=True))
  dscale = (dyf * xhat).reshape(-1, x.shape[-1]).sum(0) if scale is not None else None
  return dx.to(x.dtype), dscale


def layernorm(x, scale, bias, eps):
  y = F.layer_norm(x.float(), (x.shape[-1],), None, None, eps).to(x.dtype)
  if scale is not None:
    y = y * scale.to(x.dtype)
  if bias is not None:
    y = y + bias.to(x.dtype)
  return y


# ----------------------------------------------------------------------------- rope
def rope_inv_timescale(head_dim: int, min_ts: float, max_ts: float, linear_scaling: float = 1.0,
                       rope_type: str = "default", use_scale: bool = True, yarn: dict | None = None) -> torch.Tensor:
  """1/timescale per rotated pair, shape [head_dim/2] fp32.

  default: timescale_i = min*(max/min)^(2i/d) (x linear factor) (src/maxtext/layers/embeddings.py:318-334)
  llama3.1: same base, then the Llama-3.1 wavelength-dependent rescale (embeddings.py:646-672)
  yarn: blend of interpolated and extrapolated frequencies (embeddings.py:880-1027)
  """
  half = head_dim // 2
  frac = 2.0 * torch.arange(half, dtype=torch.float64) / head_dim
  ts = min_ts * (max_ts / min_ts) ** frac
  if rope_type == "default" and linear_scaling != 1.0:
    ts = ts * linear_scaling
  inv = 1.0 / ts
  if rope_type.startswith("llama3.1") and use_scale:
    scale_factor, low_f, high_f, old_len = 8.0, 1.0, 4.0, 8192.0
    wavelen = 2 * math.pi / inv
    smooth = (old_len / wavelen - low_f) / (high_f - low_f)
    mid = (1 - smooth) * inv / scale_factor + smooth * inv
    inv = torch.where(wavelen < old_len / high_f, inv, torch.where(wavelen > old_len / low_f, inv / scale_factor, mid))
  elif rope_type.startswith("yarn"):
    y = yarn or {}
    factor = float(y.get("rope_factor", 40))
    orig = float(y.get("original_max_position_embeddings", 4096))
    beta_fast, beta_slow = float(y.get("beta_fast", 32)), float(y.get("beta_slow", 1))
    truncate = bool(y.get("rope_truncate", True))

    def corr_dim(num_rot):
      return (head_dim * math.log(orig / (num_rot * 2 * math.pi))) / (2 * math.log(max_ts))

    low, high = corr_dim(beta_fast), corr_dim(beta_slow)
    if truncate:
      low, high = math.floor(low), math.ceil(high)
    low, high = max(low, 0), min(high, head_dim - 1)
    if low == high:
      high += 0.001
    ramp = ((torch.arange(half, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
    smooth = 1.0 - ramp
    inv = inv / factor * (1 - smooth) + inv * smooth
  return inv.float()


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_ts: torch.Tensor, interleaved: bool,
               rotary_dim: int | None = None, inverse: bool = False) -> torch.Tensor:
  """x [B,S,H,Dh]; positions [B,S]. interleaved=False rotates (first half, second half) lanes,
  True rotates adjacent pairs (Llama layout). `inverse` applies the transpose rotation (backward)."""
  d = x.shape[-1] if rotary_dim is None else rotary_dim
  xr, rest = x[..., :d], x[..., d:]
  ang = positions[:, :, None, None].float() * inv_ts.to(x.device)[None, None, None, :]
  sin, cos = torch.sin(ang), torch.cos(ang)
  if inverse:
    sin = -sin
  xf = xr.float()
  if interleaved:
    x1, x2 = xf[..., 0::2], xf[..., 1::2]
    o1, o2 = x1 * cos - x2 * sin, x2 * cos + x1 * sin
    out = torch.stack([o1, o2], dim=-1).flatten(-2)
  else:
    x1, x2 = xf[..., : d // 2], xf[..., d // 2:]
    out = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)
  out = out.to(x.dtype)
  return torch.cat([out, rest], dim=-1) if rest.shape[-1] else out


def mrope_axis_of_frequency(n_freq: int, sections) -> torch.Tensor:
  """Which position axis (0 temporal, 1 height, 2 width) drives each of the n_freq rotary frequencies under the interleaved
  multi-axis layout of Qwen3-VL / Omni (src/maxtext/layers/embeddings.py:1861-1886): temporal everywhere, except that indices
  1, 4, 7, ... below 3 * sections[1] use the height and indices 2, 5, 8, ... below 3 * sections[2] the width."""
  axis = torch.zeros(n_freq, dtype=torch.long)
  axis[1:3 * int(sections[1]):3] = 1
  axis[2:3 * int(sections[2]):3] = 2
  return axis


def apply_mrope(x: torch.Tensor, positions3: torch.Tensor, inv_ts: torch.Tensor, sections, rotary_dim: int | None = None) -> torch.Tensor:
  """Rotate-half rotary embedding whose angle for frequency i is positions3[b, s, axis(i)] * inv_ts[i]; x [B,S,H,Dh],
  positions3 [B,S,3] (text tokens carry the same number on all three axes, which makes this the ordinary embedding)."""
  d = x.shape[-1] if rotary_dim is None else rotary_dim
  xr, rest = x[..., :d], x[..., d:]
  axis = mrope_axis_of_frequency(d // 2, sections).to(x.device)
  pos = positions3.float()[..., axis]                                     # [B, S, d/2]
  ang = (pos * inv_ts.to(x.device).float())[:, :, None, :]
  sin, cos = torch.sin(ang), torch.cos(ang)
  xf = xr.float()
  x1, x2 = xf[..., : d // 2], xf[..., d // 2:]
  out = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)
  return torch.cat([out, rest], dim=-1) if rest.shape[-1] else out


# ----------------------------------------------------------------------------- activations
_ACTS = {
    "silu": F.silu, "swish": F.silu, "gelu": lambda t: F.gelu(t, approximate="tanh"), "gelu_exact": F.gelu,
    "relu": F.relu, "linear": lambda t: t, "sigmoid": torch.sigmoid, "tanh": torch.tanh,
}


def act_fn(name: str):
  return _ACTS[name]


def gated_act(gate_up: torch.Tensor, act: str = "silu") -> torch.Tensor:
  """[T, 2F] laid out [gate | up] -> act(gate) * up in the input dtype (src/maxtext/layers/linears.py:600-625)."""
  g, u = gate_up.chunk(2, dim=-1)
  return (_ACTS[act](g.float()) * u.float()).to(gate_up.dtype)


def gated_act_bwd(dy, gate_up, act="silu"):
  g, u = gate_up.float().chunk(2, dim=-1)
  dyf = dy.float()
  with torch.enable_grad():
    gg = g.detach().requires_grad_()
    a = _ACTS[act](gg)
    (da,) = torch.autograd.grad(a, gg, dyf * u)
  return torch.cat([da, dyf * a.detach()], dim=-1).to(gate_up.dtype)


# ----------------------------------------------------------------------------- attention
def attention_mask(q_pos, kv_pos, q_seg=None, kv_seg=None, causal=True, sliding_window=0, chunk=0):
  """Boolean [B,1,Sq,Skv] mask (True = attend) from original token positions and segment ids."""
  qp, kp = q_pos[:, :, None], kv_pos[:, None, :]
  m = torch.ones(qp.shape[0], qp.shape[1], kp.shape[2], dtype=torch.bool, device=q_pos.device)
  if causal:
    m &= kp <= qp
  if sliding_window and sliding_window > 0:
    m &= (qp - kp) < sliding_window
  if chunk and chunk > 0:
    m &= (qp // chunk) == (kp // chunk)
  if q_seg is not None and kv_seg is not None:
    m &= q_seg[:, :, None] == kv_seg[:, None, :]
    m &= kv_seg[:, None, :] != 0
  return m[:, None]


def attention(q, k, v, mask=None, scale: float = 1.0, soft_cap: float = 0.0, sinks=None, return_lse=False):
  """q [B,Sq,Hq,D], k [B,Skv,Hkv,D], v [B,Skv,Hkv,Dv] -> [B,Sq,Hq,Dv]; fp32 logits and softmax
  (src/maxtext/layers/attention_op.py:2480-2602). MaxText folds 1/sqrt(d) into the query weights, so
  the default scale is 1."""
  B, Sq, Hq, D = q.shape
  Hkv = k.shape[2]
  g = Hq // Hkv
  qf = q.float().view(B, Sq, Hkv, g, D)
  logits = torch.einsum("bqhgd,bkhd->bhgqk", qf, k.float()) * scale
  if soft_cap and soft_cap > 0:
    logits = torch.tanh(logits / soft_cap) * soft_cap
  if mask is not None:
    logits = logits.masked_fill(~mask[:, :, None], -1e30)
  if sinks is not None:
    s = sinks.float().view(1, Hkv, g, 1, 1).expand(B, Hkv, g, Sq, 1)
    full = torch.cat([logits, s], dim=-1)
    lse = torch.logsumexp(full, dim=-1)
  else:
    lse = torch.logsumexp(logits, dim=-1)
  p = torch.exp(logits - lse[..., None])
  if mask is not None:
    p = p.masked_fill(~mask[:, :, None], 0.0)
  out = torch.einsum("bhgqk,bkhd->bqhgd", p, v.float()).reshape(B, Sq, Hq, v.shape[-1]).to(q.dtype)
  if return_lse:
    return out, lse.reshape(B, Hq, Sq)
  return out


# ----------------------------------------------------------------------------- loss
def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, z_loss: float = 0.0):
  """Per-token xent = logsumexp - logit[target] (+ z_loss*log(z)^2) in fp32
  (src/maxtext/utils/max_utils.py:626-716). Returns (loss_per_token, z_term_per_token)."""
  lf = logits.float()
  lse = torch.logsumexp(lf, dim=-1)
  tgt = lf.gather(-1, targets.unsqueeze(-1).long()).squeeze(-1)
  z = z_loss * lse.pow(2) if z_loss else torch.zeros_like(lse)
  return lse - tgt + z, z


def cross_entropy_dlogits(logits, targets, weights, z_loss: float = 0.0):
  """d(sum_t w_t * loss_t)/dlogits = w * ((1 + 2 z lse) softmax - onehot)."""
  lf = logits.float()
  lse = torch.logsumexp(lf, dim=-1, keepdim=True)
  p = torch.exp(lf - lse)
  if z_loss:
    p = p * (1.0 + 2.0 * z_loss * lse)
  p.scatter_add_(-1, targets.unsqueeze(-1).long(), -torch.ones_like(lse))
  return p * weights.unsqueeze(-1).float()


# ----------------------------------------------------------------------------- optimizer
def adamw_step(p, g, m, v, lr, b1, b2, eps, eps_root, wd, step, grad_scale=1.0):
  """optax.adamw semantics (src/maxtext/optimizers/optimizers.py:173-182): bias-corrected moments,
  u = m_hat / (sqrt(v_hat + eps_root) + eps), p -= lr * (u + wd * p). `step` is 1-based."""
  g = g.float() * grad_scale
  m.mul_(b1).add_(g, alpha=1 - b1)
  v.mul_(b2).addcmul_(g, g, value=1 - b2)
  mh = m.float() / (1 - b1 ** step)
  vh = v.float() / (1 - b2 ** step)
  u = mh / (torch.sqrt(vh + eps_root) + eps)
  p.add_(u + wd * p, alpha=-lr)
  return p


# ----------------------------------------------------------------------------- MoE helpers
def topk_route(logits: torch.Tensor, k: int):
  vals, idx = torch.topk(logits, k, dim=-1)
  return vals, idx


def permute_by_expert(x: torch.Tensor, expert_idx: torch.Tensor, num_experts: int):
  """Dropless permutation (src/maxtext/layers/moe.py:872-1002): flatten [T,k] ids, stable argsort,
  repeat tokens k times, gather. Returns rows sorted by expert, sort order, group sizes."""
  T, k = expert_idx.shape
  flat = expert_idx.reshape(-1)
  order = torch.argsort(flat, stable=True)
  rows = x.repeat_interleave(k, dim=0)[order] if k > 1 else x[order]
  sizes = torch.bincount(flat, minlength=num_experts)
  return rows, order, sizes


def grouped_matmul(x: torch.Tensor, w: torch.Tensor, group_sizes: torch.Tensor) -> torch.Tensor:
  """Rows of x are grouped by expert; w is [E, N, K] ([out,in] per expert). Returns [rows, N]."""
  out = x.new_empty(x.shape[0], w.shape[1])
  start = 0
  for e, n in enumerate(group_sizes.tolist()):
    if n:
      out[start:start + n] = x[start:start + n] @ w[e].t().to(x.dtype)
    start += n
  if start < x.shape[0]:
    out[start:] = 0
  return out


def moba_block_mask(q, k, q_pos, chunk: int, topk: int):
  """Mixture-of-block attention gate (src/maxtext/layers/attention_op.py:1149-1259): keys are grouped into blocks of `chunk`
  positions, each query scores a block by its dot product with the block's mean key, blocks in the future are excluded, the
  query's own block always counts, and only the `topk` best blocks are attended (within them, causally).

  q [B,Sq,Hq,D], k [B,Skv,Hkv,D], q_pos [B,Sq] -> bool [B,Hkv,g,Sq,Skv] (True = attend)."""
  B, Sq, Hq, D = q.shape
  Skv, Hkv = k.shape[1], k.shape[2]
  g = Hq // Hkv
  nb = -(-Skv // chunk)
  kf = k.float()
  pad = nb * chunk - Skv
  kp = F.pad(kf, (0, 0, 0, 0, 0, pad)) if pad else kf
  cnt = torch.full((nb,), float(chunk), device=k.device)
  if pad:
    cnt[-1] = chunk - pad
  kmean = kp.view(B, nb, chunk, Hkv, D).sum(2) / cnt[None, :, None, None]                      # [B,nb,Hkv,D]
  gate = torch.einsum("bskgd,bnkd->bkgsn", q.float().view(B, Sq, Hkv, g, D), kmean)            # [B,Hkv,g,Sq,nb]
  qb = (q_pos // chunk)[:, None, None, :, None]
  blocks = torch.arange(nb, device=q.device)[None, None, None, None, :]
  gate = torch.where(qb > blocks, gate, torch.full_like(gate, float("-inf")))
  gate = torch.where(qb == blocks, torch.full_like(gate, float("inf")), gate)
  kk = min(int(topk), nb)
  top_val, top_idx = gate.topk(kk, dim=-1)
  chosen = torch.zeros_like(gate, dtype=torch.bool).scatter_(-1, top_idx, True) & (gate >= top_val.min(-1, keepdim=True).values)
  kblock = torch.arange(Skv, device=q.device) // chunk
  token = chosen[..., kblock]                                                                   # [B,Hkv,g,Sq,Skv]
  causal = q_pos[:, None, None, :, None] >= torch.arange(Skv, device=q.device)[None, None, None, None, :]
  return token & causal


def moba_attention(q, k, v, q_pos, chunk: int, topk: int, scale: float = 1.0, extra_mask=None):
  """Softmax attention restricted by `moba_block_mask` (and by `extra_mask` [B,1,Sq,Skv], e.g. segments)."""
  B, Sq, Hq, D = q.shape
  Hkv = k.shape[2]
  g = Hq // Hkv
  m = moba_block_mask(q, k, q_pos, chunk, topk)
  if extra_mask is not None:
    m = m & extra_mask[:, :, None]
  logits = torch.einsum("bqhgd,bkhd->bhgqk", q.float().view(B, Sq, Hkv, g, D), k.float()) * scale
  p = torch.softmax(logits.masked_fill(~m, -1e30), dim=-1)
  return torch.einsum("bhgqk,bkhd->bqhgd", p, v.float()).reshape(B, Sq, Hq, v.shape[-1]).to(q.dtype)
