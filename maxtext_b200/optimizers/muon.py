"""Muon: momentum + Newton-Schulz orthogonalisation for weight matrices, AdamW for everything else.

Follows src/maxtext/optimizers/muon.py:287-555 and the parameter selection of src/maxtext/utils/muon_utils.py:47-128:
  mu <- beta*mu + (1-beta)*g;  Nesterov blend of bias-corrected mu and g;  X <- X / (||X||_F + eps);
  five quintic iterations X <- a X + (b A + c A^2) X with A = X X^T, (a, b, c) = (3.4445, -4.7750, 2.0315);
  update = X * sqrt(max(1, fan_out/fan_in))  (or sqrt(max(fan_in, fan_out)) * consistent_rms);
  p <- p - lr * (update + muon_weight_decay * p).
Embeddings, the output head, norm scales and biases use AdamW with the Adam hyper-parameters.
Expert weights are orthogonalised per expert; attention kernels as [in, heads*dim] matrices.

Storage is the flat ZeRO-3 shard, so for each matrix the momentum shard is all-gathered over the unit's shard
group, orthogonalised (the three GEMMs per iteration run on the tcgen05 GEMM when the operands are bf16 on a GPU)
and the local chunk of the result is applied. Ranks orthogonalise every matrix of the unit redundantly.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..ops import functional as F
from .factory import _Base

NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz(x: torch.Tensor, steps: int = 5, coeffs=NS_COEFFS, eps: float = 1e-8) -> torch.Tensor:
  """Approximate orthogonalisation of the last two dims (batched over leading dims)."""
  a, b, c = coeffs
  transposed = x.shape[-2] > x.shape[-1]
  if transposed:
    x = x.transpose(-1, -2)
  x = x / (x.norm(dim=(-2, -1), keepdim=True) + eps)
  if x.is_cuda and x.dim() == 2:
    # bf16 iterations on this repository's GEMM (nt, then two nn products per step), as the reference runs them in bf16
    xb = x.to(torch.bfloat16).contiguous()
    for _ in range(steps):
      A = F.mm(xb, xb, False, True)
      B = (b * A + c * F.mm(A, A, False, False)).to(torch.bfloat16)
      xb = (a * xb + F.mm(B, xb, False, False)).to(torch.bfloat16)
    x = xb.to(x.dtype)
  else:
    for _ in range(steps):
      A = x @ x.transpose(-1, -2)
      B = b * A + c * (A @ A)
      x = a * x + B @ x
  return x.transpose(-1, -2) if transposed else x


def is_muon_param(pdef) -> bool:
  """Matrices inside decoder layers; not embeddings / logits head / vectors (src/maxtext/utils/muon_utils.py:47-128)."""
  if pdef.layer is None:
    return False
  return pdef.kind in ("linear", "expert_linear") and len(pdef.shape) >= 2 and "gate" not in pdef.ref_path


class Muon(_Base):
  def __init__(self, config, store, model):
    super().__init__(config, store, model)
    store.ensure_opt_state()
    self.muon_params = [p for p in store.params.values() if is_muon_param(p.pdef)]
    self.steps = 10 if config.decoder_block == "deepseek4" else 5

  def _ranges(self):
    """Contiguous local-shard ranges of the parameters that stay on AdamW."""
    store = self.store
    out = []
    for u in store.units.values():
      lo, hi = u.group_rank * u.chunk, (u.group_rank + 1) * u.chunk
      for p, off in zip(u.params, u.offsets):
        if is_muon_param(p.pdef):
          continue
        a, b = max(off, lo), min(off + p.pdef.numel, hi)
        if a < b:
          out.append((u.shard_offset + a - lo, u.shard_offset + b - lo))
    return out

  def step(self, grad_scale, lr, step, **kw):
    c, s = self.c, self.store
    for a, b in self._ranges():
      _adamw_torch(s, a, b, lr, c, step, grad_scale)
    beta = float(c.muon_beta)
    bc1, bc2 = 1 - beta ** step, 1 - beta ** (step + 1)
    for p in self.muon_params:
      u = s.unit_of(p)
      off = u.offsets[u.params.index(p)]
      n = p.pdef.numel
      lo, hi = u.group_rank * u.chunk, (u.group_rank + 1) * u.chunk
      a, b = max(off, lo), min(off + n, hi)
      base = u.shard_offset - lo
      if a < b:
        g = s.grad_shard[base + a: base + b].float() * grad_scale
        m = s.exp_avg[base + a: base + b]
        m.mul_(beta).add_(g, alpha=1 - beta)
        local = beta * (m.float() / bc2) + (1 - beta) * (g / bc1)        # Nesterov look-ahead on bias-corrected terms
      else:
        local = torch.zeros(0, device=s.device)
      full = self._gather_param(u, off, n, a, b, local).view(p.pdef.shape)
      d = p.pdef
      mat = full if d.kind == "expert_linear" else full.view(d.shape[0], -1)
      ortho = newton_schulz(mat.float(), self.steps, eps=float(c.adam_eps))
      fan_out, fan_in = mat.shape[-2], mat.shape[-1]
      scale = math.sqrt(max(fan_in, fan_out)) * float(c.muon_consistent_rms) if c.muon_consistent_rms is not None \
          else math.sqrt(max(1.0, fan_out / fan_in))
      upd = (ortho * scale).reshape(-1)
      if a < b:
        w = s.master[base + a: base + b]
        w.add_(upd[a - off: b - off].to(w.dtype) + float(c.muon_weight_decay) * w, alpha=-lr)
    s.sync_compute_from_master()
    return {}

  def _gather_param(self, u, off, n, a, b, local):
    """Assemble the whole tensor from the chunks each rank of the shard group holds."""
    if u.group_size == 1:
      return local
    pieces = [None] * u.group_size
    dist.all_gather_object(pieces, (a - off, b - off), group=u.group)
    full = torch.zeros(n, device=local.device)
    bufs = [torch.zeros(max(0, e - st), device=local.device) for st, e in pieces]
    # variable-size gather: pad to the largest piece
    mx = max(max(0, e - st) for st, e in pieces)
    pad = torch.zeros(mx, device=local.device)
    pad[: local.numel()] = local
    got = [torch.empty_like(pad) for _ in range(u.group_size)]
    dist.all_gather(got, pad, group=u.group)
    for (st, e), gpiece in zip(pieces, got):
      if e > st:
        full[st:e] = gpiece[: e - st]
    del bufs
    return full

  def state_arrays(self):
    return {"mu": self.store.exp_avg, "nu": self.store.exp_avg_sq}


def _adamw_torch(s, a, b, lr, c, step, grad_scale):
  F.adamw_flat(s.master[a:b], s.grad_shard[a:b], s.exp_avg[a:b], s.exp_avg_sq[a:b],
               None if s.alias_compute else s.compute_shard[a:b], lr, c.adam_b1, c.adam_b2, c.adam_eps, c.adam_eps_root,
               c.adam_weight_decay, step, grad_scale)
