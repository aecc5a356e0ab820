"""Optimizers over the flat parameter shards.

`opt_type` values and hyper-parameters are those of src/maxtext/optimizers/optimizers.py:169-252:
adamw (optax.adamw semantics), adam_pax, sgd and muon (src/maxtext/optimizers/muon.py), optionally
wrapped by skip-step-on-spikes (optimizers.py:67-166). Every optimizer receives the device scalar
`grad_scale` = clip_factor / total_weights so that normalisation, clipping and the update happen in
one pass over memory without a host synchronisation.
"""
from __future__ import annotations

import math

import torch

from ..ops import functional as F


class _Base:
  def __init__(self, config, store, model):
    self.c, self.store, self.model = config, store, model

  def state_arrays(self) -> dict:
    return {}


class AdamW(_Base):
  """One fused launch: m, v, bias correction, decoupled weight decay, fp32 master and bf16 shadow write."""

  def __init__(self, config, store, model, pax: bool = False):
    super().__init__(config, store, model)
    self.pax = pax
    store.ensure_opt_state()
    self.param_sumsq = torch.zeros(1, dtype=torch.float32, device=store.device)

  def step(self, grad_scale, lr, step, **kw):
    c, s = self.c, self.store
    wd = c.adam_weight_decay
    trainable = s.decay_slices()
    if trainable is not None:
      # some parameters are frozen (LoRA, trainable_parameters_mask) or excluded from decay (adamw_mask). A frozen one has an
      # exactly zero gradient, so with no decay term the fused update leaves it untouched; the decoupled decay
      # w <- w (1 - lr wd) is applied to the decayed ranges first, which gives the same result as the fused w - lr (u + wd w)
      if wd:
        for a, b in trainable:
          s.master[a:b].mul_(1.0 - lr * wd)
      wd = 0.0
    F.adamw_flat(s.master, s.grad_shard, s.exp_avg, s.exp_avg_sq, s.compute_shard, lr, c.adam_b1, c.adam_b2, c.adam_eps,
                 c.adam_eps_root, wd, step, grad_scale, pax=self.pax)
    return {}

  def state_arrays(self):
    return {"mu": self.store.exp_avg, "nu": self.store.exp_avg_sq}


class SGD(_Base):
  def step(self, grad_scale, lr, step, **kw):
    s = self.store
    s.master.add_(s.grad_shard.float() * grad_scale, alpha=-lr)
    s.sync_compute_from_master()
    return {}


class SkipOnSpikes:
  """Skip the update when loss or gradient norm exceeds mean + k*std of a rolling window
  (src/maxtext/optimizers/optimizers.py:67-166). The decision is made on the device: a spike turns
  the step into a no-op by zeroing the learning rate through `grad_scale` and restoring the moments."""

  def __init__(self, inner, interval: int, factor: float):
    self.inner, self.interval, self.factor = inner, int(interval), float(factor)
    self.hist_loss: list = []
    self.hist_norm: list = []
    self.skipped = 0

  def _is_spike(self, hist, value):
    if len(hist) < 2:
      return False
    t = torch.stack(hist[-self.interval:]).float()
    mean, std = t.mean(), t.std()
    return bool((value.float() > mean + self.factor * std).item())

  def step(self, grad_scale, lr, step, loss=None, grad_norm=None, **kw):
    spike = False
    if loss is not None and grad_norm is not None and len(self.hist_loss) >= self.interval:
      spike = self._is_spike(self.hist_loss, loss) or self._is_spike(self.hist_norm, grad_norm)
    if loss is not None:
      self.hist_loss.append(loss.detach().clone())
      self.hist_norm.append(grad_norm.detach().clone())
      self.hist_loss, self.hist_norm = self.hist_loss[-self.interval:], self.hist_norm[-self.interval:]
    if spike:
      self.skipped += 1
      return {"learning/skipped_step": torch.ones(())}
    out = self.inner.step(grad_scale, lr, step, loss=loss, grad_norm=grad_norm, **kw)
    out["learning/skipped_step"] = torch.zeros(())
    return out

  def state_arrays(self):
    return self.inner.state_arrays()


def make_optimizer(config, store, model):
  t = config.opt_type
  if t == "adamw":
    opt = AdamW(config, store, model)
  elif t == "adam_pax":
    opt = AdamW(config, store, model, pax=True)
  elif t == "sgd":
    opt = SGD(config, store, model)
  elif t == "muon":
    from .muon import Muon
    opt = Muon(config, store, model)
  else:
    raise ValueError(t)
  if config.skip_step_on_spikes:
    opt = SkipOnSpikes(opt, config.skip_step_interval, config.skip_step_scaling_factor)
  return opt
