"""Learning-rate schedules: linear warm-up, cosine or warmup-stable-decay, optional zero tail.

Same piecewise definition as src/maxtext/utils/maxtext_utils.py:2283-2351; each piece sees the step
count relative to its own start (optax.join_schedules semantics).
"""
from __future__ import annotations

import math


def _cosine(init_lr, final_lr, n):
  def f(step):
    pct = step / (n - 1) if n > 1 else 1.0
    a = 0.5 * (math.cos(math.pi * pct) + 1.0)
    return init_lr * a + final_lr * (1.0 - a)
  return f


def _linear(a, b, n):
  def f(step):
    if n <= 0:
      return b
    t = min(max(step / n, 0.0), 1.0)
    return a + (b - a) * t
  return f


def make_schedule(config):
  lr = float(config.learning_rate)
  final_lr = lr * float(config.learning_rate_final_fraction)
  total = int(config.learning_rate_schedule_steps)
  warm = int(total * float(config.warmup_steps_fraction))
  zero_tail = int(config.steps) - total
  pieces, bounds = [], []
  if warm > 0:
    pieces.append(_linear(0.0, lr, warm))
    bounds.append(warm)
  if config.lr_schedule_type == "cosine":
    n = total - warm
    if n > 0:
      pieces.append(_cosine(lr, final_lr, n))
      bounds.append(warm + n)
  else:
    decay = int(total * float(config.wsd_decay_steps_fraction))
    stable = total - warm - decay
    if stable > 0:
      pieces.append(lambda s: lr)
      bounds.append(warm + stable)
    if decay > 0:
      pieces.append(_linear(lr, final_lr, decay - 1) if config.wsd_decay_style == "linear" else _cosine(lr, final_lr, decay))
      bounds.append(warm + max(stable, 0) + decay)
  if zero_tail > 0:
    pieces.append(lambda s: 0.0)
  if not pieces:
    return lambda step: lr

  def schedule(step: int) -> float:
    start = 0
    for i, p in enumerate(pieces):
      end = bounds[i] if i < len(bounds) and i < len(pieces) - 1 else None
      if end is None or step < end:
        return float(p(step - start))
      start = end
    return float(pieces[-1](step - start))

  return schedule
