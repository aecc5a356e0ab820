"""Callbacks around a post-training run: what happens at the start and end of training, of every train step and of every
evaluation step, and where the batches come from.

The reference passes such hook objects to the Tunix trainer (src/maxtext/trainers/post_train/hooks.py:36-238,
sft/hooks.py, dpo/hooks.py, rl/hooks.py): the training hooks feed the metric logger and the goodput recorder and stop the
run when the target evaluation loss is reached; the data hooks own the train / eval iterators. Here the same two
interfaces drive `run_with_hooks`, a loop over any stepper with a `train_step(batch)` method (the pre-training engine,
`DPOStepper`, a user's own objective), so the SFT / DPO / RL entry points share their bookkeeping."""
from __future__ import annotations

import math
import time

from ...input_pipeline import interface
from ...utils import max_logging
from ...utils.metric_logger import MetricLogger


class StopTraining(Exception):
  pass


class TrainingHooks:
  """Base class: every callback is optional."""

  def on_train_start(self, loop):
    pass

  def on_train_end(self, loop):
    pass

  def on_train_step_start(self, loop, step: int, batch):
    pass

  def on_train_step_end(self, loop, step: int, metrics: dict, step_time: float):
    pass

  def on_eval_step_start(self, loop, batch):
    pass

  def on_eval_step_end(self, loop, eval_loss_sum: float, eval_weights: float):
    pass


class DataHooks:
  """Owns the iterators. `load_next_eval_batch` returns None when the evaluation pass is over."""

  def __init__(self, config, data_rank: int = 0, data_world: int = 1, train_iterator=None, eval_iterator=None):
    self.config = config
    self.train_iterator = train_iterator or interface.create_data_iterator(config, data_rank, data_world)
    self._eval_factory = (lambda: eval_iterator) if eval_iterator is not None else \
        (lambda: interface.create_data_iterator(config, data_rank, data_world, split="eval"))
    self.eval_iterator = None
    self.train_batch = None
    self.eval_batch = None
    self._eval_count = 0

  def load_next_train_batch(self, loop):
    try:
      self.train_batch = next(self.train_iterator)
    except StopIteration:
      self.train_batch = None
    return self.train_batch

  def load_next_eval_batch(self, loop):
    c = self.config
    if self.eval_iterator is None:
      self.eval_iterator, self._eval_count = self._eval_factory(), 0
    if int(c.eval_steps) > 0 and self._eval_count >= int(c.eval_steps):
      self.eval_iterator, self.eval_batch = None, None
      return None
    try:
      self.eval_batch = next(self.eval_iterator)
      self._eval_count += 1
    except StopIteration:
      self.eval_iterator, self.eval_batch = None, None
    return self.eval_batch


def _total_weights(batch) -> float:
  """Number of target tokens that carry loss in a batch."""
  if batch is None:
    return 0.0
  if "loss_weights" in batch:
    return float(batch["loss_weights"].float().sum())
  if "targets_segmentation" in batch:
    return float((batch["targets_segmentation"] != 0).sum())
  if "targets" in batch:
    return float(batch["targets"].numel())
  return float(len(batch.get("prompts", ())))


class MetricTrainingHooks(TrainingHooks):
  """The shared bookkeeping (hooks.py:36-190): step timing, train / eval metrics to the metric logger under the
  reference's names, perplexity, and `target_eval_loss` as a stop condition."""

  def __init__(self, config, is_writer: bool = True, logger: MetricLogger | None = None):
    self.config = config
    self.logger = logger or MetricLogger(config, is_writer=is_writer)
    self.first_step = None
    self.train_weights = {}
    self.eval_steps = 0
    self.history = []

  def on_train_start(self, loop):
    self.first_step = loop.step

  def on_train_end(self, loop):
    assert self.first_step is not None, "on_train_start() must run before on_train_end()"
    self.logger.close()

  def on_train_step_start(self, loop, step, batch):
    self.train_weights[step] = _total_weights(batch)

  def on_train_step_end(self, loop, step, metrics, step_time):
    assert step in self.train_weights, "on_train_step_start() must run before on_train_step_end()"
    m = dict(metrics)
    m.setdefault("learning/total_weights", self.train_weights.pop(step))
    if "learning/loss" in m:
      try:
        m.setdefault("learning/perplexity", math.exp(min(float(m["learning/loss"]), 80.0)))
      except (TypeError, ValueError):
        pass
    self.history.append((step, {k: float(v) for k, v in m.items() if _is_number(v)}))
    self.logger.record(step, m, step_time)

  def on_eval_step_start(self, loop, batch):
    self.eval_steps += 1

  def on_eval_step_end(self, loop, eval_loss_sum, eval_weights):
    assert self.eval_steps > 0, "on_eval_step_start() must run before on_eval_step_end()"
    avg = eval_loss_sum / max(eval_weights, 1e-8)
    out = {"eval/total_loss": eval_loss_sum, "eval/avg_loss": avg, "eval/total_weights": eval_weights,
           "eval/avg_perplexity": math.exp(min(avg, 80.0))}
    max_logging.log(f"eval after step {loop.step}: " + ", ".join(f"{k}: {v:.4f}" for k, v in out.items()))
    self.history.append((loop.step, out))
    self.eval_steps = 0
    if float(self.config.target_eval_loss) > 0 and avg <= float(self.config.target_eval_loss):
      raise StopTraining(f"target_eval_loss={self.config.target_eval_loss} reached")


def _is_number(v) -> bool:
  try:
    float(v)
    return True
  except (TypeError, ValueError):
    return False


class HookedLoop:
  """`steps` train steps of `stepper` with the callbacks of `hooks` and the batches of `data`; evaluation every
  `eval_interval` steps through `eval_fn(batch) -> (loss_sum, weights)` when one is given."""

  def __init__(self, config, stepper, hooks: TrainingHooks, data: DataHooks, eval_fn=None, start_step: int = 0):
    self.config, self.stepper, self.hooks, self.data, self.eval_fn = config, stepper, hooks, data, eval_fn
    self.step = int(start_step)

  def evaluate(self):
    tot, w = 0.0, 0.0
    while True:
      batch = self.data.load_next_eval_batch(self)
      if batch is None:
        break
      self.hooks.on_eval_step_start(self, batch)
      a, b = self.eval_fn(batch)
      tot, w = tot + float(a), w + float(b)
    self.hooks.on_eval_step_end(self, tot, w)

  def run(self):
    c = self.config
    self.hooks.on_train_start(self)
    try:
      while self.step < int(c.steps):
        batch = self.data.load_next_train_batch(self)
        if batch is None:
          break
        self.hooks.on_train_step_start(self, self.step, batch)
        t0 = time.perf_counter()
        metrics = self.stepper.train_step(batch)
        self.hooks.on_train_step_end(self, self.step, metrics, time.perf_counter() - t0)
        self.step += 1
        if self.eval_fn is not None and int(c.eval_interval) > 0 and self.step % int(c.eval_interval) == 0:
          self.evaluate()
    except StopTraining as e:
      max_logging.log(f"training stopped: {e}")
    finally:
      self.hooks.on_train_end(self)
    return self.step


def run_with_hooks(config, stepper, hooks: TrainingHooks | None = None, data: DataHooks | None = None, eval_fn=None, start_step: int = 0):
  hooks = hooks or MetricTrainingHooks(config)
  data = data or DataHooks(config)
  return HookedLoop(config, stepper, hooks, data, eval_fn, start_step).run()
