"""Goodput-style event log: how wall time splits into job / init / data loading / step.

Replaces the ml-goodput-measurement recorder used by src/maxtext/common/goodput.py:31-140 with a local
JSONL event stream (same event names: JOB, TPU_INIT -> DEVICE_INIT, TRAINING_PREPARATION, DATA_LOADING,
STEP) plus a step-time-deviation monitor.
"""
from __future__ import annotations

import contextlib
import json
import os
import time


class Recorder:
  def __init__(self, path: str | None, enabled: bool):
    self.enabled = enabled and bool(path)
    self.fh = open(path, "a", encoding="utf-8") if self.enabled else None
    self.totals: dict[str, float] = {}
    self.t_job = time.time()
    self.step_times: list[float] = []

  @contextlib.contextmanager
  def span(self, event: str, step: int | None = None):
    t0 = time.time()
    try:
      yield
    finally:
      dt = time.time() - t0
      self.totals[event] = self.totals.get(event, 0.0) + dt
      if event == "STEP":
        self.step_times.append(dt)
      if self.fh:
        self.fh.write(json.dumps({"event": event, "step": step, "start": t0, "seconds": dt}) + "\n")

  def goodput(self) -> float:
    """Fraction of job wall time spent inside productive steps."""
    total = max(time.time() - self.t_job, 1e-9)
    return self.totals.get("STEP", 0.0) / total

  def step_time_deviation(self) -> float:
    if len(self.step_times) < 3:
      return 0.0
    s = sorted(self.step_times)
    med = s[len(s) // 2]
    return max(abs(t - med) for t in self.step_times[-10:]) / max(med, 1e-9)

  def close(self):
    if self.fh:
      self.fh.write(json.dumps({"event": "JOB", "seconds": time.time() - self.t_job, "goodput": self.goodput()}) + "\n")
      self.fh.close()
      self.fh = None


def create_recorder(config, rank: int = 0) -> Recorder:
  enabled = bool(config.enable_goodput_recording) and rank == 0
  path = os.path.join(config.metrics_dir, "goodput.jsonl") if (enabled and config.metrics_dir) else None
  if path:
    os.makedirs(os.path.dirname(path), exist_ok=True)
  return Recorder(path, enabled)
