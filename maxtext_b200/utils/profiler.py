"""Profiler window control (src/maxtext/common/profiler.py:32-167).

`profiler=nsys` brackets the window with cudaProfilerStart/Stop so that a job launched under
`nsys profile --capture-range=cudaProfilerApi` records exactly those steps; `profiler=xplane` writes a
Chrome/TensorBoard trace with torch.profiler. Steps are also wrapped in NVTX ranges `train/step_N`.
"""
from __future__ import annotations

import os

import torch


class Profiler:
  def __init__(self, config, rank: int = 0):
    self.c = config
    self.mode = config.profiler
    self.active = False
    self.enabled = bool(self.mode) and (rank == 0 or config.upload_all_profiler_results)
    self.first = int(config.skip_first_n_steps_for_profiler)
    self.n = int(config.profiler_steps)
    self.period = int(config.profile_periodically_period)
    self.tp = None
    self.out_dir = os.path.join(config.tensorboard_dir or "/tmp/maxtext_b200_profile", "profile")
    self._nvtx = torch.cuda.is_available()

  def _window_start(self, step):
    if self.period > 0:
      return step >= self.first and (step - self.first) % self.period == 0
    return step == self.first

  def maybe_start(self, step):
    if self._nvtx:
      torch.cuda.nvtx.range_push(f"train/step_{step}")
    if not self.enabled or self.active or not self._window_start(step):
      return
    if self.c.profile_cleanly and torch.cuda.is_available():
      torch.cuda.synchronize()
    if self.mode == "nsys" and torch.cuda.is_available():
      torch.cuda.profiler.start()
    elif self.mode == "xplane":
      acts = [torch.profiler.ProfilerActivity.CPU]
      if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
      self.tp = torch.profiler.profile(activities=acts)
      self.tp.__enter__()
    self.active, self.start_step = True, step

  def maybe_stop(self, step):
    if self._nvtx:
      torch.cuda.nvtx.range_pop()
    if not self.active or step < self.start_step + self.n - 1:
      return
    self._stop()

  def _stop(self):
    if self.c.profile_cleanly and torch.cuda.is_available():
      torch.cuda.synchronize()
    if self.mode == "nsys" and torch.cuda.is_available():
      torch.cuda.profiler.stop()
    elif self.tp is not None:
      self.tp.__exit__(None, None, None)
      os.makedirs(self.out_dir, exist_ok=True)
      self.tp.export_chrome_trace(os.path.join(self.out_dir, f"trace_step{self.start_step}.json"))
      self.tp = None
    self.active = False

  def close(self):
    if self.active:
      self._stop()
