"""Step metrics: console line, JSONL file, optional TensorBoard, optional Prometheus endpoint (`prometheus_port`).

Follows src/maxtext/common/metric_logger.py:91-510: the metrics of step n are written while step
n+1 runs (the device tensors are read one step late, so logging never stalls the GPU), the console
line has the reference's shape (`completed step: N, seconds: ..., TFLOP/s/device: ..., Tokens/s/device:
..., total_weights: ..., loss: ...`), `metrics_file` receives one JSON object per step, and a NaN/Inf
loss aborts after the metrics are flushed (metric_logger.py:294-302).
"""
from __future__ import annotations

import json
import math
import os

import torch

from . import flops, max_logging


class TrainingAborted(RuntimeError):
  pass


class MetricLogger:
  def __init__(self, config, is_writer: bool = True):
    self.c = config
    self.is_writer = is_writer
    self.pending = None
    self.tflops, _, _ = flops.training_tflops_per_device(config)
    self.tokens = flops.tokens_per_device(config)
    self.file = None
    if is_writer and config.metrics_file:
      os.makedirs(os.path.dirname(os.path.abspath(config.metrics_file)), exist_ok=True)
      self.file = open(config.metrics_file, "a", encoding="utf-8")
    self.tb = None
    if is_writer and config.enable_tensorboard and config.tensorboard_dir:
      try:
        from torch.utils.tensorboard import SummaryWriter
        self.tb = SummaryWriter(config.tensorboard_dir)
      except Exception:  # tensorboard is optional
        self.tb = None
    self.history = []
    self.prom = None
    port = int(getattr(config, "prometheus_port", 0) or 0)
    if is_writer and port > 0:
      # one gauge per metric (slashes are not legal in Prometheus names), served from a daemon thread on `port`
      import prometheus_client
      self.prom_registry = prometheus_client.CollectorRegistry()
      prometheus_client.start_http_server(port, registry=self.prom_registry)
      self.prom = {}

  def _export(self, scal):
    import prometheus_client
    for k, v in scal.items():
      name = "maxtext_" + "".join(ch if ch.isalnum() else "_" for ch in k)
      g = self.prom.get(name)
      if g is None:
        g = self.prom[name] = prometheus_client.Gauge(name, k, registry=self.prom_registry)
      g.set(v)

  def record(self, step: int, metrics: dict, step_time_s: float):
    """Buffer this step's (device) metrics; write the previous step's."""
    prev = self.pending
    self.pending = (step, metrics, step_time_s)
    if prev is not None:
      self._write(*prev)

  def flush(self):
    if self.pending is not None:
      prev, self.pending = self.pending, None
      self._write(*prev)
    if self.file:
      self.file.flush()
    if self.tb:
      self.tb.flush()

  def _write(self, step, metrics, dt):
    scal = {}
    for k, v in metrics.items():
      scal[k] = float(v.item()) if isinstance(v, torch.Tensor) else float(v)
    scal["perf/step_time_seconds"] = dt
    scal["perf/per_device_tflops"] = self.tflops
    scal["perf/per_device_tflops_per_sec"] = self.tflops / max(dt, 1e-9)
    scal["perf/per_device_tokens"] = self.tokens
    scal["perf/per_device_tokens_per_sec"] = self.tokens / max(dt, 1e-9)
    if "learning/lm_loss" in scal:
      scal["learning/perplexity"] = math.exp(min(scal["learning/lm_loss"], 50.0))
    scal["step"] = step
    self.history.append(scal)
    if self.is_writer:
      max_logging.log(
          f"completed step: {step}, seconds: {dt:.3f}, TFLOP/s/device: {scal['perf/per_device_tflops_per_sec']:.3f}, "
          f"Tokens/s/device: {scal['perf/per_device_tokens_per_sec']:.3f}, "
          f"total_weights: {int(scal.get('learning/total_weights', 0))}, loss: {scal.get('learning/loss', float('nan')):.3f}")
      if self.file:
        self.file.write(json.dumps(scal) + "\n")
      if self.prom is not None:
        self._export(scal)
      if self.tb and step % max(1, self.c.log_period) == 0:
        for k, v in scal.items():
          self.tb.add_scalar(k, v, step)
    loss = scal.get("learning/loss")
    if loss is not None:
      if (self.c.abort_on_nan_loss and math.isnan(loss)) or (self.c.abort_on_inf_loss and math.isinf(loss)):
        self.flush()
        raise TrainingAborted(f"loss is {loss} at step {step}")

  def close(self):
    self.flush()
    if self.file:
      self.file.close()
    if self.tb:
      self.tb.close()
