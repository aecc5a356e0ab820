"""Prefill / generate micro-benchmark (src/maxtext/inference/inference_microbenchmark.py): device-timed latency per
prefill length and per generate step, tokens/s, KV-cache bytes."""
from __future__ import annotations

import json
import sys
import time

import torch

from ..config import pyconfig
from .maxengine import MaxEngine


def _time(fn, iters, cuda):
  fn()
  if cuda:
    torch.cuda.synchronize()
  t0 = time.perf_counter()
  for _ in range(iters):
    fn()
  if cuda:
    torch.cuda.synchronize()
  return (time.perf_counter() - t0) / iters


def run(config, engine: MaxEngine | None = None) -> dict:
  eng = engine or MaxEngine(config)
  if engine is None:
    eng.load_params()
  cuda = eng.device.type == "cuda"
  iters = int(config.inference_microbenchmark_loop_iters)
  out = {"prefill": {}, "generate": {}}
  stages = config.inference_microbenchmark_stages.split(",")
  if "prefill" in stages:
    for n in [int(x) for x in str(config.inference_microbenchmark_prefill_lengths).split(",")]:
      if n > config.max_prefill_predict_length:
        continue
      toks = torch.randint(1, config.vocab_size, (n,))
      dt = _time(lambda: eng.prefill(toks, n), iters, cuda)
      from ..utils import flops
      n_par = sum(p.pdef.numel for p in eng.model.all_params())
      tf = flops.prefill_tflops_per_device(config, n_par, n)[0]
      out["prefill"][n] = {"ms": dt * 1e3, "tokens_per_s": n / dt, "tflops": tf, "tflops_per_s": tf / dt}
  if "generate" in stages:
    slots = max(1, int(config.per_device_batch_size))
    state = eng.init_decode_state(slots)
    toks = torch.randint(1, config.vocab_size, (min(16, int(config.max_prefill_predict_length)),))
    for s in range(slots):
      p, _ = eng.prefill(toks, toks.numel())
      state = eng.insert(p, state, s)
    holder = {"s": state}
    def step():
      holder["s"], _ = eng.generate(holder["s"])
    dt = _time(step, iters, cuda)
    cache_bytes = sum(t.numel() * t.element_size() for layer in state.caches for cc in layer for t in vars(cc).values() if isinstance(t, torch.Tensor))
    out["generate"] = {"ms_per_step": dt * 1e3, "tokens_per_s": slots / dt, "slots": slots, "kv_cache_bytes": cache_bytes}
  return out


def main(argv=None):
  config = pyconfig.initialize(list(sys.argv if argv is None else argv))
  res = run(config)
  print(json.dumps(res))
  if config.inference_microbenchmark_log_file_path:
    with open(config.inference_microbenchmark_log_file_path, "w") as fh:
      json.dump(res, fh)
  return res


if __name__ == "__main__":
  main()
