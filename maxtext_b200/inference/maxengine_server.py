"""Serving front end: `python -m maxtext_b200.inference.maxengine_server <yml> model_name=... [port=9000]`.

The reference exposes MaxEngine through a JetStream gRPC server (src/maxtext/inference/maxengine/maxengine_server.py:105) and a
small OpenAI-style HTTP server (benchmarks/api_server/). Here one process owns the decode engine and a continuous-batching
loop (`OfflineEngine`) in a background thread; HTTP handlers only enqueue requests and wait for their result, so any number of
clients share the decode slots.

  POST /v1/completions   {"prompt": "...", "max_tokens": 32}      or {"prompt_tokens": [1, 2, 3], ...}
  GET  /v1/health
"""
from __future__ import annotations

import sys
import threading
import time

from ..config import pyconfig
from ..input_pipeline.tokenizer import build_tokenizer
from .maxengine import MaxEngine
from .offline_engine import OfflineEngine


class ServingLoop:
  """Owns the engine; `submit` is thread-safe, the loop thread is the only one that touches the device."""

  def __init__(self, config, engine: MaxEngine | None = None, tokenizer=None):
    self.config = config
    self.engine = engine or MaxEngine(config)
    if engine is None:
      self.engine.load_params()
    self.tok = tokenizer if tokenizer is not None else build_tokenizer(config)
    self.batcher = OfflineEngine(self.engine, slots=max(1, int(config.per_device_batch_size)), eos_id=getattr(self.tok, "eos_id", -1))
    self._lock = threading.Lock()
    self._pending = []
    self._stop = threading.Event()
    self._thread = None
    self.served = 0

  def start(self):
    self._thread = threading.Thread(target=self._run, daemon=True, name="decode-loop")
    self._thread.start()
    return self

  def stop(self):
    self._stop.set()
    if self._thread is not None:
      self._thread.join(timeout=10)

  def submit(self, tokens, max_new_tokens: int):
    done = threading.Event()
    item = {"tokens": list(tokens), "max_new": int(max_new_tokens), "event": done, "request": None}
    with self._lock:
      self._pending.append(item)
    return item

  def _run(self):
    inflight = []
    while not self._stop.is_set():
      with self._lock:
        new, self._pending = self._pending, []
      for it in new:
        it["request"] = self.batcher.submit(it["tokens"], it["max_new"])
        inflight.append(it)
      if self.batcher.queue or self.batcher.running:
        self.batcher.step()
      else:
        time.sleep(0.002)
      for it in list(inflight):
        if it["request"].done:
          it["event"].set()
          inflight.remove(it)
          self.served += 1

  def complete(self, body: dict, timeout: float = 600.0) -> dict:
    if "prompt_tokens" in body:
      toks = [int(t) for t in body["prompt_tokens"]]
    else:
      toks = self.tok.encode(str(body.get("prompt", "")), add_bos=bool(self.config.add_bos))
    toks = toks[-int(self.config.max_prefill_predict_length):] or [0]
    max_new = int(body.get("max_tokens", 32))
    max_new = max(1, min(max_new, int(self.config.max_target_length) - len(toks) - 1))
    t0 = time.perf_counter()
    item = self.submit(toks, max_new)
    if not item["event"].wait(timeout):
      raise TimeoutError("generation timed out")
    out = item["request"].output
    return {"object": "text_completion", "model": self.config.model_name,
            "choices": [{"index": 0, "text": self.tok.decode(out), "tokens": out, "finish_reason": "length" if len(out) >= max_new else "stop"}],
            "usage": {"prompt_tokens": len(toks), "completion_tokens": len(out), "total_tokens": len(toks) + len(out)},
            "latency_s": round(time.perf_counter() - t0, 4)}


def create_app(loop: ServingLoop):
  from fastapi import FastAPI, HTTPException
  app = FastAPI(title="maxtext_b200")

  @app.get("/v1/health")
  def health():
    return {"status": "ok", "served": loop.served, "slots": loop.batcher.slots, "running": len(loop.batcher.running)}

  @app.post("/v1/completions")
  def completions(body: dict):
    try:
      return loop.complete(body)
    except TimeoutError as e:
      raise HTTPException(status_code=504, detail=str(e)) from e

  return app


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  port = next((int(a.split("=", 1)[1]) for a in argv if a.startswith("port=")), 9000)
  argv = [a for a in argv if not a.startswith("port=")]
  config = pyconfig.initialize(argv)
  loop = ServingLoop(config).start()
  import uvicorn
  uvicorn.run(create_app(loop), host="127.0.0.1", port=port, log_level="warning")


if __name__ == "__main__":
  main()
