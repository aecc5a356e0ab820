"""Serving front end: `python -m maxtext_b200.inference.maxengine_server <yml> model_name=... [port=9000]`.

The reference exposes MaxEngine through a JetStream gRPC server (src/maxtext/inference/maxengine/maxengine_server.py:105) and a
small OpenAI-style HTTP server (benchmarks/api_server/). Here one process owns the decode engine and a continuous-batching
loop (`OfflineEngine`) in a background thread; HTTP handlers only enqueue requests and wait for their result, so any number of
clients share the decode slots.

  POST /v1/completions        {"prompt": "..." | ["...", "..."], "max_tokens": 32}      or {"prompt_tokens": [1, 2, 3], ...}
  POST /v1/chat/completions   {"messages": [{"role": "user", "content": "..."}], "max_tokens": 32}   (benchmarks/api_server/maxtext_server.py:144-156)
  GET  /v1/health
A list of prompts is served as one request with one choice per prompt; the prompts share the decode slots like any others.
Chat messages are rendered with the configured chat template (`chat_template`, `chat_template_path`) and the generation prompt.
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

  def _generate_many(self, token_lists, max_tokens: int, timeout: float):
    """Submit every prompt at once (they share the slots), wait for all: [(prompt tokens, output tokens, token limit)]."""
    items = []
    for toks in token_lists:
      toks = toks[-int(self.config.max_prefill_predict_length):] or [0]
      max_new = max(1, min(int(max_tokens), int(self.config.max_target_length) - len(toks) - 1))
      items.append((toks, max_new, self.submit(toks, max_new)))
    deadline = time.perf_counter() + timeout
    for _, _, it in items:
      if not it["event"].wait(max(0.0, deadline - time.perf_counter())):
        raise TimeoutError("generation timed out")
    return [(toks, it["request"].output, max_new) for toks, max_new, it in items]

  def complete(self, body: dict, timeout: float = 600.0) -> dict:
    if "prompt_tokens" in body:
      pt = body["prompt_tokens"]
      prompts = [[int(t) for t in p] for p in pt] if pt and isinstance(pt[0], (list, tuple)) else [[int(t) for t in pt]]
    else:
      raw = body.get("prompt", "")
      prompts = [self.tok.encode(str(p), add_bos=bool(self.config.add_bos)) for p in (raw if isinstance(raw, (list, tuple)) else [raw])]
    t0 = time.perf_counter()
    res = self._generate_many(prompts, int(body.get("max_tokens", 32)), timeout)
    return {"object": "text_completion", "model": self.config.model_name,
            "choices": [{"index": i, "text": self.tok.decode(out), "tokens": out, "finish_reason": "length" if len(out) >= mx else "stop"}
                        for i, (_, out, mx) in enumerate(res)],
            "usage": {"prompt_tokens": sum(len(t) for t, _, _ in res), "completion_tokens": sum(len(o) for _, o, _ in res),
                      "total_tokens": sum(len(t) + len(o) for t, o, _ in res)},
            "latency_s": round(time.perf_counter() - t0, 4)}

  def chat(self, body: dict, timeout: float = 600.0) -> dict:
    """OpenAI-style chat completion: the messages are rendered with the chat template plus the generation prompt."""
    from ..input_pipeline import chat as chat_lib
    msgs = body.get("messages")
    if not isinstance(msgs, list) or not msgs or not all(isinstance(m, dict) and "role" in m and "content" in m for m in msgs):
      raise ValueError("`messages` must be a non-empty list of {role, content}")
    text = chat_lib.render(msgs, chat_lib.load_template(self.config), add_generation_prompt=True)
    t0 = time.perf_counter()
    toks, out, mx = self._generate_many([self.tok.encode(text, add_bos=bool(self.config.add_bos))], int(body.get("max_tokens", 32)), timeout)[0]
    return {"object": "chat.completion", "model": self.config.model_name,
            "choices": [{"index": 0, "message": {"role": "assistant", "content": self.tok.decode(out)},
                         "finish_reason": "length" if len(out) >= mx else "stop"}],
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

  @app.post("/v1/chat/completions")
  def chat_completions(body: dict):
    try:
      return loop.chat(body)
    except ValueError as e:
      raise HTTPException(status_code=400, detail=str(e)) from e
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
