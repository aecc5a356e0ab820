"""Evaluation runner (src/maxtext/eval/runner/{run,eval_runner,async_client,common}.py, reporting/json_reporter.py).

    python -m maxtext_b200.eval.runner <config.yml> [key=value ...] --dataset jsonl --path data.jsonl --scorer rouge

Two backends produce the model's answers: `LocalBackend` drives this repository's inference engine in-process (slot
batching through `OfflineEngine`, log-likelihoods through the model's forward pass); `ServerBackend` is an asynchronous
client of a running `maxengine_server` (`/v1/completions`), many requests in flight, which is how a served model is
evaluated. Results go to a JSON report (per-sample predictions plus the aggregate metrics).
"""
from __future__ import annotations

import argparse
import asyncio
import json
import math
import os
import time

import torch

from .datasets import EvalSample, load_dataset
from .scoring import SCORERS


class LocalBackend:
  """In-process generation and scoring with a `MaxEngine`."""

  def __init__(self, config, engine=None, tokenizer=None, slots: int = 4):
    from ..inference.maxengine import MaxEngine
    from ..inference.offline_engine import OfflineEngine
    from ..input_pipeline.tokenizer import build_tokenizer
    self.c = config
    self.engine = engine or MaxEngine(config)
    if engine is None:
      self.engine.load_params()
    self.tok = tokenizer or build_tokenizer(config)
    self.offline = OfflineEngine(self.engine, slots=slots, eos_id=int(getattr(self.tok, "eos_id", -1) or -1))

  def _ids(self, text: str, bos: bool = True) -> list[int]:
    ids = self.tok.encode(text, add_bos=bos and bool(self.c.add_bos))
    return [i % self.c.vocab_size for i in ids]

  def generate(self, prompts: list[str], max_new_tokens: int) -> list[str]:
    lim = int(self.c.max_prefill_predict_length)
    outs = self.offline.batch_inference([self._ids(p)[-lim:] or [0] for p in prompts], max_new_tokens)
    return [self.tok.decode(o) for o in outs]

  @torch.no_grad()
  def loglikelihood(self, prompt: str, continuation: str) -> tuple[float, int]:
    """(sum of log p(continuation tokens | prompt), number of continuation tokens)."""
    a, b = self._ids(prompt), self._ids(continuation, bos=False)
    b = b or [0]
    ids = (a + b)[-int(self.c.max_target_length):]
    n = min(len(b), len(ids) - 1)
    t = torch.tensor(ids, device=self.engine.device)[None]
    logits = self.engine.model.forward(t)[0].float()
    lp = torch.log_softmax(logits[:-1], -1).gather(1, t[0, 1:, None])[:, 0]
    return float(lp[-n:].sum()), n


class ServerBackend:
  """Asynchronous client of `maxengine_server` (src/maxtext/eval/runner/async_client.py)."""

  def __init__(self, url: str, concurrency: int = 16, timeout_s: float = 600.0):
    self.url, self.concurrency, self.timeout_s = url.rstrip("/"), int(concurrency), float(timeout_s)

  async def _one(self, session, sem, prompt, max_new_tokens):
    async with sem:
      async with session.post(self.url + "/v1/completions", json={"prompt": prompt, "max_tokens": int(max_new_tokens)}) as r:
        r.raise_for_status()
        return (await r.json())["choices"][0]["text"]

  async def _all(self, prompts, max_new_tokens):
    import aiohttp
    sem = asyncio.Semaphore(self.concurrency)
    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout_s)) as session:
      return await asyncio.gather(*[self._one(session, sem, p, max_new_tokens) for p in prompts])

  def generate(self, prompts: list[str], max_new_tokens: int) -> list[str]:
    return list(asyncio.run(self._all(prompts, max_new_tokens)))

  def loglikelihood(self, prompt, continuation):
    raise NotImplementedError("the completions endpoint returns text only; multiple-choice tasks need the local backend")


class EvalRunner:
  def __init__(self, backend, max_new_tokens: int = 64):
    self.backend, self.max_new_tokens = backend, int(max_new_tokens)

  def run(self, samples: list[EvalSample], scorer: str | None = None, scorer_kwargs: dict | None = None) -> dict:
    t0 = time.perf_counter()
    kinds = {s.kind for s in samples}
    assert len(kinds) == 1, f"one task kind per run, got {sorted(kinds)}"
    kind = kinds.pop()
    records = []
    if kind == "generate":
      preds = self.backend.generate([s.prompt for s in samples], self.max_new_tokens)
      metrics = SCORERS[scorer or "rouge"](preds, [s.reference for s in samples], **(scorer_kwargs or {}))
      records = [{"prompt": s.prompt, "prediction": p, "reference": s.reference} for s, p in zip(samples, preds)]
    elif kind == "choice":
      picks = []
      for s in samples:
        scores = []
        for ch in s.choices:
          ll, n = self.backend.loglikelihood(s.prompt, " " + ch)
          scores.append(ll / max(1, n))                       # length-normalised, the lm-eval `acc_norm` convention
        picks.append(int(max(range(len(scores)), key=scores.__getitem__)))
        records.append({"prompt": s.prompt, "choices": s.choices, "scores": scores, "prediction": picks[-1], "answer": s.answer})
      metrics = SCORERS["accuracy"](picks, [s.answer for s in samples])
    elif kind == "perplexity":
      nll, toks = 0.0, 0
      for s in samples:
        words = s.prompt.split(" ", 1)
        ll, n = self.backend.loglikelihood(words[0], " " + words[1] if len(words) > 1 else "")
        nll, toks = nll - ll, toks + n
        records.append({"prompt": s.prompt, "nll": -ll, "tokens": n})
      metrics = {"perplexity": math.exp(nll / max(1, toks)), "nll_per_token": nll / max(1, toks), "tokens": toks, "samples": len(samples)}
    else:
      raise ValueError(f"unknown task kind {kind!r}")
    metrics["seconds"] = round(time.perf_counter() - t0, 3)
    return {"task": kind, "metrics": metrics, "records": records}


def write_report(result: dict, directory: str, name: str = "eval") -> str:
  """JSON reporter: `<directory>/<name>_results.json` (metrics) and `<name>_samples.jsonl` (one record per sample)."""
  os.makedirs(directory, exist_ok=True)
  path = os.path.join(directory, f"{name}_results.json")
  with open(path, "w", encoding="utf-8") as fh:
    json.dump({"task": result["task"], "metrics": result["metrics"]}, fh, indent=1)
  with open(os.path.join(directory, f"{name}_samples.jsonl"), "w", encoding="utf-8") as fh:
    for r in result["records"]:
      fh.write(json.dumps(r) + "\n")
  return path


def main(argv=None):
  ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
  ap.add_argument("config", nargs="+", help="config.yml followed by key=value overrides")
  ap.add_argument("--dataset", default="synthetic_copy")
  ap.add_argument("--path", default="")
  ap.add_argument("--kind", default=None, choices=[None, "generate", "choice", "perplexity"])
  ap.add_argument("--scorer", default=None)
  ap.add_argument("--numeric", action="store_true", help="exact_match on the last number (GSM8K style)")
  ap.add_argument("--num_samples", type=int, default=None)
  ap.add_argument("--max_new_tokens", type=int, default=64)
  ap.add_argument("--server", default="", help="URL of a running maxengine_server; empty evaluates in-process")
  ap.add_argument("--concurrency", type=int, default=16)
  ap.add_argument("--slots", type=int, default=4)
  ap.add_argument("--output", default="")
  a = ap.parse_args(argv)
  from ..config import pyconfig
  cfg = pyconfig.initialize(["eval"] + a.config, num_devices=1)
  kw = {k: v for k, v in (("path", a.path), ("num_samples", a.num_samples), ("kind", a.kind)) if v not in ("", None)}
  samples = load_dataset(a.dataset, **kw)
  backend = ServerBackend(a.server, a.concurrency) if a.server else LocalBackend(cfg, slots=a.slots)
  res = EvalRunner(backend, a.max_new_tokens).run(samples, a.scorer, {"numeric": True} if a.numeric else None)
  out = a.output or os.path.join(cfg.base_output_directory or ".", cfg.run_name or "eval", "eval")
  path = write_report(res, out)
  print(json.dumps({"report": path, **res["metrics"]}))
  return res


if __name__ == "__main__":
  main()
