"""Adapter for lm-evaluation-harness (src/maxtext/eval/runner/harness_runner.py): an `LM`-shaped object over this
repository's engine, so `lm_eval.simple_evaluate(model=MaxTextLM(backend), tasks=[...])` scores a checkpoint with the
harness's own task definitions. The harness is an optional dependency: without it the class still works stand-alone
(requests are anything with an `.args` tuple), which is how the tests drive it.

  loglikelihood(requests)          (context, continuation) -> (sum log p, is the continuation the greedy choice)
  loglikelihood_rolling(requests)  (text,) -> sum log p of the whole text
  generate_until(requests)         (context, {"until": [...], "max_gen_toks": n}) -> generated text, cut at a stop string
"""
from __future__ import annotations

import torch

try:                                             # pragma: no cover - optional dependency
  from lm_eval.api.model import LM as _Base
except Exception:  # pylint: disable=broad-except
  _Base = object


class MaxTextLM(_Base):
  def __init__(self, backend, max_gen_toks: int = 256):
    if _Base is not object:
      super().__init__()
    self.backend, self.max_gen_toks = backend, int(max_gen_toks)

  @staticmethod
  def _args(r):
    return r.args if hasattr(r, "args") else tuple(r)

  @torch.no_grad()
  def _score(self, context: str, continuation: str):
    b = self.backend
    ctx_ids = b._ids(context) if context else [0]                      # pylint: disable=protected-access
    cont_ids = b._ids(continuation, bos=False) or [0]                  # pylint: disable=protected-access
    ids = (ctx_ids + cont_ids)[-int(b.c.max_target_length):]
    n = min(len(cont_ids), len(ids) - 1)
    t = torch.tensor(ids, device=b.engine.device)[None]
    logp = torch.log_softmax(b.engine.model.forward(t)[0].float()[:-1], -1)
    tail = logp[-n:]
    tgt = t[0, 1:][-n:]
    return float(tail.gather(1, tgt[:, None]).sum()), bool((tail.argmax(-1) == tgt).all())

  def loglikelihood(self, requests):
    return [self._score(*self._args(r)[:2]) for r in requests]

  def loglikelihood_rolling(self, requests):
    out = []
    for r in requests:
      text = self._args(r)[0]
      head, _, rest = text.partition(" ")
      out.append(self._score(head, (" " + rest) if rest else "")[0])
    return out

  def generate_until(self, requests):
    out = []
    for r in requests:
      context, opts = (self._args(r) + ({},))[:2]
      opts = opts or {}
      until = opts.get("until") or []
      until = [until] if isinstance(until, str) else list(until)
      text = self.backend.generate([context], int(opts.get("max_gen_toks", self.max_gen_toks)))[0]
      for s in until:
        if s and s in text:
          text = text[: text.index(s)]
      out.append(text)
    return out


def run_harness(backend, tasks: list[str], **kw):
  """`lm_eval.simple_evaluate` with this adapter; raises ImportError when the harness is not installed."""
  import lm_eval
  return lm_eval.simple_evaluate(model=MaxTextLM(backend), tasks=tasks, **kw)
