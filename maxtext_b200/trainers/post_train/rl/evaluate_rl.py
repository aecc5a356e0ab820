"""Held-out evaluation for the RL trainer: greedy answers to each question, scored for answer correctness and for
format (src/maxtext/trainers/post_train/rl/evaluate_rl.py:51-300: generate_responses / score_responses / evaluate)."""
from __future__ import annotations

import json

from . import math_verify_pool as mvp
from . import rewards as R


def score_response(c, response: str, answers: list[str]) -> tuple[bool, bool]:
  """(answer correct, format correct) for one response."""
  fmt = R.match_format_regex(c).search(response) is not None
  guess = R.extract_answer(response, c)
  if guess == R.FALLBACK_ANSWER:
    return False, fmt
  golds = [R.boxed(R.preprocess_math_string(a)) for a in answers]
  return mvp.verify_math_worker(golds, [R.boxed(R.preprocess_math_string(guess))]) > 0, fmt


def evaluate(trainer, rows: list[dict]) -> dict:
  prompts = [trainer._encode_prompt(r["question"]) for r in rows]          # pylint: disable=protected-access
  comps = trainer.greedy.generate(prompts, trainer.max_new)
  n_ok = n_fmt = 0
  for r, cm in zip(rows, comps):
    ok, fmt = score_response(trainer.c, trainer.tok.decode(cm), json.loads(r["answer"]))
    n_ok += int(ok)
    n_fmt += int(fmt)
  n = max(1, len(rows))
  return {"accuracy": n_ok / n, "format_accuracy": n_fmt / n, "num_questions": len(rows)}
