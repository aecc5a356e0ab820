"""Scorers (src/maxtext/eval/scoring/{registry,rouge_scorer}.py): ROUGE-1 / 2 / L F-measures, exact match, accuracy."""
from __future__ import annotations

import re
from collections import Counter
from typing import Callable

SCORERS: dict[str, Callable] = {}


def register_scorer(name: str):
  def deco(fn):
    SCORERS[name] = fn
    return fn
  return deco


def _tokens(s: str) -> list[str]:
  return re.findall(r"[a-z0-9]+", s.lower())


def _f(p: float, r: float) -> float:
  return 2 * p * r / (p + r) if p + r > 0 else 0.0


def _ngram_f(pred: list[str], ref: list[str], n: int) -> float:
  a = Counter(tuple(pred[i:i + n]) for i in range(len(pred) - n + 1))
  b = Counter(tuple(ref[i:i + n]) for i in range(len(ref) - n + 1))
  hit = sum((a & b).values())
  return _f(hit / max(1, sum(a.values())), hit / max(1, sum(b.values())))


def _lcs(a: list[str], b: list[str]) -> int:
  prev = [0] * (len(b) + 1)
  for x in a:
    cur = [0]
    for j, y in enumerate(b):
      cur.append(prev[j] + 1 if x == y else max(prev[j + 1], cur[j]))
    prev = cur
  return prev[-1]


@register_scorer("rouge")
def rouge(predictions: list[str], references: list[str]) -> dict:
  """Mean ROUGE-1, ROUGE-2 and ROUGE-L F-measures (x100, the MLPerf reporting convention) over the pairs."""
  r1 = r2 = rl = 0.0
  for p, r in zip(predictions, references):
    pt, rt = _tokens(p), _tokens(r)
    r1 += _ngram_f(pt, rt, 1)
    r2 += _ngram_f(pt, rt, 2)
    l = _lcs(pt, rt)
    rl += _f(l / max(1, len(pt)), l / max(1, len(rt)))
  n = max(1, len(predictions))
  return {"rouge1": 100 * r1 / n, "rouge2": 100 * r2 / n, "rougeL": 100 * rl / n, "samples": len(predictions)}


def _last_number(s: str) -> str | None:
  m = re.findall(r"-?\d+(?:[.,]\d+)*", s)
  return m[-1].replace(",", "") if m else None


@register_scorer("exact_match")
def exact_match(predictions: list[str], references: list[str], numeric: bool = False) -> dict:
  """Share of predictions equal to the reference after normalisation; `numeric` compares the last number in each
  (the GSM8K convention, where the reference ends in `#### 42`)."""
  hit = 0
  for p, r in zip(predictions, references):
    if numeric:
      hit += int(_last_number(p) is not None and _last_number(p) == _last_number(r))
    else:
      pn, rn = " ".join(_tokens(p)), " ".join(_tokens(r))
      hit += int(pn == rn or (bool(rn) and pn.startswith(rn + " ")))
  return {"exact_match": hit / max(1, len(predictions)), "samples": len(predictions)}


@register_scorer("accuracy")
def accuracy(predictions: list[int], references: list[int]) -> dict:
  return {"accuracy": sum(int(p == r) for p, r in zip(predictions, references)) / max(1, len(predictions)), "samples": len(predictions)}
