"""Evaluation datasets (src/maxtext/eval/datasets/{base,registry,mlperf}.py).

A dataset yields `EvalSample`s. Three task kinds are understood by the runner:
  generate   prompt -> free text, scored against `reference` (ROUGE, exact match)
  choice     prompt + `choices` -> the choice with the highest length-normalised log-likelihood, scored against `answer`
  perplexity `prompt` alone -> token-level negative log-likelihood
Files are JSON lines; the field names of common public sets (question / input / prompt, output / reference / answer,
choices / options) are mapped on load, so an exported MMLU-, GSM8K- or OpenOrca-style file can be used as it is.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Callable, Iterable


@dataclass
class EvalSample:
  prompt: str
  reference: str = ""
  choices: list = field(default_factory=list)
  answer: int = -1
  kind: str = "generate"
  meta: dict = field(default_factory=dict)


DATASETS: dict[str, Callable[..., Iterable[EvalSample]]] = {}


def register_dataset(name: str):
  def deco(fn):
    DATASETS[name] = fn
    return fn
  return deco


def _first(d: dict, keys, default=""):
  for k in keys:
    if k in d and d[k] is not None:
      return d[k]
  return default


def sample_from_record(rec: dict, kind: str | None = None) -> EvalSample:
  prompt = str(_first(rec, ("prompt", "question", "input", "text", "instruction")))
  if rec.get("system_prompt"):
    prompt = f"{rec['system_prompt']}\n\n{prompt}"
  choices = list(_first(rec, ("choices", "options"), []))
  ans = _first(rec, ("answer", "label", "target"), -1)
  if choices:
    if isinstance(ans, str) and len(ans) == 1 and ans.upper() in "ABCDEFGHIJ":
      ans = "ABCDEFGHIJ".index(ans.upper())
    elif isinstance(ans, str) and ans in choices:
      ans = choices.index(ans)
    return EvalSample(prompt, choices=[str(c) for c in choices], answer=int(ans), kind=kind or "choice", meta=rec)
  ref = str(_first(rec, ("reference", "output", "response", "completion", "answer", "target")))
  return EvalSample(prompt, reference=ref, kind=kind or ("generate" if ref else "perplexity"), meta=rec)


@register_dataset("jsonl")
def jsonl(path: str, num_samples: int | None = None, kind: str | None = None, **_):
  with open(path, "r", encoding="utf-8") as fh:
    for i, line in enumerate(fh):
      if num_samples is not None and i >= num_samples:
        break
      line = line.strip()
      if line:
        yield sample_from_record(json.loads(line), kind)


@register_dataset("mlperf_openorca")
def mlperf_openorca(path: str, num_samples: int | None = None, **_):
  """The MLPerf inference OpenOrca subset exported as JSON lines (system_prompt, question, output): ROUGE against `output`."""
  yield from jsonl(path, num_samples, kind="generate")


@register_dataset("synthetic_copy")
def synthetic_copy(num_samples: int = 8, **_):
  """Self-contained smoke task: the reference repeats the prompt's last word."""
  words = ["alpha", "beta", "gamma", "delta", "epsilon", "zeta", "eta", "theta"]
  for i in range(int(num_samples)):
    w = words[i % len(words)]
    yield EvalSample(f"repeat the word {w}", reference=w, kind="generate")


def load_dataset(name: str, **kw) -> list[EvalSample]:
  if name not in DATASETS:
    raise KeyError(f"unknown eval dataset {name!r}; registered: {sorted(DATASETS)}")
  return list(DATASETS[name](**kw))
