"""Generation tasks in the style of OpenAI's simple-evals (src/maxtext/eval/simple_evals_template/, runner/simple_evals_runner.py):
every task is a prompt template, an answer extractor and a scorer; a *sampler* turns a list of chat messages into text.

  tasks: gsm8k (final "Answer:" line, integer match), aime (integer 0..999), mmlu and gpqa (letter choice, gpqa with shuffled
  options), drop (bag-of-words F1 against any reference answer).

Rows come from local JSON-lines / parquet files with the public field names of each set (there is no network on training
machines). `EngineSampler` answers with this repository's decode engine through the chat template; any callable
`messages -> str` works (a client of the HTTP server, a stub in tests).

  python -m maxtext_b200.eval.simple_evals <config.yml> [key=value ...] --task gsm8k --path gsm8k_test.jsonl [--limit N] [--out DIR]
"""
from __future__ import annotations

import json
import os
import random
import re
import string
import sys
from dataclasses import dataclass, field
from typing import Callable

Sampler = Callable[[list], str]


@dataclass
class SingleResult:
  score: float
  prompt: list
  response: str
  extracted: str | None
  target: str
  meta: dict = field(default_factory=dict)


@dataclass
class TaskResult:
  task: str
  score: float
  n: int
  metrics: dict
  samples: list

  def to_json(self) -> dict:
    return {"task": self.task, "score": self.score, "n": self.n, "metrics": self.metrics,
            "samples": [s.__dict__ for s in self.samples]}


# ------------------------------------------------------------------------------------------ answer handling
_NUM_LINE = re.compile(r"(?i)(?:^|\n)\s*Answer\s*:\s*\$?\s*(-?[\d,]*\.?\d+)\s*\.?\s*\Z")
_LETTER = re.compile(r"(?i)Answer\s*:\s*\$?\(?([A-J])\)?\$?")


def extract_number(text: str) -> str | None:
  """The number on a final `Answer:` line (thousands separators and a trailing period tolerated)."""
  m = _NUM_LINE.search(text.strip())
  return m.group(1).replace(",", "") if m else None


def numbers_equal(a: str | None, b: str) -> bool:
  if a is None:
    return False
  try:
    return abs(float(a) - float(str(b).replace(",", ""))) < 1e-6
  except ValueError:
    return False


def extract_letter(text: str) -> str | None:
  m = None
  for m in _LETTER.finditer(text):        # the last statement counts
    pass
  return m.group(1).upper() if m else None


def _normalize_words(s: str) -> list[str]:
  s = s.lower()
  s = "".join(ch for ch in s if ch not in set(string.punctuation))
  s = re.sub(r"\b(a|an|the)\b", " ", s)
  return s.split()


def f1_words(pred: str, ref: str) -> float:
  p, r = _normalize_words(pred), _normalize_words(ref)
  if not p or not r:
    return float(p == r)
  common = 0
  rest = list(r)
  for w in p:
    if w in rest:
      rest.remove(w)
      common += 1
  if common == 0:
    return 0.0
  prec, rec = common / len(p), common / len(r)
  return 2 * prec * rec / (prec + rec)


# ------------------------------------------------------------------------------------------ tasks
GSM8K_TEMPLATE = ("Solve this math problem. Give the reasoning steps before giving the final answer on the last line by itself in the format "
                  'of "Answer:". Do not add anything other than the integer answer after "Answer:".\n\n{question}')
AIME_TEMPLATE = ("Solve the following competition problem. The answer is an integer between 0 and 999. Think step by step, then give the final "
                 'answer on the last line in the format "Answer: N".\n\n{question}')
CHOICE_TEMPLATE = ("Answer the following multiple choice question. The last line of your response should be of the following format: "
                   "'Answer: $LETTER' (without quotes) where LETTER is one of {letters}. Think step by step before answering.\n\n{question}\n\n{options}")
DROP_TEMPLATE = ("Read the passage and answer the question. Think step by step, then write a line of the form \"Answer: $ANSWER\" at the end of "
                 "your response.\n\nPassage: {passage}\n\nQuestion: {question}")


def _user(text: str) -> list:
  return [{"role": "user", "content": text}]


def _gsm8k(row, rng):
  target = str(row["answer"]).split("####")[-1].strip().replace(",", "")
  return _user(GSM8K_TEMPLATE.format(question=row["question"])), target, extract_number, lambda got: float(numbers_equal(got, target))


def _aime(row, rng):
  target = str(int(str(row.get("answer", row.get("Answer"))).strip()))
  return _user(AIME_TEMPLATE.format(question=row.get("problem", row.get("question")))), target, extract_number, \
      lambda got: float(numbers_equal(got, target))


def _choice(question, options, answer_index, rng, shuffle):
  order = list(range(len(options)))
  if shuffle:
    rng.shuffle(order)
  letters = string.ascii_uppercase[:len(options)]
  text = CHOICE_TEMPLATE.format(letters="".join(letters), question=question,
                                options="\n".join(f"{letters[i]}) {options[j]}" for i, j in enumerate(order)))
  target = letters[order.index(answer_index)]
  return _user(text), target, extract_letter, lambda got: float(got == target)


def _mmlu(row, rng):
  ans = row["answer"]
  idx = "ABCD".index(ans.strip().upper()[0]) if isinstance(ans, str) else int(ans)
  return _choice(row["question"], list(row["choices"]), idx, rng, shuffle=False)


def _gpqa(row, rng):
  opts = [row["Correct Answer"], row["Incorrect Answer 1"], row["Incorrect Answer 2"], row["Incorrect Answer 3"]]
  return _choice(row["Question"], opts, 0, rng, shuffle=True)


def _drop(row, rng):
  refs = row.get("answers") or row.get("ref_text") or [row.get("answer", "")]
  refs = [str(r) for r in (refs if isinstance(refs, (list, tuple)) else str(refs).split("|"))]

  def get(text):
    m = re.search(r"(?i)Answer\s*:\s*(.+)\s*\Z", text.strip())
    return m.group(1).strip() if m else None
  return _user(DROP_TEMPLATE.format(passage=row.get("passage", row.get("context", "")), question=row["question"])), refs[0], get, \
      lambda got: max((f1_words(got, r) for r in refs), default=0.0) if got else 0.0


TASKS = {"gsm8k": _gsm8k, "aime": _aime, "mmlu": _mmlu, "gpqa": _gpqa, "drop": _drop}


def load_rows(path: str, limit: int | None = None) -> list[dict]:
  rows: list[dict] = []
  if path.endswith(".parquet"):
    import pyarrow.parquet as pq
    rows = pq.read_table(path).to_pylist()
  else:
    with open(path, encoding="utf-8") as fh:
      rows = [json.loads(line) for line in fh if line.strip()]
  return rows[:limit] if limit else rows


def run_task(task: str, rows: list[dict], sampler: Sampler, seed: int = 0) -> TaskResult:
  if task not in TASKS:
    raise KeyError(f"unknown task {task!r}; available: {sorted(TASKS)}")
  rng = random.Random(seed)
  out = []
  for row in rows:
    messages, target, extract, score = TASKS[task](row, rng)
    response = sampler(messages)
    got = extract(response)
    out.append(SingleResult(float(score(got)), messages, response, got, str(target), {"subject": row.get("subject", "")}))
  n = len(out)
  mean = sum(s.score for s in out) / max(1, n)
  std = (sum((s.score - mean) ** 2 for s in out) / max(1, n)) ** 0.5
  return TaskResult(task, mean, n, {"score": mean, "score:std": std, "extracted": sum(s.extracted is not None for s in out) / max(1, n)}, out)


def write_report(result: TaskResult, directory: str) -> str:
  os.makedirs(directory, exist_ok=True)
  path = os.path.join(directory, f"simple_evals_{result.task}.json")
  with open(path, "w") as fh:
    json.dump(result.to_json(), fh, indent=1)
  return path


class EngineSampler:
  """Answers with the in-process decode engine: chat template + generation prompt, greedy or configured sampling."""

  def __init__(self, config, backend=None, max_new_tokens: int = 256):
    from ..input_pipeline import chat
    from .runner import LocalBackend
    self.backend = backend or LocalBackend(config)
    self.template, self.chat, self.max_new = chat.load_template(config), chat, int(max_new_tokens)

  def __call__(self, messages: list) -> str:
    return self.backend.generate([self.chat.render(messages, self.template, add_generation_prompt=True)], self.max_new)[0]


def main(argv=None):
  import argparse
  argv = list(sys.argv[1:] if argv is None else argv)
  ap = argparse.ArgumentParser()
  ap.add_argument("config", nargs="+")
  ap.add_argument("--task", required=True)
  ap.add_argument("--path", required=True)
  ap.add_argument("--limit", type=int)
  ap.add_argument("--out", default="")
  ap.add_argument("--max-new-tokens", type=int, default=256)
  a = ap.parse_args(argv)
  from ..config import pyconfig
  cfg = pyconfig.initialize(["eval"] + a.config)
  res = run_task(a.task, load_rows(a.path, a.limit), EngineSampler(cfg, max_new_tokens=a.max_new_tokens))
  print(json.dumps({"task": res.task, "n": res.n, **res.metrics}))
  if a.out:
    print(write_report(res, a.out))
  return res


if __name__ == "__main__":
  main()
