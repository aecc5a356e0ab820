"""MMLU accuracy of a checkpoint, overall and per subject / field / area.

  python -m maxtext_b200.benchmarks.mmlu.mmlu_eval maxtext_b200/configs/base.yml model_name=... load_parameters_path=... \\
      mmlu_path=<dir or file> [mmlu_split=test] [mmlu_limit=N] [prompt_template='...{subject}...{question}...{choices}...']

`mmlu_path`: a JSON-lines or parquet file (or a directory of them) with the fields of the public set (`question`, `subject`,
`choices` [4], `answer` index or letter); with HuggingFace `datasets` and a local copy of `cais/mmlu`, `mmlu_path=hf:cais/mmlu`.
Two scoring modes (benchmarks/mmlu/mmlu_eval.py:79-237 uses the first): `generate` decodes a few tokens and parses
"Answer: X"; `loglik` (default here: no parsing failures) picks the letter whose next-token log-probability is highest.
"""
from __future__ import annotations

import collections
import glob
import json
import os
import re
import sys

import torch

from .subjects import AREA_OF, FIELD_OF

DEFAULT_PROMPT_TEMPLATE = """The following are multiple choice questions (with answers) about {subject}.

{question}
{choices}
Answer:"""
LETTERS = "ABCD"


def construct_prompt(subject: str, question: str, choices, template: str = DEFAULT_PROMPT_TEMPLATE) -> str:
  lines = "\n".join(f"{chr(ord('A') + i)}. {c}" for i, c in enumerate(choices))
  return template.format(subject=subject.replace("_", " "), question=question, choices=lines)


def parse_answer(output: str) -> str | None:
  """The letter after "Answer:" / "The answer is", else None."""
  m = re.search(r"Answer:\s*\(?([A-D])\b|The answer is\s*\(?([A-D])\b", output, re.IGNORECASE)
  return (m.group(1) or m.group(2)).upper() if m else None


def load_samples(path: str, split: str = "test", limit: int | None = None) -> list[dict]:
  rows: list[dict] = []
  if path.startswith("hf:"):
    import datasets                                         # local cache only: there is no network on training machines
    ds = datasets.load_dataset(path[3:], "all", split=split)
    rows = [dict(r) for r in ds]
  else:
    files = sorted(glob.glob(os.path.join(path, "**", "*"), recursive=True)) if os.path.isdir(path) else [path]
    for f in files:
      if f.endswith((".jsonl", ".json")):
        with open(f, encoding="utf-8") as fh:
          rows += [json.loads(line) for line in fh if line.strip()]
      elif f.endswith(".parquet"):
        import pyarrow.parquet as pq
        rows += pq.read_table(f).to_pylist()
  out = []
  for r in rows:
    ans = r.get("answer")
    if isinstance(ans, str):
      ans = LETTERS.index(ans.strip().upper()[0])
    out.append({"subject": str(r.get("subject", "miscellaneous")), "question": str(r["question"]), "choices": [str(c) for c in r["choices"]],
                "answer": int(ans)})
  return out[:limit] if limit else out


class Tally:
  """Correct / total per subject, field and area."""

  def __init__(self):
    self.by = {k: collections.defaultdict(lambda: [0, 0]) for k in ("subject", "field", "area")}
    self.correct = self.total = 0

  def add(self, subject: str, ok: bool):
    field = FIELD_OF.get(subject, "other")
    for kind, key in (("subject", subject), ("field", field), ("area", AREA_OF.get(field, "other (business, health, misc.)"))):
      c = self.by[kind][key]
      c[0] += int(ok)
      c[1] += 1
    self.correct += int(ok)
    self.total += 1

  def report(self) -> dict:
    acc = lambda c: c[0] / max(1, c[1])                     # noqa: E731
    return {"accuracy": self.correct / max(1, self.total), "total": self.total,
            **{kind: {k: round(acc(v), 4) for k, v in sorted(d.items())} for kind, d in self.by.items()}}


def letter_token_ids(tokenizer) -> list[int]:
  """Token id of each answer letter as it appears after "Answer:" (with the leading space when the tokenizer has one)."""
  ids = []
  for ch in LETTERS:
    with_space = tokenizer.encode(" " + ch)
    plain = tokenizer.encode(ch)
    ids.append(int((with_space if len(with_space) == 1 else plain)[-1]))
  return ids


def evaluate(engine, tokenizer, samples: list[dict], template: str = DEFAULT_PROMPT_TEMPLATE, mode: str = "loglik",
             max_new_tokens: int = 8) -> dict:
  tally = Tally()
  letters = letter_token_ids(tokenizer) if mode == "loglik" else None
  limit = int(engine.config.max_prefill_predict_length)
  for s in samples:
    ids = tokenizer.encode(construct_prompt(s["subject"], s["question"], s["choices"], template))[-limit:]
    t = torch.tensor(ids, dtype=torch.long)
    prefix, first = engine.prefill(t, len(ids))
    if mode == "loglik":
      pred = int(torch.as_tensor(prefix.logits).reshape(-1)[letters].argmax())
    else:
      state = engine.init_decode_state(1)
      state = engine.insert(prefix, state, 0)
      out = [int(first.data[0, 0])]
      for _ in range(max_new_tokens - 1):
        state, res = engine.generate(state)
        out.append(int(res.data[0, 0]))
      got = parse_answer("Answer:" + tokenizer.decode(out))
      pred = LETTERS.index(got) if got else -1
    tally.add(s["subject"], pred == s["answer"])
  return tally.report()


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  own = {}
  rest = []
  for a in argv:
    k = a.split("=", 1)[0]
    if k in ("mmlu_path", "mmlu_split", "mmlu_limit", "prompt_template", "mmlu_mode"):
      own[k] = a.split("=", 1)[1]
    else:
      rest.append(a)
  from ...config import pyconfig
  from ...inference.maxengine import MaxEngine
  from ...input_pipeline.tokenizer import build_tokenizer
  cfg = pyconfig.initialize(rest)
  eng = MaxEngine(cfg)
  eng.load_params(cfg.load_parameters_path or None)
  samples = load_samples(own["mmlu_path"], own.get("mmlu_split", "test"), int(own["mmlu_limit"]) if own.get("mmlu_limit") else None)
  rep = evaluate(eng, build_tokenizer(cfg), samples, own.get("prompt_template", DEFAULT_PROMPT_TEMPLATE).replace("\\n", "\n"), own.get("mmlu_mode", "loglik"))
  print(json.dumps(rep, indent=1))
  return rep


if __name__ == "__main__":
  main()
