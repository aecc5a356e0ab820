"""Reward functions for reasoning-style RL and the answer extraction they share.

Behaviour follows the reference's `utils_rl.py` (src/maxtext/trainers/post_train/rl/utils_rl.py:165-584): completions
are expected as `<reasoning>...</reasoning><answer>...</answer>` (tags from the config), the format rewards score the
tag structure, `check_numbers` scores the extracted answer against a JSON list of acceptable answers (exact, up to white
space, or mathematically equal through the verification pool), and user code can be named with
`reward_functions_path` / `reward_functions`. Every reward has the signature
`fn(prompts, completions, config, answer=..., question=...) -> list[float]`."""
from __future__ import annotations

import importlib.util
import json
import re

from . import math_verify_pool as mvp

FALLBACK_ANSWER = "<no answer>"


def boxed(x: str) -> str:
  return x if x.startswith("\\boxed{") else "\\boxed{" + x + "}"


def match_format_regex(c) -> re.Pattern:
  start = "" if getattr(c, "reasoning_start_token_in_prompt", False) else re.escape(c.reasoning_start_token)
  return re.compile(rf"{start}.*?{re.escape(c.reasoning_end_token)}.*?{re.escape(c.solution_start_token)}(.+?){re.escape(c.solution_end_token)}",
                    flags=re.MULTILINE | re.DOTALL)


def answer_tag_regex(c) -> re.Pattern:
  return re.compile(rf"{re.escape(c.solution_start_token)}(.+?){re.escape(c.solution_end_token)}", flags=re.MULTILINE | re.DOTALL)


def match_format_exactly(prompts, completions, c, **kw) -> list[float]:
  rx = match_format_regex(c)
  return [float(c.reward_exact_format_match) if rx.search(comp) is not None else 0.0 for comp in completions]


def match_format_approximately(prompts, completions, c, **kw) -> list[float]:
  out = []
  for comp in completions:
    s = 0.0
    tags = [c.reasoning_end_token, c.solution_start_token, c.solution_end_token]
    ok_start = getattr(c, "reasoning_start_token_in_prompt", False) or comp.count(c.reasoning_start_token) == 1
    s += c.reward_partial_format_match if ok_start else c.penalty_incorrect_format
    for t in tags:
      s += c.reward_partial_format_match if comp.count(t) == 1 else c.penalty_incorrect_format
    out.append(float(s))
  return out


def extract_answer(response: str, c) -> str:
  """The last `\\boxed{...}` (brace balanced) inside the last answer block, else the block's text, else FALLBACK_ANSWER."""
  rx = answer_tag_regex(c)
  blocks = rx.findall(response)
  content = blocks[-1] if blocks else response
  found, stack = [], []
  for i, ch in enumerate(content):
    if ch == "{":
      stack.append(i)
    elif ch == "}" and stack:
      op = stack.pop()
      if content[:op].endswith("\\boxed"):
        found.append(content[op + 1:i].strip())
  if found:
    return found[-1]
  m = re.search(r"\\boxed\s*\{?\s*([a-zA-Z0-9\.,\-]+)\s*\}?", content)
  if m:
    return m.group(1).strip()
  return blocks[-1].strip() if blocks else FALLBACK_ANSWER


def extract_hash_answer(text: str):
  """GSM8K style gold answers: the text after `####`."""
  return text.split("####")[1].strip() if "####" in text else None


def preprocess_math_string(text: str) -> str:
  text = text.strip().rstrip(".")
  text = re.sub(r"\\text\{[^}]*\}", "", text)
  text = text.replace("\\!", "").replace("\\,", "").replace("\\ ", "").replace("dollars", "").replace("$", "")
  return text.strip()


def check_numbers(prompts, completions, c, answer=None, **kw) -> list[float]:
  """answer: per completion, a JSON list of acceptable answers (or a plain string)."""
  guesses = [extract_answer(comp, c) for comp in completions]
  scores = [float(c.penalty_incorrect_format)] * len(completions)
  queue = []
  for i, (guess, ans) in enumerate(zip(guesses, answer or [])):
    try:
      golds = json.loads(ans) if isinstance(ans, str) and ans.strip().startswith("[") else [ans]
    except json.JSONDecodeError:
      golds = [ans]
    golds = list(dict.fromkeys(str(g) for g in golds))
    if guess == FALLBACK_ANSWER:
      scores[i] = float(c.penalty_incorrect_answer)
      continue
    hit = False
    for g in golds:
      if guess == g:
        scores[i], hit = max(scores[i], float(c.reward_exact_answer)), True
      elif guess.strip() == g.strip():
        scores[i], hit = max(scores[i], float(c.reward_white_space_format_match)), True
    if not hit:
      queue.append((i, [boxed(preprocess_math_string(g)) for g in golds], [boxed(preprocess_math_string(guess))]))
  if queue:
    scores = mvp.math_verify_pool(queue, scores, reward=float(c.reward_exact_answer), timeout=float(getattr(c, "math_verify_timeout", 30.0) or 30.0),
                                  num_procs=getattr(c, "math_verify_num_procs", None))
  return scores


BUILTIN = {"match_format_exactly": match_format_exactly, "match_format_approximately": match_format_approximately,
           "check_numbers": check_numbers}


def load_custom_callable(module_path: str, function_name: str):
  spec = importlib.util.spec_from_file_location("maxtext_b200_user_rewards", module_path)
  mod = importlib.util.module_from_spec(spec)
  spec.loader.exec_module(mod)
  return getattr(mod, function_name)


def build_reward_fns(c) -> list:
  """`reward_functions` (comma separated names) from `reward_functions_path` when given, else the three built-in ones."""
  names = [n.strip() for n in str(getattr(c, "reward_functions", "") or "").split(",") if n.strip()]
  path = str(getattr(c, "reward_functions_path", "") or "")
  if names and path:
    return [load_custom_callable(path, n) for n in names]
  if names:
    return [BUILTIN[n] for n in names]
  return [match_format_exactly, match_format_approximately, check_numbers]


def total_reward(fns, prompts, completions, c, **kw):
  tot = [0.0] * len(completions)
  for fn in fns:
    for i, s in enumerate(fn(prompts, completions, c, **kw)):
      tot[i] += float(s)
  return tot
