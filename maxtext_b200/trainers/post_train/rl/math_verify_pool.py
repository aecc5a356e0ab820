"""Answer verification in worker processes with a deadline.

Comparing a model's answer with the gold answer can mean parsing arbitrary text as a number or an expression; a
malformed string must not stall the trainer. The reference hands batches of (gold answers, predictions) to a spawn-based
process pool and terminates the pool when a batch runs past its deadline (src/maxtext/trainers/post_train/rl/
math_verify_pool.py:95-260). This module does the same with the standard library: `verify_math_worker` decides one item
(exact text, numeric value with tolerance, simple fractions / percentages, and `sympy` when it is installed), and
`math_verify_pool` scores a batch, replacing timed-out or crashed items by 0."""
from __future__ import annotations

import atexit
import multiprocessing as mp
import re
from fractions import Fraction

_POOL = None
_POOL_PROCS = 0


def _strip_boxed(s: str) -> str:
  s = s.strip()
  m = re.fullmatch(r"\\boxed\{(.*)\}", s, flags=re.DOTALL)
  return m.group(1).strip() if m else s


def _to_number(s: str):
  s = _strip_boxed(s).replace(",", "").replace("$", "").strip()
  pct = s.endswith("%") or s.endswith("\\%")
  s = s.rstrip("%").rstrip("\\").strip()
  m = re.fullmatch(r"\\d?frac\{(-?[\d.]+)\}\{(-?[\d.]+)\}", s) or re.fullmatch(r"(-?[\d.]+)\s*/\s*(-?[\d.]+)", s)
  try:
    v = Fraction(m.group(1)) / Fraction(m.group(2)) if m else Fraction(s)
  except (ValueError, ZeroDivisionError):
    return None
  return v / 100 if pct else v


def are_equal(gold: str, pred: str, rel_tol: float = 1e-6) -> bool:
  g, p = _strip_boxed(gold), _strip_boxed(pred)
  if g == p or g.replace(" ", "") == p.replace(" ", ""):
    return True
  a, b = _to_number(g), _to_number(p)
  if a is not None and b is not None:
    return a == b or abs(float(a) - float(b)) <= rel_tol * max(1.0, abs(float(a)))
  try:
    import sympy
    from sympy.parsing.sympy_parser import parse_expr
    return bool(sympy.simplify(parse_expr(g.replace("^", "**")) - parse_expr(p.replace("^", "**"))) == 0)
  except Exception:  # pylint: disable=broad-except
    return False


def verify_math_worker(golds: list[str], predictions: list[str]) -> float:
  """1.0 when any prediction equals any gold answer."""
  return 1.0 if any(are_equal(g, p) for g in golds for p in predictions) else 0.0


def _shutdown_pool():
  global _POOL
  if _POOL is not None:
    _POOL.terminate()
    _POOL = None


def _get_pool(num_procs: int):
  global _POOL, _POOL_PROCS
  if _POOL is None or _POOL_PROCS != num_procs:
    _shutdown_pool()
    _POOL = mp.get_context("spawn").Pool(num_procs)
    _POOL_PROCS = num_procs
    atexit.register(_shutdown_pool)
  return _POOL


def math_verify_pool(items, scores: list[float], reward: float = 1.0, timeout: float = 30.0, num_procs: int | None = None, log_fn=None):
  """items: (index into scores, gold answers, predictions). A verified item raises its score to `reward`; an item whose
  worker does not answer within `timeout` seconds (for the whole batch) keeps its score, and the pool is rebuilt."""
  if not items:
    return scores
  procs = int(num_procs or min(4, max(1, (mp.cpu_count() or 2) // 2)))
  if procs <= 1 and len(items) <= 4:
    for idx, golds, preds in items:                       # tiny batches: not worth a pool
      if verify_math_worker(golds, preds) > 0:
        scores[idx] = max(scores[idx], reward)
    return scores
  pool = _get_pool(procs)
  pending = [(idx, pool.apply_async(verify_math_worker, (golds, preds))) for idx, golds, preds in items]
  import time
  deadline = time.time() + timeout
  timed_out = False
  for idx, res in pending:
    try:
      if res.get(max(0.0, deadline - time.time())) > 0:
        scores[idx] = max(scores[idx], reward)
    except mp.TimeoutError:
      timed_out = True
    except Exception as e:  # pylint: disable=broad-except
      if log_fn:
        log_fn(f"math verification failed for item {idx}: {e!r}")
  if timed_out:
    if log_fn:
      log_fn("math verification ran past its deadline; restarting the worker pool")
    _shutdown_pool()
  return scores
