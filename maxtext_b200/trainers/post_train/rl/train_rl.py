"""Reinforcement learning with group-relative policy optimisation: `python -m maxtext.trainers.post_train.rl.train_rl
<config.yml> key=value ...`.

One iteration = for a batch of questions, render the prompt with the chat template, sample `rl.num_generations`
completions per question with this repository's decode engine (the policy's own weights, so there is nothing to
synchronise), score them with the reward functions, turn the rewards into group-relative advantages, and take
`rl.num_iterations` clipped policy-gradient steps (GRPO or GSPO-token) with an optional KL penalty to the frozen
starting policy (`rl.grpo_beta`). Every `eval_interval` iterations the held-out questions are answered greedily and
scored. The reference builds the same loop from Tunix's RL cluster with vLLM rollout workers
(src/maxtext/trainers/post_train/rl/train_rl.py:427-827); here trainer and sampler share one set of weights in one
process group.

Data: JSON-lines files with `question` and `answer` columns (`hf_train_files` / `hf_eval_files`; GSM8K style `#### 42`
answers are reduced to the final value)."""
from __future__ import annotations

import json
import os
import sys

import torch

from ....config import pyconfig
from ....input_pipeline.file_pipeline import _expand
from ....input_pipeline.tokenizer import build_tokenizer
from ....inference.maxengine import MaxEngine
from ....train import train as train_lib
from ....utils import max_logging
from .. import objectives as O
from ..trainers import make_lm_batch
from . import rewards as R

DEFAULT_TEMPLATE = ("You are given a problem. Think about it and provide your working out between {reasoning_start} and {reasoning_end}. "
                    "Then give the final answer between {solution_start} and {solution_end}.\n\n{question}\n")


def _rl(c, key, default):
  block = getattr(c, "rl", None) or {}
  return block.get(key, default) if isinstance(block, dict) else default


def load_questions(patterns: str) -> list[dict]:
  rows = []
  for f in _expand(patterns):
    with open(f, "r", encoding="utf-8") as fh:
      for line in fh:
        if not line.strip():
          continue
        r = json.loads(line)
        ans = R.extract_hash_answer(str(r["answer"])) or str(r["answer"])
        rows.append({"question": str(r["question"]), "answer": json.dumps([ans])})
  if not rows:
    raise FileNotFoundError(f"no question / answer records in {patterns!r}")
  return rows


def render_prompt(c, question: str) -> str:
  template = DEFAULT_TEMPLATE
  path = str(getattr(c, "data_template_path", "") or "")
  if path and os.path.isfile(path):
    with open(path, "r", encoding="utf-8") as fh:
      template = json.load(fh).get("TEMPLATE", template)
  return template.format(question=question, reasoning_start=c.reasoning_start_token, reasoning_end=c.reasoning_end_token,
                         solution_start=c.solution_start_token, solution_end=c.solution_end_token, system_prompt="")


class Sampler:
  """Batched rollouts on the policy's own weights: every prompt fills one decode slot, generation stops at EOS or at the
  token budget."""

  def __init__(self, engine, tok, strategy: str, temperature: float, top_k: int, top_p: float, slots: int):
    c = engine.config.replace(decode_sampling_strategy=strategy, decode_sampling_temperature=float(temperature),
                              decode_sampling_top_k=int(top_k), decode_sampling_nucleus_p=float(top_p), per_device_batch_size=float(slots))
    self.eng = MaxEngine(c, device=engine.device, model=engine.model)
    self.tok, self.slots = tok, slots

  @torch.no_grad()
  def generate(self, prompts: list[list[int]], max_new: int) -> list[list[int]]:
    out = [[] for _ in prompts]
    eos = getattr(self.tok, "eos_id", -1)
    for lo in range(0, len(prompts), self.slots):
      chunk = prompts[lo:lo + self.slots]
      st = self.eng.init_decode_state(self.slots)
      for j, p in enumerate(chunk):
        prefix, first = self.eng.prefill(torch.tensor(p), len(p))
        st = self.eng.insert(prefix, st, j)
        out[lo + j].append(int(first.data[0, 0]))
      alive = [out[lo + j][-1] != eos for j in range(len(chunk))]
      for _ in range(max_new - 1):
        if not any(alive):
          break
        st, res = self.eng.generate(st)
        toks = res.data[:, 0].tolist()
        for j in range(len(chunk)):
          if alive[j]:
            out[lo + j].append(int(toks[j]))
            if toks[j] == eos or len(chunk[j]) + len(out[lo + j]) >= self.eng.max_len - 1:
              alive[j] = False
    return out


class RLTrainer:
  def __init__(self, config, engine, mesh=None, reward_fns=None):
    self.c, self.eng, self.mesh = config, engine, mesh
    self.tok = build_tokenizer(config)
    self.G = int(_rl(config, "num_generations", 2))
    self.iters = int(_rl(config, "num_iterations", 1))
    self.beta = float(_rl(config, "grpo_beta", 0.0) or 0.0)
    self.clip = float(_rl(config, "grpo_epsilon", 0.2))
    self.algo = str(_rl(config, "loss_algo", "grpo"))
    assert self.algo in ("grpo", "gspo-token"), self.algo
    self.max_new = int(getattr(config, "max_target_length", 64)) - int(getattr(config, "max_prefill_predict_length", 16)) - 1
    self.reward_fns = reward_fns or R.build_reward_fns(config)
    slots = max(1, int(config.per_device_batch_size)) * self.G
    self.sampler = Sampler(engine, self.tok, "weighted" if float(config.decode_sampling_temperature) > 0 else "greedy",
                           config.decode_sampling_temperature, config.decode_sampling_top_k, config.decode_sampling_nucleus_p, slots)
    self.greedy = Sampler(engine, self.tok, "greedy", 1.0, 1, 1.0, slots)
    self.ref_master = engine.store.master.clone() if self.beta > 0 else None

  def _encode_prompt(self, q: str) -> list[int]:
    ids = [t % self.c.vocab_size for t in self.tok.encode(render_prompt(self.c, q), add_bos=bool(self.c.add_bos), add_eos=False)]
    return ids[-int(self.c.max_prefill_predict_length):]

  def _ref_token_losses(self, batch):
    s = self.eng.store
    cur = s.master.clone()
    s.master.copy_(self.ref_master)
    s.sync_compute_from_master()
    out = self.eng.token_losses(batch).cpu()
    s.master.copy_(cur)
    s.sync_compute_from_master()
    return out

  def step(self, rows: list[dict]) -> dict:
    """One RL iteration over a batch of question records."""
    S = int(self.c.max_target_length)
    prompts, questions, answers = [], [], []
    for r in rows:
      ids = self._encode_prompt(r["question"])
      for _ in range(self.G):
        prompts.append(ids)
        questions.append(r["question"])
        answers.append(r["answer"])
    comps = self.sampler.generate(prompts, self.max_new)
    texts = [self.tok.decode(cm) for cm in comps]
    rewards = torch.tensor(R.total_reward(self.reward_fns, questions, texts, self.c, answer=answers, question=questions))
    adv = O.grpo_advantages(rewards, self.G) if self.G > 1 else rewards - rewards.mean()
    batch, total = make_lm_batch([p + cm for p, cm in zip(prompts, comps)], S)
    mask = O.sft_mask(torch.tensor([len(p) for p in prompts]), total, S)
    old = self.eng.token_losses(batch).cpu()
    ref = self._ref_token_losses(batch) if self.beta > 0 else None
    weights_fn = O.gspo_weights if self.algo == "gspo-token" else O.grpo_weights
    m = {}
    for it in range(self.iters):
      cur = old if it == 0 else self.eng.token_losses(batch).cpu()
      surrogate, w = weights_fn(cur, old, adv, mask, self.clip)
      if ref is not None:
        # k3 estimator of KL(pi || ref) per token: exp(d) - d - 1 with d = log ref - log pi; its gradient w.r.t. log pi is
        # 1 - exp(d), and the engine differentiates sum_t w_t * (-log pi_t), hence the sign
        d = cur - ref
        w = w - self.beta * (1.0 - torch.exp(d)) * mask
        m["rl/kl"] = ((torch.exp(d) - d - 1.0) * mask).sum() / mask.sum().clamp_min(1)
      b = dict(batch)
      b["loss_weights"], b["loss_normalizer"] = w, float(mask.sum().clamp_min(1))
      m.update(self.eng.train_step(b))
      m["rl/surrogate"] = surrogate
    m["rl/mean_reward"], m["rl/reward_std"] = rewards.mean(), rewards.std() if len(rewards) > 1 else torch.tensor(0.0)
    m["rl/completion_tokens"] = float(sum(len(cm) for cm in comps)) / max(1, len(comps))
    return m

  def evaluate(self, rows: list[dict]) -> dict:
    from .evaluate_rl import evaluate
    return evaluate(self, rows)


def rl_train(config, engine=None, mesh=None, reward_fns=None):
  if engine is None:
    config, mesh, engine = train_lib.setup(config)
  c = config
  train_rows = load_questions(c.hf_train_files or c.dataset_path)
  eval_rows = load_questions(c.hf_eval_files) if getattr(c, "hf_eval_files", "") else []
  trainer = RLTrainer(c, engine, mesh, reward_fns)
  bs = max(1, int(c.per_device_batch_size))
  history = []
  for it in range(int(c.steps)):
    rows = [train_rows[(it * bs + j) % len(train_rows)] for j in range(bs)]
    m = trainer.step(rows)
    history.append({k: float(v) for k, v in m.items() if _num(v)})
    max_logging.log(f"rl iteration {it}: reward {float(m['rl/mean_reward']):.3f}, loss {float(m['learning/loss']):.4f}")
    if eval_rows and int(c.eval_interval) > 0 and (it + 1) % int(c.eval_interval) == 0:
      ev = trainer.evaluate(eval_rows[: max(1, int(c.eval_steps) if int(c.eval_steps) > 0 else len(eval_rows))])
      history[-1].update({f"eval/{k}": v for k, v in ev.items()})
      max_logging.log(f"rl eval after iteration {it}: {ev}")
  return trainer, history


def _num(v):
  try:
    float(v)
    return True
  except (TypeError, ValueError):
    return False


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  return rl_train(pyconfig.initialize(argv))


if __name__ == "__main__":
  main()
