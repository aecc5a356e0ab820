"""Post-training loops built on the step-wise engine API (`fwd_bwd` / `update`): SFT, DPO, GRPO-style RL, distillation
(src/maxtext/trainers/post_train/{sft/train_sft.py, dpo/train_dpo.py, rl/train_rl.py, distillation/train_distill.py}).
Rollouts for RL come from this repository's decode engine instead of an external vLLM / Tunix cluster."""
from __future__ import annotations

import math

import copy

import torch

from ...inference.maxengine import MaxEngine
from ...train.engine import TrainEngine
from . import objectives as O


def _pad(seqs, S, pad=0):
  out = torch.full((len(seqs), S + 1), pad, dtype=torch.long)
  for i, s in enumerate(seqs):
    s = list(s)[: S + 1]
    out[i, :len(s)] = torch.tensor(s)
  return out


def make_lm_batch(seqs, S):
  t = _pad(seqs, S)
  return {"inputs": t[:, :-1].int(), "targets": t[:, 1:].int()}, torch.tensor([min(len(s), S + 1) for s in seqs])


# ------------------------------------------------------------------------------------------------ SFT
def sft_step(engine: TrainEngine, prompts, completions) -> dict:
  S = int(engine.config.max_target_length)
  seqs = [list(p) + list(c) for p, c in zip(prompts, completions)]
  batch, total = make_lm_batch(seqs, S)
  mask = O.sft_mask(torch.tensor([len(p) for p in prompts]), total, S, bool(engine.config.sft_train_on_completion_only))
  batch["loss_weights"] = mask
  return engine.train_step(batch)


# ------------------------------------------------------------------------------------------------ DPO
class DPOTrainer:
  def __init__(self, engine: TrainEngine, beta: float = 0.1, label_smoothing: float = 0.0):
    self.eng, self.beta, self.ls = engine, beta, label_smoothing
    self.ref_master = engine.store.master.clone()          # frozen reference policy = the starting weights

  def _logps(self, batch, mask, reference: bool):
    s = self.eng.store
    if reference:
      cur = s.master.clone()
      s.master.copy_(self.ref_master)
      s.sync_compute_from_master()
    lp = O.sequence_logprob(self.eng.token_losses(batch).cpu(), mask)
    if reference:
      s.master.copy_(cur)
      s.sync_compute_from_master()
    return lp

  def step(self, prompts, chosen, rejected) -> dict:
    S = int(self.eng.config.max_target_length)
    pl = torch.tensor([len(p) for p in prompts])
    bc, tc = make_lm_batch([list(p) + list(c) for p, c in zip(prompts, chosen)], S)
    br, tr = make_lm_batch([list(p) + list(c) for p, c in zip(prompts, rejected)], S)
    mc, mr = O.sft_mask(pl, tc, S), O.sft_mask(pl, tr, S)
    pi_c, pi_r = self._logps(bc, mc, False), self._logps(br, mr, False)
    ref_c, ref_r = self._logps(bc, mc, True), self._logps(br, mr, True)
    loss, wc, wr, acc = O.dpo_weights(pi_c, pi_r, ref_c, ref_r, mc, mr, self.beta, self.ls)
    n = len(prompts)
    for b, w in ((bc, wc), (br, wr)):
      b["loss_weights"], b["loss_normalizer"] = w, float(n)
      self.eng.fwd_bwd(b)
    m = self.eng.update()
    m["dpo/loss"], m["dpo/reward_accuracy"] = loss.mean(), acc
    return m


class DPODataIterator:
  """`use_dpo` input (src/maxtext/input_pipeline, dpo_utils.py): JSON-lines records with prompt / chosen / rejected text
  (columns from `train_data_columns`, default those three names), tokenised and cut to fit, `batch` records at a time,
  dealt round-robin to the data shards; loops over the files."""

  def __init__(self, config, data_rank: int = 0, data_world: int = 1):
    import json
    from ...input_pipeline.file_pipeline import _expand
    from ...input_pipeline.tokenizer import build_tokenizer
    c = self.c = config
    cols = list(c.train_data_columns)
    self.cols = cols if len(cols) >= 3 else ["prompt", "chosen", "rejected"]
    tok = build_tokenizer(c)
    S = int(c.max_target_length)
    self.records = []
    for f in _expand(c.hf_train_files or c.grain_train_files or c.dataset_path):
      with open(f, "r", encoding="utf-8") as fh:
        for i, line in enumerate(l for l in fh if l.strip()):
          if i % data_world != data_rank:
            continue
          r = json.loads(line)
          enc = lambda t, bos: [x % c.vocab_size for x in tok.encode(str(t), add_bos=bos and bool(c.add_bos), add_eos=False)]  # noqa: E731
          p = enc(r[self.cols[0]], True)[: S // 2]
          self.records.append((p, enc(r[self.cols[1]], False)[: S - len(p)], enc(r[self.cols[2]], False)[: S - len(p)]))
    if not self.records:
      raise FileNotFoundError("use_dpo: no prompt / chosen / rejected records found")
    self.batch = max(1, int(c.global_batch_size_to_load) // data_world)
    self.pos = 0

  def __iter__(self):
    return self

  def __next__(self):
    rows = [self.records[(self.pos + i) % len(self.records)] for i in range(self.batch)]
    self.pos += self.batch
    return {"prompts": [r[0] for r in rows], "chosen": [r[1] for r in rows], "rejected": [r[2] for r in rows]}

  def state(self):
    return {"pos": self.pos}

  def load_state(self, st):
    self.pos = int(st.get("pos", 0))


class DPOStepper:
  """Adapter that lets the pre-training loop drive `DPOTrainer` (`use_dpo=true`)."""

  def __init__(self, engine: TrainEngine):
    c = engine.config
    self.trainer = DPOTrainer(engine, float(getattr(c, "dpo_beta", 0.1)), float(getattr(c, "dpo_label_smoothing", 0.0)))

  def train_step(self, batch: dict) -> dict:
    return self.trainer.step(batch["prompts"], batch["chosen"], batch["rejected"])


# ------------------------------------------------------------------------------------------------ GRPO
class GRPOTrainer:
  """Sample `group_size` completions per prompt with the decode engine, score them, take one clipped policy step."""

  def __init__(self, engine: TrainEngine, reward_fn, group_size: int = 4, clip: float = 0.2, max_new_tokens: int = 8,
               loss_algo: str = "grpo"):
    self.eng, self.reward_fn, self.G, self.clip, self.max_new = engine, reward_fn, group_size, clip, max_new_tokens
    assert loss_algo in ("grpo", "gspo-token"), loss_algo
    self.loss_algo = loss_algo
    icfg = engine.config.replace(decode_sampling_strategy="weighted")
    self.sampler = MaxEngine(icfg, device=engine.device, model=engine.model)

  def rollout(self, prompt):
    prefix, first = self.sampler.prefill(torch.tensor(prompt), len(prompt))
    st = self.sampler.insert(prefix, self.sampler.init_decode_state(1), 0)
    out = [int(first.data[0, 0])]
    for _ in range(self.max_new - 1):
      st, res = self.sampler.generate(st)
      out.append(int(res.data[0, 0]))
    return out

  def step(self, prompts) -> dict:
    S = int(self.eng.config.max_target_length)
    ps, cs = [], []
    for p in prompts:
      for _ in range(self.G):
        ps.append(list(p))
        cs.append(self.rollout(list(p)))
    rewards = torch.tensor([float(self.reward_fn(p, c)) for p, c in zip(ps, cs)])
    adv = O.grpo_advantages(rewards, self.G)
    batch, total = make_lm_batch([p + c for p, c in zip(ps, cs)], S)
    mask = O.sft_mask(torch.tensor([len(p) for p in ps]), total, S)
    old = self.eng.token_losses(batch).cpu()
    weights_fn = O.gspo_weights if self.loss_algo == "gspo-token" else O.grpo_weights
    surrogate, w = weights_fn(old, old, adv, mask, self.clip)           # on-policy: ratio = 1 at the first step
    batch["loss_weights"], batch["loss_normalizer"] = w, float(mask.sum().clamp_min(1))
    m = self.eng.train_step(batch)
    m["rl/mean_reward"], m["rl/surrogate"] = rewards.mean(), surrogate
    return m


# ------------------------------------------------------------------------------------------------ distillation
def scheduled(step: int, max_steps: int, start: float, end, kind: str) -> float:
  """A loss weight that moves from `start` to `end` over the run: `constant`, `linear` or `cosine` in step / max_steps
  (`distill_{alpha,temperature,beta}_schedule` and `_end`; distillation_utils.py:165 `compute_schedule`)."""
  if end is None or str(end) in ("None", "") or kind == "constant":
    return float(start)
  start, end = float(start), float(end)
  prog = min(max(step / max(1, max_steps), 0.0), 1.0)
  if kind == "linear":
    return start + (end - start) * prog
  if kind == "cosine":
    return end + (start - end) * 0.5 * (1.0 + math.cos(math.pi * prog))
  raise ValueError(f"unsupported schedule {kind!r}: constant, linear or cosine")


def distill_step(student: TrainEngine, teacher: TrainEngine, batch: dict, alpha: float | None = None, temperature: float | None = None,
                 step: int | None = None):
  """Online distillation on small models: full logits of both models, loss by autograd through the student's head and
  the engine's layer schedule (the hidden-state gradient is injected with `fwd_bwd_from_hidden_grad`). With `step`
  given, alpha and the temperature follow their configured schedules over `steps`."""
  c = student.config
  if step is not None:
    if alpha is None:
      alpha = scheduled(step, c.steps, c.distill_alpha, c.distill_alpha_end, str(c.distill_alpha_schedule))
    if temperature is None:
      temperature = scheduled(step, c.steps, c.distill_temperature, c.distill_temperature_end, str(c.distill_temperature_schedule))
  alpha = float(c.distill_alpha if alpha is None else alpha)
  temperature = float(c.distill_temperature if temperature is None else temperature)
  with torch.no_grad():
    t_logits = teacher.model.forward(batch["inputs"].to(teacher.device))
  return student.custom_loss_step(batch, lambda logits, targets, mask: O.distillation_loss(
      logits, t_logits.reshape(-1, t_logits.shape[-1]), targets, mask, alpha, temperature))
