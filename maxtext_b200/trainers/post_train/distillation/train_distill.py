"""Knowledge distillation: `python -m maxtext.trainers.post_train.distillation.train_distill <student.yml> key=value ...`.

Two sources of the teacher's distribution (src/maxtext/trainers/post_train/distillation/train_distill.py:209-842):
  * online  - a second, frozen engine built from `teacher_overrides` (a dict of config keys, e.g. its model_name and
              load_parameters_path) scores every batch;
  * offline - `offline_data_dir` points at top-k logits written by `save_top_k_teacher_logits`; the KL term then runs over
              the teacher's top-k support, renormalised.
The loss is alpha * CE(targets) + (1 - alpha) * T^2 * KL(teacher_T || student_T) with alpha and T on their configured
schedules. Learn-to-init (`student_init_from_teacher: true`): before training, every student tensor whose name and shape
exist in the teacher is copied from it, and stacked-layer tensors take the teacher layers named in `distill_layer_indices`
(lti_utils.py:52 `prepare_student_weights`)."""
from __future__ import annotations

import sys

import torch

from ....config import pyconfig
from ....train import train as train_lib
from ....train.engine import TrainEngine
from ....utils import max_logging
from .. import objectives as O
from ..trainers import scheduled
from .save_top_k_teacher_logits import TopKShardIterator


def top_k_distillation_loss(student_logits, top_vals, top_idx, targets, mask, alpha: float, temperature: float):
  """CE on the targets plus KL over the teacher's top-k support: p_t = softmax(top_vals / T) (renormalised on the k
  entries), q_s = the student's full-vocabulary softmax at temperature T evaluated at those k indices."""
  ce = torch.nn.functional.cross_entropy(student_logits.float(), targets, reduction="none")
  t = float(temperature)
  logp_t = torch.log_softmax(top_vals.float() / t, -1)
  logq_s = torch.log_softmax(student_logits.float() / t, -1).gather(-1, top_idx.long())
  kl = (logp_t.exp() * (logp_t - logq_s)).sum(-1)
  per_tok = alpha * ce + (1.0 - alpha) * t * t * kl
  return (per_tok * mask).sum() / mask.sum().clamp_min(1)


def init_student_from_teacher(student: TrainEngine, teacher: TrainEngine, layer_indices=None) -> int:
  """Copies matching tensors from the teacher; student layer i takes teacher layer layer_indices[i] (default: evenly spaced).
  Returns how many tensors were initialised."""
  s_store, t_store = student.store, teacher.store
  n_s, n_t = int(student.config.num_decoder_layers), int(teacher.config.num_decoder_layers)
  if not layer_indices:
    layer_indices = [round(i * (n_t - 1) / max(1, n_s - 1)) for i in range(n_s)] if n_s > 1 else [n_t - 1]
  copied = 0
  for name, p in s_store.params.items():
    d = p.pdef
    src = name
    if d.layer is not None:
      src = name.replace(f"{d.stack}_{d.layer}/", f"{d.stack}_{layer_indices[d.layer]}/", 1)
    q = t_store.params.get(src)
    if q is None or tuple(q.pdef.shape) != tuple(d.shape):
      continue
    s_store.load_full(name, t_store.full_master(q))           # both engines share the mesh, so the rank-local slices line up
    copied += 1
  s_store.sync_compute_from_master()
  return copied


def train_distill(config, student: TrainEngine | None = None, teacher: TrainEngine | None = None, mesh=None, data_iterator=None):
  c = config
  if student is None:
    c, mesh, student = train_lib.setup(c)
  offline_dir = str(getattr(c, "offline_data_dir", "") or "")
  if teacher is None and not offline_dir:
    over = getattr(c, "teacher_overrides", None) or {}
    assert isinstance(over, dict) and over, "online distillation needs teacher_overrides (or set offline_data_dir)"
    t_cfg = c.replace(**over)
    teacher = TrainEngine(t_cfg, mesh, student.device)
    if t_cfg.load_parameters_path:
      from ....checkpoint import manager as ckpt_lib
      ckpt_lib.load_params_only(t_cfg.load_parameters_path, teacher, mesh)
  if teacher is not None and bool(getattr(c, "student_init_from_teacher", False)):
    idx = getattr(c, "distill_layer_indices", None)
    n = init_student_from_teacher(student, teacher, list(idx) if idx else None)
    max_logging.log(f"learn-to-init: {n} student tensors copied from the teacher")
  rank, world = train_lib.data_shard(mesh)
  if data_iterator is None:
    data_iterator = TopKShardIterator(offline_dir, int(c.global_batch_size_to_load) // world, rank, world) if offline_dir \
        else train_lib.create_data_iterator(c, mesh)
  history = []
  for step in range(int(c.steps)):
    batch = next(data_iterator)
    alpha = scheduled(step, c.steps, c.distill_alpha, c.distill_alpha_end, str(c.distill_alpha_schedule))
    temp = scheduled(step, c.steps, c.distill_temperature, c.distill_temperature_end, str(c.distill_temperature_schedule))
    if "top_k_logits" in batch:
      tv = batch["top_k_logits"].to(student.device).reshape(-1, batch["top_k_logits"].shape[-1])
      ti = batch["top_k_indices"].to(student.device).reshape(-1, batch["top_k_indices"].shape[-1])
      lm = {k: v for k, v in batch.items() if not k.startswith("top_k")}
      m = student.custom_loss_step(lm, lambda logits, targets, mask: top_k_distillation_loss(logits, tv, ti, targets, mask, alpha, temp))
    else:
      with torch.no_grad():
        t_logits = teacher.model.forward(batch["inputs"].to(teacher.device), batch.get("inputs_position"), batch.get("inputs_segmentation"))
      tl = t_logits.reshape(-1, t_logits.shape[-1])
      m = student.custom_loss_step(batch, lambda logits, targets, mask: O.distillation_loss(logits, tl, targets, mask, alpha, temp))
    m["distill/alpha"], m["distill/temperature"] = alpha, temp
    history.append({k: float(v) for k, v in m.items() if _num(v)})
    if step % max(1, int(c.log_period)) == 0:
      max_logging.log(f"distill step {step}: loss {float(m['learning/loss']):.4f} alpha {alpha:.3f} T {temp:.3f}")
  return student, history


def _num(v):
  try:
    float(v)
    return True
  except (TypeError, ValueError):
    return False


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  return train_distill(pyconfig.initialize(argv))


if __name__ == "__main__":
  main()
