"""Convergence runs: turn a throughput recipe into a train-to-target run (benchmarks/convergence/convergence_utils.py and
c4_exp.py in the reference).

A convergence specification is written in SAMPLES and TOKENS so that it does not depend on the batch a machine can hold:
warm-up and decay end in samples, the training budget and the evaluation interval in tokens, the learning rate per sample.
`convergence_recipe` resolves it for a global batch and a GPU count: steps, schedule fractions, per-GPU batch, evaluation
cadence, and the data keys of the named dataset."""
from __future__ import annotations

import dataclasses
import math

from .recipes import Recipe


@dataclasses.dataclass
class DatasetSpec:
  name: str
  dataset_type: str
  dataset_path: str = ""
  dataset_name: str = ""
  eval_dataset_name: str = ""
  train_split: str = "train"
  eval_split: str = "validation"
  eval_tokens: int = 0
  add_bos: bool = False
  add_eos: bool = False


@dataclasses.dataclass
class ConvergenceSpec:
  warmup_samples: int
  decay_end_samples: int
  total_tokens_to_train: int
  learning_rate_per_sample: float
  eval_interval_tokens: int
  eval_tokens: int = -1                 # -1: the dataset's own number
  target_eval_loss: float | None = None
  seed: int = 1238


# the MLPerf C4 split the reference trains GPT-3 / Llama convergence runs on (24 567 evaluation sequences of 2048 tokens)
C4_MLPERF = DatasetSpec("c4mlperf", "c4_mlperf", dataset_name="c4/en:3.0.4", eval_dataset_name="c4/en:3.0.5", train_split="train2",
                        eval_split="validation_24567exp", eval_tokens=24567 * 2048)

LLAMA_C4 = ConvergenceSpec(warmup_samples=8216000, decay_end_samples=12 * 10 ** 6 * 8, total_tokens_to_train=int(1.2e10),
                           learning_rate_per_sample=2e-5 / 1152, eval_interval_tokens=377487360, target_eval_loss=2.69)


def convergence_recipe(recipe: Recipe, dataset: DatasetSpec, spec: ConvergenceSpec, gpus: int, global_batch: int) -> Recipe:
  seq = int(recipe.tuning.get("max_target_length", 2048))
  if global_batch % gpus != 0 and gpus % global_batch != 0:
    raise ValueError(f"global batch {global_batch} does not spread over {gpus} GPUs")
  warm = math.ceil(spec.warmup_samples / global_batch - 1e-6)
  decay_end = max(1, math.ceil(spec.decay_end_samples / global_batch - 1e-6))
  steps = int(spec.total_tokens_to_train / (global_batch * seq))
  eval_tokens = spec.eval_tokens if spec.eval_tokens > 0 else dataset.eval_tokens
  t = dict(recipe.tuning)
  t.update(per_device_batch_size=global_batch / gpus, learning_rate=spec.learning_rate_per_sample * global_batch,
           warmup_steps_fraction=min(1.0, warm / decay_end), learning_rate_schedule_steps=decay_end, steps=steps,
           eval_interval=max(1, math.ceil(spec.eval_interval_tokens / seq / global_batch)),
           eval_steps=max(1, math.ceil(eval_tokens / seq / global_batch)), data_shuffle_seed=spec.seed, reuse_example_batch=0,
           dataset_type=dataset.dataset_type, add_bos=dataset.add_bos, add_eos=dataset.add_eos, train_split=dataset.train_split,
           eval_split=dataset.eval_split, enable_checkpointing="true")
  for k in ("dataset_path", "dataset_name", "eval_dataset_name"):
    if getattr(dataset, k):
      t[k] = getattr(dataset, k)
  if spec.target_eval_loss is not None:
    t["target_eval_loss"] = spec.target_eval_loss
  return Recipe(f"{recipe.name}-{dataset.name}", recipe.model, gpus, t, f"convergence run of {recipe.name} on {dataset.name}")
