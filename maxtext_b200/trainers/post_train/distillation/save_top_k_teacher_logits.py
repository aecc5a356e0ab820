"""Offline teacher pass: the top-k logits of a teacher for every token of a dataset, saved in shards.

  python -m maxtext.trainers.post_train.distillation.save_top_k_teacher_logits <teacher.yml> key=value ... \
      --top_k=128 --output_dir=/data/teacher_topk --shard_batches=64

The reference's tool writes ArrayRecord shards of serialized examples (src/maxtext/trainers/post_train/distillation/
save_top_k_teacher_logits.py:55-330); here every shard is one `.npz` with the batch tensors (inputs, targets, optional
segmentation / positions) and `top_k_logits` [N, S, k] (bf16 bits) / `top_k_indices` [N, S, k] (int32), and a
`manifest.json` lists the shards, k, and where to resume (the pass continues after the last complete shard).
`train_distill` reads these directories with `offline_data_dir`."""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

from ....config import pyconfig
from ....train import train as train_lib


@torch.no_grad()
def teacher_top_k(engine, batch: dict, k: int):
  """(values [B,S,k] fp32, indices [B,S,k] int32) of the teacher's logits for a batch."""
  logits = engine.model.forward(batch["inputs"].to(engine.device), batch.get("inputs_position"), batch.get("inputs_segmentation"))
  vals, idx = torch.topk(logits.float(), int(k), dim=-1)
  return vals, idx.to(torch.int32)


def _write_shard(out_dir, n, rows):
  arrs = {key: np.concatenate([r[key] for r in rows]) for key in rows[0]}
  tmp = os.path.join(out_dir, f".shard_{n:05d}.tmp.npz")
  np.savez(tmp, **arrs)
  os.replace(tmp, os.path.join(out_dir, f"shard_{n:05d}.npz"))


def generate_and_save(config, engine, data_iterator, top_k: int, output_dir: str, shard_batches: int = 64, max_batches: int | None = None) -> dict:
  os.makedirs(output_dir, exist_ok=True)
  man_path = os.path.join(output_dir, "manifest.json")
  manifest = {"top_k": int(top_k), "vocab_size": int(config.vocab_size), "seq_len": int(config.max_target_length), "shards": [],
              "batches_done": 0}
  if os.path.isfile(man_path):
    with open(man_path, "r", encoding="utf-8") as fh:
      manifest = json.load(fh)
    assert manifest["top_k"] == int(top_k), "output_dir holds shards of a different k"
  total = int(max_batches if max_batches is not None else config.steps)
  for _ in range(manifest["batches_done"]):          # resume: skip what complete shards already cover
    next(data_iterator)
  rows = []
  done = manifest["batches_done"]
  while done < total:
    batch = next(data_iterator)
    vals, idx = teacher_top_k(engine, batch, top_k)
    row = {"inputs": batch["inputs"].numpy().astype(np.int32), "targets": batch["targets"].numpy().astype(np.int32),
           "top_k_logits": vals.to(torch.bfloat16).view(torch.int16).cpu().numpy(), "top_k_indices": idx.cpu().numpy()}
    for key in ("inputs_segmentation", "targets_segmentation", "inputs_position"):
      if key in batch:
        row[key] = batch[key].numpy().astype(np.int32)
    rows.append(row)
    done += 1
    if len(rows) == shard_batches or done == total:
      n = len(manifest["shards"])
      _write_shard(output_dir, n, rows)
      manifest["shards"].append(f"shard_{n:05d}.npz")
      manifest["batches_done"] = done
      with open(man_path + ".tmp", "w", encoding="utf-8") as fh:
        json.dump(manifest, fh)
      os.replace(man_path + ".tmp", man_path)
      rows = []
  return manifest


class TopKShardIterator:
  """Batches of `batch` rows from a directory written by `generate_and_save`, sharded over data ranks by row, looping."""

  def __init__(self, directory: str, batch: int, data_rank: int = 0, data_world: int = 1):
    with open(os.path.join(directory, "manifest.json"), "r", encoding="utf-8") as fh:
      self.manifest = json.load(fh)
    self.dir, self.batch, self.rank, self.world = directory, int(batch), data_rank, data_world
    self.shard, self.row, self._cur = 0, 0, None

  def __iter__(self):
    return self

  def _load(self):
    if self._cur is None or self._cur[0] != self.shard:
      z = np.load(os.path.join(self.dir, self.manifest["shards"][self.shard]))
      self._cur = (self.shard, {k: z[k][self.rank::self.world] for k in z.files})
    return self._cur[1]

  def __next__(self):
    parts, need = [], self.batch
    while need > 0:
      d = self._load()
      n = len(d["inputs"])
      take = min(need, n - self.row)
      if take > 0:
        parts.append({k: v[self.row:self.row + take] for k, v in d.items()})
        self.row += take
        need -= take
      if self.row >= n:
        self.shard, self.row = (self.shard + 1) % len(self.manifest["shards"]), 0
    out = {k: torch.from_numpy(np.concatenate([p[k] for p in parts])) for k in parts[0]}
    out["top_k_logits"] = out["top_k_logits"].view(torch.bfloat16)
    return out

  def state(self):
    return {"shard": self.shard, "row": self.row}

  def load_state(self, s):
    self.shard, self.row = int(s.get("shard", 0)), int(s.get("row", 0))


def main(argv=None):
  argv = list(sys.argv if argv is None else argv)
  ap = argparse.ArgumentParser(add_help=False)
  ap.add_argument("--top_k", type=int, default=128)
  ap.add_argument("--output_dir", required=True)
  ap.add_argument("--shard_batches", type=int, default=64)
  local, rest = ap.parse_known_args(argv[1:])
  config = pyconfig.initialize([argv[0]] + rest)
  config, mesh, engine = train_lib.setup(config)
  if config.load_parameters_path:
    from ....checkpoint import manager as ckpt_lib
    ckpt_lib.load_params_only(config.load_parameters_path, engine, mesh)
  it = train_lib.create_data_iterator(config, mesh)
  return generate_and_save(config, engine, it, local.top_k, local.output_dir, local.shard_batches)


if __name__ == "__main__":
  main()
