"""OLMo-style token mixes (`dataset_type=olmo_grain`; src/maxtext/input_pipeline/olmo_data.py, olmo_data_grain.py,
olmo_grain_data_processing.py).

A mix is a list of flat token-id files (.npy, or raw arrays of a given dtype). Training instances are the non-overlapping
windows of `max_target_length` tokens of every file (a file's tail that does not fill a window is dropped); an index maps a
global instance number to (file, element offset). One epoch is one random permutation of all instances drawn from
(seed, epoch); data rank r of n takes every n-th entry of it. Because the order is a pure function of (seed, epoch, position),
the reader's whole state is the number of batches delivered.

Instances that contain a span of period 1..13 repeated 32 times or more (degenerate repetitions) stay in the batch, so the
sharding does not move, but their targets are masked (`olmo_apply_ngram_filter`).

  python -m maxtext_b200.input_pipeline.olmo_data --out index.json --sequence-length 8192 [--dtype uint32] FILE...
"""
from __future__ import annotations

import bisect
import hashlib
import json
import os
from dataclasses import asdict, dataclass

import numpy as np
import torch


@dataclass(frozen=True)
class FileEntry:
  path: str
  n_tokens: int
  n_instances: int
  instance_offset: int
  dtype: str
  data_offset: int          # bytes before the first token (the .npy header; 0 for raw files)


@dataclass
class MixIndex:
  sequence_length: int
  files: list

  @property
  def total_instances(self) -> int:
    return self.files[-1].instance_offset + self.files[-1].n_instances if self.files else 0

  def locate(self, instance: int) -> tuple[FileEntry, int]:
    """Global instance number -> (file, index of its first token in that file)."""
    if not 0 <= instance < self.total_instances:
      raise IndexError(instance)
    starts = [f.instance_offset for f in self.files]
    f = self.files[bisect.bisect_right(starts, instance) - 1]
    return f, (instance - f.instance_offset) * self.sequence_length

  def fingerprint(self) -> str:
    h = hashlib.sha256(str(self.sequence_length).encode())
    for f in self.files:
      h.update(f"{os.path.basename(f.path)}:{f.n_tokens}:{f.dtype}".encode())
    return h.hexdigest()[:16]

  def save(self, path: str):
    with open(path, "w") as fh:
      json.dump({"version": "1", "sequence_length": self.sequence_length, "fingerprint": self.fingerprint(),
                 "files": [asdict(f) for f in self.files]}, fh, indent=1)


def _describe(path: str, dtype: str | None):
  """(dtype name, token count, byte offset of the data) of a .npy file, or of a raw array of `dtype`."""
  with open(path, "rb") as fh:
    magic = fh.read(6)
  if magic == b"\x93NUMPY":
    arr = np.load(path, mmap_mode="r")
    if arr.ndim != 1:
      raise ValueError(f"{path}: expected a flat token array, got shape {arr.shape}")
    return arr.dtype.name, int(arr.shape[0]), int(arr.offset)
  if not dtype:
    raise ValueError(f"{path} is not a .npy file: a raw token file needs its dtype")
  item = np.dtype(dtype).itemsize
  size = os.path.getsize(path)
  if size % item:
    raise ValueError(f"{path}: {size} bytes is not a whole number of {dtype} tokens")
  return np.dtype(dtype).name, size // item, 0


def build_index(paths, sequence_length: int, dtype: str | None = None) -> MixIndex:
  files, off = [], 0
  for p in paths:
    dt, n, data_off = _describe(p, dtype)
    k = n // int(sequence_length)
    files.append(FileEntry(p, n, k, off, dt, data_off))
    off += k
  return MixIndex(int(sequence_length), files)


def load_index(path: str, remap_from: str = "", remap_to: str = "") -> MixIndex:
  with open(path) as fh:
    d = json.load(fh)
  files = []
  for f in d["files"]:
    p = f["path"]
    if remap_from and p.startswith(remap_from):
      p = remap_to + p[len(remap_from):]
    files.append(FileEntry(**{**f, "path": p}))
  return MixIndex(int(d["sequence_length"]), files)


def longest_repetition(tokens: np.ndarray, max_period: int = 13, min_period: int = 1) -> int:
  """The largest number of times any span of period p (min_period <= p <= max_period) repeats back to back."""
  t = np.asarray(tokens)
  best = 1
  for p in range(min_period, min(max_period, len(t) // 2) + 1):
    same = t[p:] == t[:-p]
    if not same.any():
      continue
    # longest run of equal-to-p-back: a run of L means L + p tokens with period p
    edges = np.flatnonzero(np.diff(np.concatenate(([0], same.view(np.int8), [0]))))
    run = int((edges[1::2] - edges[0::2]).max())
    best = max(best, (run + p) // p)
  return best


def is_clean_instance(tokens: np.ndarray, max_period: int = 13, min_period: int = 1, max_count: int = 32) -> bool:
  return longest_repetition(tokens, max_period, min_period) < max_count


class OlmoSampler:
  """position (per data rank, unbounded) -> global instance number."""

  def __init__(self, total_instances: int, seed: int, shard_index: int = 0, shard_count: int = 1, shuffle: bool = True):
    self.total, self.seed, self.rank, self.count, self.shuffle = int(total_instances), int(seed), int(shard_index), int(shard_count), shuffle
    self.per_shard = self.total // self.count              # every rank sees the same number of instances per epoch
    if self.per_shard <= 0:
      raise ValueError(f"{self.total} instances cannot feed {self.count} data ranks")
    self._epoch, self._perm = -1, None

  def _permutation(self, epoch: int):
    if epoch != self._epoch:
      self._perm = np.random.default_rng([self.seed, epoch]).permutation(self.total) if self.shuffle else np.arange(self.total)
      self._epoch = epoch
    return self._perm

  def __getitem__(self, position: int) -> int:
    epoch, k = divmod(int(position), self.per_shard)
    return int(self._permutation(epoch)[k * self.count + self.rank])


class OlmoDataIterator:
  """Batches for the pre-training loop: inputs = the window, targets = the window shifted left (last position masked)."""

  def __init__(self, config, data_rank: int = 0, data_world: int = 1, split: str = "train"):
    c = self.c = config
    self.index = load_index(c.olmo_index_path, str(getattr(c, "olmo_path_remap_from", "") or ""), str(getattr(c, "olmo_path_remap_to", "") or ""))
    self.S = int(c.max_target_length)
    if self.index.sequence_length != self.S:
      raise ValueError(f"the index was built for sequence length {self.index.sequence_length}, the run uses {self.S}")
    gb = int(c.global_batch_size_to_load if split == "train" else c.global_batch_size_to_load_eval)
    self.batch = gb // data_world
    self.sampler = OlmoSampler(self.index.total_instances, int(c.data_shuffle_seed), data_rank, data_world,
                               shuffle=bool(c.enable_data_shuffling) and split == "train")
    self.filter = bool(getattr(c, "olmo_apply_ngram_filter", True))
    self.step = 0
    self._maps: dict = {}

  def _tokens(self, instance: int) -> np.ndarray:
    f, start = self.index.locate(instance)
    m = self._maps.get(f.path)
    if m is None:
      m = self._maps[f.path] = np.memmap(f.path, dtype=np.dtype(f.dtype), mode="r", offset=f.data_offset, shape=(f.n_tokens,))
    return np.asarray(m[start:start + self.S])

  def __iter__(self):
    return self

  def __next__(self):
    S = self.S
    inp = np.empty((self.batch, S), dtype=np.int32)
    seg = np.ones((self.batch, S), dtype=np.int32)
    for i in range(self.batch):
      t = self._tokens(self.sampler[self.step * self.batch + i])
      inp[i] = t.astype(np.int32)
      if self.filter and not is_clean_instance(t):
        seg[i] = 0
    self.step += 1
    tgt = np.zeros_like(inp)
    tgt[:, :-1] = inp[:, 1:]
    seg[:, -1] = 0                                           # nothing follows the last token of a window
    pos = np.broadcast_to(np.arange(S, dtype=np.int32), inp.shape).copy()
    out = {"inputs": inp, "targets": tgt, "inputs_position": pos, "targets_position": pos, "inputs_segmentation": np.ones_like(inp),
           "targets_segmentation": seg}
    return {k: torch.from_numpy(v) for k, v in out.items()}

  def state(self) -> dict:
    return {"step": self.step, "fingerprint": self.index.fingerprint()}

  def load_state(self, st: dict):
    if st.get("fingerprint") not in (None, self.index.fingerprint()):
      raise ValueError("the saved reader position belongs to another data mix")
    self.step = int(st.get("step", 0))


def main(argv=None):
  import argparse
  ap = argparse.ArgumentParser()
  ap.add_argument("--out", required=True)
  ap.add_argument("--sequence-length", type=int, required=True)
  ap.add_argument("--dtype", default=None)
  ap.add_argument("files", nargs="+")
  a = ap.parse_args(argv)
  idx = build_index(a.files, a.sequence_length, a.dtype)
  idx.save(a.out)
  print(json.dumps({"files": len(idx.files), "instances": idx.total_instances, "fingerprint": idx.fingerprint()}))


if __name__ == "__main__":
  main()
