"""File-backed input pipeline for dataset_type in {hf, grain, tfds, c4_mlperf, olmo_grain}.

The reference wires Grain / HF datasets / TFDS readers (src/maxtext/input_pipeline/{grain,hf,tfds}_data_processing.py).
Here one reader covers local files of the common formats (jsonl, txt, parquet, and .npy token arrays for the OLMo
style): read -> tokenize -> (optionally) pack -> shift -> batch, sharded across data-parallel ranks by example index,
with an iterator state (epoch, position) that checkpoints save and restore for sample-exact resume.
File selection: `hf_train_files` / `grain_train_files` / `dataset_path` (glob patterns, comma separated)."""
from __future__ import annotations

import glob
import json
import os

import numpy as np
import torch

from . import packing
from .tokenizer import build_tokenizer


def _expand(patterns: str) -> list[str]:
  files = []
  for pat in str(patterns).split(","):
    pat = pat.strip()
    if not pat:
      continue
    if os.path.isdir(pat):
      pat = os.path.join(pat, "*")
    files.extend(sorted(glob.glob(pat)))
  return files


def _read_examples(path: str, column: str):
  if path.endswith(".jsonl") or path.endswith(".json"):
    with open(path, "r", encoding="utf-8") as fh:
      for line in fh:
        line = line.strip()
        if line:
          yield json.loads(line)
  elif path.endswith(".parquet"):
    import pyarrow.parquet as pq
    for batch in pq.ParquetFile(path).iter_batches():
      for row in batch.to_pylist():
        yield row
  elif path.endswith(".npy"):
    arr = np.load(path, mmap_mode="r")
    yield {"__tokens__": arr}
  else:
    with open(path, "r", encoding="utf-8", errors="replace") as fh:
      for line in fh:
        if line.strip():
          yield {column: line.rstrip("\n")}


class FileDataIterator:
  def __init__(self, config, data_rank=0, data_world=1, split="train"):
    c = self.c = config
    pats = (c.hf_train_files or c.grain_train_files or c.dataset_path) if split == "train" else (c.hf_eval_files or c.grain_eval_files or c.dataset_path)
    self.files = _expand(pats)
    if not self.files:
      raise FileNotFoundError(f"dataset_type={c.dataset_type}: no files match {pats!r}")
    self.columns = list(c.train_data_columns if split == "train" else c.eval_data_columns)
    self.column = self.columns[0]
    self.tok = build_tokenizer(c)
    self.rank, self.world, self.split = data_rank, data_world, split
    gb = int(c.global_batch_size_to_load if split == "train" else c.global_batch_size_to_load_eval)
    assert gb % data_world == 0
    self.batch = gb // data_world
    self.S = int(c.max_target_length)
    self.epoch, self.index = 0, 0       # index = examples consumed (globally) in this epoch
    self.pack = bool(c.packing)
    self._rows = self._row_stream()

  def _examples(self):
    """The epoch's examples in training order. With `enable_data_shuffling` the file order is permuted per epoch and the
    examples are permuted inside consecutive windows of 4096, both as pure functions of (data_shuffle_seed, epoch, window),
    so every rank derives the same order and a resumed run continues in it."""
    c = self.c
    shuffle = self.split == "train" and bool(getattr(c, "enable_data_shuffling", False))
    files = list(self.files)
    if not shuffle:
      for f in files:
        yield from _read_examples(f, self.column)
      return
    seed = int(getattr(c, "data_shuffle_seed", 0) or 0)
    rng = np.random.default_rng([seed, self.epoch])
    files = [files[j] for j in rng.permutation(len(files))]
    window, w_id = [], 0

    def flush():
      order = np.random.default_rng([seed, self.epoch, w_id + 1]).permutation(len(window))
      return [window[j] for j in order]
    for f in files:
      for ex in _read_examples(f, self.column):
        window.append(ex)
        if len(window) == 4096:
          yield from flush()
          window, w_id = [], w_id + 1
    if window:
      yield from flush()

  def _token_stream(self):
    """All ranks walk the same example sequence; rank r keeps examples with index % world == r."""
    c = self.c
    while c.num_epoch <= 0 or self.epoch < max(1, int(c.num_epoch)):
      i = 0
      for _once in (0,):
        for ex in self._examples():
          if i >= self.index:
            self.index = i + 1
            if i % self.world == self.rank:
              if "__tokens__" in ex:
                arr = np.asarray(ex["__tokens__"]).reshape(-1)
                for s in range(0, len(arr) - 1, self.S + 1):
                  yield arr[s:s + self.S + 1].astype(np.int32)
              elif bool(getattr(c, "use_sft", False)) and isinstance(ex.get(self.columns[0]), list):
                # chat data: a `messages` column; rendered with the chat template, trained on the last assistant turn
                from . import chat
                if not hasattr(self, "_chat_template"):
                  self._chat_template = chat.load_template(c)
                ptxt, ctxt = chat.split_for_sft(ex[self.columns[0]], self._chat_template)
                pr = [t % c.vocab_size for t in self.tok.encode(ptxt, add_bos=bool(c.add_bos), add_eos=False)]
                co = [t % c.vocab_size for t in self.tok.encode(ctxt, add_bos=False, add_eos=bool(c.add_eos))]
                if bool(getattr(c, "sft_train_on_completion_only", False)):
                  pr = [-(t + 1) for t in pr]
                yield np.asarray((pr + co)[: self.S + 1], dtype=np.int32)
              elif bool(getattr(c, "use_sft", False)) and len(self.columns) >= 2 and self.columns[1] in ex:
                # supervised fine-tuning (`use_sft`, src/maxtext/input_pipeline/input_pipeline_utils.py): prompt + completion in
                # one sequence; with sft_train_on_completion_only the prompt tokens carry no loss
                pr = [t % c.vocab_size for t in self.tok.encode(str(ex[self.columns[0]]), add_bos=bool(c.add_bos), add_eos=False)]
                co = [t % c.vocab_size for t in self.tok.encode(str(ex[self.columns[1]]), add_bos=False, add_eos=bool(c.add_eos))]
                if bool(getattr(c, "sft_train_on_completion_only", False)):
                  pr = [-(t + 1) for t in pr]
                yield np.asarray((pr + co)[: self.S + 1], dtype=np.int32)
              else:
                text = ex[self.column]
                ids = self.tok.encode(text, add_bos=bool(c.add_bos), add_eos=bool(c.add_eos)) if c.tokenize_train_data else list(text)
                ids = [t % c.vocab_size for t in ids]
                yield np.asarray(ids[: self.S + 1] if c.use_truncation else ids, dtype=np.int32)
          i += 1
      self.epoch += 1
      self.index = 0

  def _row_stream(self):
    S1 = self.S + 1
    if self.pack:
      window = []
      for ids in self._token_stream():
        window.append(ids)
        if len(window) >= 8 * self.batch:
          mode = self.c.grain_packing_type
          rows = packing.concat_then_split(window, S1) if mode == "concat_then_split" else \
              packing.pack_first_fit(window, S1, int(self.c.max_segments_per_seq), "best_fit" if mode == "best_fit" else "first_fit")
          yield from rows
          window = []
      if window:
        yield from packing.pack_first_fit(window, S1, int(self.c.max_segments_per_seq))
    else:
      for ids in self._token_stream():
        yield packing._emit([ids[:S1]], S1)

  def __iter__(self):
    return self

  def __next__(self):
    rows = []
    for _ in range(self.batch):
      try:
        rows.append(packing.shift_for_lm(next(self._rows)))
      except StopIteration:
        if not rows:
          raise
        rows.append({k: np.zeros_like(v) for k, v in rows[-1].items()})      # pad the last batch
    return {k: torch.from_numpy(np.stack([r[k] for r in rows]).astype(np.int32)) for k in rows[0]}

  def state(self) -> dict:
    return {"epoch": self.epoch, "index": self.index}

  def load_state(self, st: dict):
    self.epoch, self.index = int(st.get("epoch", 0)), int(st.get("index", 0))
    self._rows = self._row_stream()


def create_file_iterator(config, data_rank=0, data_world=1, split="train"):
  return FileDataIterator(config, data_rank, data_world, split)
