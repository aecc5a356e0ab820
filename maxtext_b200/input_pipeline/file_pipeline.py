"""File-backed input pipeline for dataset_type in {hf, grain, tfds, c4_mlperf, olmo_grain}.

The reference wires Grain / HF datasets / TFDS readers (src/maxtext/input_pipeline/{grain,hf,tfds}_data_processing.py).
Here one reader covers local files of the common formats (jsonl, txt, parquet, Arrow IPC, TFRecord shards of
tf.train.Example, and .npy token arrays for the OLMo style): read -> tokenize -> (optionally) pack -> shift -> batch, sharded across data-parallel ranks by example index,
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
  elif ".tfrecord" in os.path.basename(path):
    # TFDS shards (c4-train.tfrecord-00000-of-01024): tf.train.Example records; token id features pass through as arrays
    from .record_formats import read_tfrecord_examples
    for row in read_tfrecord_examples(path, (column,)):
      v = row.get(column)
      if isinstance(v, np.ndarray):
        yield {"__tokens__": v}
      else:
        yield row
  elif path.endswith(".arrow"):
    from .record_formats import read_arrow
    yield from read_arrow(path)
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
    # dataset_type=hf with hf_path set: the HuggingFace `datasets` library opens the source as a STREAMING dataset
    # (src/maxtext/input_pipeline/hf_data_processing.py:206-240 `load_dataset(hf_path, data_dir, data_files, split, streaming=True)`);
    # rows arrive one at a time, nothing is materialised. hf_path is a builder ("json", "parquet", "text", "csv", "arrow") for
    # local files or a hub name when the machine has network access.
    self.hf_stream = c.dataset_type == "hf" and bool(str(getattr(c, "hf_path", "") or ""))
    if not self.files and not self.hf_stream:
      raise FileNotFoundError(f"dataset_type={c.dataset_type}: no files match {pats!r}")
    self.columns = list(c.train_data_columns if split == "train" else c.eval_data_columns)
    self.column = self.columns[0]
    self.tok = build_tokenizer(c)
    self.rank, self.world, self.split = data_rank, data_world, split
    gb = int(c.global_batch_size_to_load if split == "train" else c.global_batch_size_to_load_eval)
    assert gb % data_world == 0
    self.batch = gb // data_world
    self.S = int(c.max_target_length)
    self.epoch, self.index, self.sub = 0, 0, 0       # next array to read: chunk `sub` of example `index` (global numbering) of `epoch`
    self._sync, self._used = self._pos(), 0
    self.pack = bool(c.packing)
    self._rows = self._row_stream()

  def _examples(self):
    """The epoch's examples in training order. With `enable_data_shuffling` the file order is permuted per epoch and the
    examples are permuted inside consecutive windows of 4096, both as pure functions of (data_shuffle_seed, epoch, window),
    so every rank derives the same order and a resumed run continues in it."""
    c = self.c
    shuffle = self.split == "train" and bool(getattr(c, "enable_data_shuffling", False))
    files = list(self.files)
    if self.hf_stream:
      yield from self._hf_examples(shuffle)
      return
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

  def _hf_examples(self, shuffle: bool):
    """Rows of a streaming HuggingFace dataset in training order; the shuffle is the library's buffered one, seeded by
    (data_shuffle_seed, epoch) so that every rank and a resumed run see the same order."""
    import datasets
    c = self.c
    split = (c.hf_eval_split or "validation") if self.split != "train" else (getattr(c, "hf_train_split", "") or "train")
    kw = dict(split=split, streaming=True)
    if str(c.hf_data_dir or ""):
      kw["data_dir"] = c.hf_data_dir
    if self.files:
      kw["data_files"] = list(self.files)
    if str(getattr(c, "hf_name", "") or ""):
      kw["name"] = c.hf_name
    if str(c.hf_access_token or ""):
      kw["token"] = c.hf_access_token
    ds = datasets.load_dataset(c.hf_path, **kw)
    if shuffle:
      ds = ds.shuffle(seed=int(getattr(c, "data_shuffle_seed", 0) or 0) + self.epoch, buffer_size=int(getattr(c, "hf_shuffle_buffer_size", 0) or 4096))
    yield from ds

  def _encode(self, ex):
    """Token arrays of one example: one array, or consecutive S+1 chunks of a pre-tokenized .npy file."""
    c = self.c
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

  def _token_stream(self):
    """All ranks walk the same example sequence; rank r keeps examples with index % world == r. The reader position is
    (epoch, index, sub): the next array to produce is chunk `sub` of example `index` of that epoch."""
    c = self.c
    while c.num_epoch <= 0 or self.epoch < max(1, int(c.num_epoch)):
      start_i, start_sub = self.index, self.sub
      for i, ex in enumerate(self._examples()):
        if i < start_i:
          continue
        if i % self.world == self.rank:
          for j, ids in enumerate(self._encode(ex)):
            if i == start_i and j < start_sub:
              continue
            self.index, self.sub = i, j + 1
            yield ids
        self.index, self.sub = i + 1, 0
      self.epoch += 1
      self.index, self.sub = 0, 0

  def _pos(self):
    return {"epoch": self.epoch, "index": self.index, "sub": self.sub}

  def _group_stream(self):
    """Yields (reader position before the group, rows of the group). A group is what one packing window produces (or the
    single row of one array without packing): the smallest unit that can be rebuilt from a reader position alone."""
    S1 = self.S + 1
    ts = self._token_stream()
    if not self.pack:
      while True:
        pos = self._pos()
        try:
          ids = next(ts)
        except StopIteration:
          return
        yield pos, [packing._emit([ids[:S1]], S1)]
    # the MLPerf C4 recipe concatenates the tokenised documents and cuts rows of the target length, whatever packing type is
    # configured for the other pipelines (src/maxtext/input_pipeline/tfds_data_processing_c4_mlperf.py `reduce_concat_tokens`
    # + `split_tokens_to_targets_length`)
    mode = "concat_then_split" if self.c.dataset_type == "c4_mlperf" else self.c.grain_packing_type
    while True:
      pos, window = self._pos(), []
      for ids in ts:
        window.append(ids)
        if len(window) >= 8 * self.batch:
          break
      if not window:
        return
      last = len(window) < 8 * self.batch
      if mode == "concat_then_split":
        rows = list(packing.concat_then_split(window, S1))
      else:
        rows = list(packing.pack_first_fit(window, S1, int(self.c.max_segments_per_seq), "best_fit" if mode == "best_fit" and not last else "first_fit"))
      yield pos, rows
      if last:
        return

  def _row_stream(self, skip: int = 0):
    for pos, rows in self._group_stream():
      self._sync, self._used = pos, 0
      for r in rows:
        self._used += 1
        if self._used > skip:
          yield r
      skip = 0

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
    """Position of the last delivered row: the reader position at which the current group began plus the number of its
    rows already handed out. Rebuilding that group and dropping those rows continues exactly where the run stopped, although
    the reader itself runs up to a packing window ahead of what was delivered."""
    return {**self._sync, "used": self._used}

  def load_state(self, st: dict):
    self.epoch, self.index, self.sub = int(st.get("epoch", 0)), int(st.get("index", 0)), int(st.get("sub", 0))
    self._sync, self._used = self._pos(), 0
    self._rows = self._row_stream(skip=int(st.get("used", 0)))


def create_file_iterator(config, data_rank=0, data_world=1, split="train"):
  return FileDataIterator(config, data_rank, data_world, split)
