"""Dataset dispatch by `dataset_type` (src/maxtext/input_pipeline/input_pipeline_interface.py:34-120)."""
from __future__ import annotations


def create_data_iterator(config, data_rank: int = 0, data_world: int = 1, split: str = "train"):
  it = _create(config, data_rank, data_world, split)
  if str(getattr(config, "training_objective", "causal_lm")) == "block_diffusion":
    from ..diffusion.block_diffusion.batches import BlockDiffusionIterator
    it = BlockDiffusionIterator(config, it, data_rank)
  if split == "train" and config.enable_rampup_batch_size:
    it = RampupIterator(config, it, data_world)
  return it


def _create(config, data_rank: int = 0, data_world: int = 1, split: str = "train"):
  t = config.dataset_type
  if t == "synthetic":
    from .synthetic import SyntheticDataIterator
    return SyntheticDataIterator(config, data_rank, data_world)
  if t == "olmo_grain" and str(getattr(config, "olmo_index_path", "") or ""):
    # windows of flat token files in a seeded global shuffle (input_pipeline/olmo_data.py); without an index the type reads
    # files like the other file pipelines
    from .olmo_data import OlmoDataIterator
    return OlmoDataIterator(config, data_rank, data_world, split)
  if t in ("hf", "grain", "tfds", "c4_mlperf", "olmo_grain"):
    from .file_pipeline import create_file_iterator
    it = create_file_iterator(config, data_rank, data_world, split)
    depth = int(config.grain_worker_count if split == "train" else config.grain_worker_count_eval) * \
        int(config.grain_per_worker_buffer_size if split == "train" else config.grain_per_worker_buffer_size_eval)
    return PrefetchIterator(it, depth) if depth > 0 else it
  if t == "tokens":
    # pre-tokenized int32 streams (.bin / .npy), packed and prefetched by the native loader (csrc/host/data_loader.cpp)
    from .file_pipeline import _expand
    from .native_loader import NativeTokenIterator
    from .tokenizer import build_tokenizer
    pats = (config.grain_train_files or config.hf_train_files or config.dataset_path) if split == "train" else \
        (config.grain_eval_files or config.hf_eval_files or config.dataset_path)
    files = [f for f in _expand(pats) if f.endswith((".bin", ".npy"))]
    if not files:
      raise FileNotFoundError(f"dataset_type=tokens: no .bin / .npy files match {pats!r}")
    gb = int(config.global_batch_size_to_load if split == "train" else config.global_batch_size_to_load_eval)
    eos = getattr(build_tokenizer(config), "eos_id", None)
    return NativeTokenIterator(files, int(config.max_target_length), gb // data_world, int(eos if eos is not None else 1), data_rank, data_world)
  raise ValueError(f"unknown dataset_type {t}")


class PrefetchIterator:
  """Reads, tokenizes and packs batches on a background thread, `depth` batches ahead of the training loop (the role of Grain's
  worker processes and per-worker buffers, src/maxtext/input_pipeline/grain_data_processing.py: `grain_worker_count` x
  `grain_per_worker_buffer_size` batches in flight). Every queued batch carries the reader state taken right after it was
  produced, so `state()` describes the last batch that was DELIVERED, whatever the thread has read ahead; `load_state`
  stops the thread, repositions the reader and starts over."""

  def __init__(self, inner, depth: int):
    import queue
    import threading
    self.inner, self.depth = inner, max(1, int(depth))
    self._queue_mod, self._threading = queue, threading
    self._state = inner.state()
    self._start()

  def _start(self):
    self._q = self._queue_mod.Queue(maxsize=self.depth)
    self._stop = self._threading.Event()
    # the thread holds the reader, the queue and the stop flag, not this wrapper: dropping the wrapper ends the thread
    self._thread = self._threading.Thread(target=PrefetchIterator._work, args=(self.inner, self._q, self._stop, self._queue_mod.Full),
                                          daemon=True)
    self._thread.start()

  @staticmethod
  def _work(inner, q, stop, full_exc):
    def put(item):
      while not stop.is_set():
        try:
          q.put(item, timeout=0.1)
          return True
        except full_exc:
          continue
      return False
    try:
      while not stop.is_set():
        try:
          batch = next(inner)
        except StopIteration:
          put(("end", None, None))
          return
        if not put(("batch", batch, inner.state())):
          return
    except BaseException as e:  # pylint: disable=broad-except
      put(("error", e, None))

  def __del__(self):
    try:
      self._stop.set()
    except Exception:  # pylint: disable=broad-except
      pass

  def __iter__(self):
    return self

  def __next__(self):
    kind, payload, st = self._q.get()
    if kind == "end":
      self._q.put(("end", None, None))         # stay exhausted
      raise StopIteration
    if kind == "error":
      raise payload
    self._state = st
    return payload

  def state(self):
    return self._state

  def _halt(self):
    self._stop.set()
    while self._thread.is_alive():
      try:
        self._q.get_nowait()
      except self._queue_mod.Empty:
        pass
      self._thread.join(timeout=0.05)

  def load_state(self, st):
    self._halt()
    self.inner.load_state(st)
    self._state = self.inner.state()
    self._start()

  def close(self):
    self._halt()

  def __getattr__(self, name):
    return getattr(self.inner, name)


class RampupIterator:
  """Batch-size ramp-up: start small and grow by a fixed increment every `rampup_samples_per_increment_to_load` samples
  (src/maxtext/common/data_loader.py:104-190 `RampUpDataLoader`, src/maxtext/utils/rampup_batch.py). Full-size batches
  are read from the wrapped iterator into a rolling buffer and handed out in slices of the current size, so no sample is
  skipped or repeated; once the full size is reached the wrapper is a pass-through. Sizes are per data shard."""

  def __init__(self, config, inner, data_world: int = 1):
    self.inner = inner
    c = config
    self.full = int(c.global_batch_size_to_load) // data_world
    self.cur = int(c.global_batch_size_to_load_start) // data_world
    self.inc = int(c.global_batch_size_to_load_increment) // data_world
    self.per_inc = float(c.rampup_samples_per_increment_to_load) / data_world
    assert self.cur >= 1 and self.inc >= 1, "ramp-up sizes must leave at least one row per data shard"
    self.consumed = 0.0          # samples handed out at the current size
    self.buf = None
    self.start = 0
    self.active = self.cur < self.full
    self._before_buf = None      # the wrapped iterator's state just before `buf` was read from it

  def __iter__(self):
    return self

  def _slice(self, batch, lo, hi):
    import torch
    return {k: (v[lo:hi] if torch.is_tensor(v) else v) for k, v in batch.items()}

  def _pull(self):
    self._before_buf = self.inner.state() if hasattr(self.inner, "state") else None
    return next(self.inner)

  def __next__(self):
    import torch
    if not self.active:
      if self.buf is not None and self.start > 0:       # finish the partially used buffer first
        rest = self._slice(self.buf, self.start, self.full)
        nxt = self._pull()
        out = {k: (torch.cat([rest[k], v[: self.start]]) if torch.is_tensor(v) else v) for k, v in nxt.items()}
        self.buf = nxt
        return out
      self.buf = None
      return next(self.inner)
    if self.buf is None:
      self.buf, self.start = self._pull(), 0
    lo, hi = self.start, self.start + self.cur
    if hi > self.full:
      old, self.buf = self.buf, self._pull()
      a, b = self._slice(old, lo, self.full), self._slice(self.buf, 0, hi - self.full)
      out = {k: (torch.cat([a[k], b[k]]) if torch.is_tensor(v) else v) for k, v in old.items()}
      self.start = hi - self.full
    else:
      out = self._slice(self.buf, lo, hi)
      self.start = hi
    self.consumed += self.cur
    if self.consumed >= self.per_inc:
      self.consumed = 0.0
      self.cur = min(self.full, self.cur + self.inc)
      if self.cur >= self.full:
        self.active = False
    return out

  def state(self):
    """With a partly used buffer the wrapped iterator is recorded as it was before that buffer was read, so that a resumed
    run reads the same buffer again and continues at row `start` of it."""
    held = self.buf is not None and (self.active or self.start > 0)
    if held and self._before_buf is not None:
      inner = self._before_buf
    else:
      inner = self.inner.state() if hasattr(self.inner, "state") else {}
    return {"inner": inner, "cur": self.cur, "consumed": self.consumed, "start": self.start if held else 0, "active": self.active,
            "held": held}

  def load_state(self, s):
    if hasattr(self.inner, "load_state"):
      self.inner.load_state(s.get("inner", {}))
    self.cur, self.consumed, self.active = s["cur"], s["consumed"], s["active"]
    self.buf, self.start = None, 0
    if s.get("held"):
      self.buf, self.start = self._pull(), int(s.get("start", 0))
