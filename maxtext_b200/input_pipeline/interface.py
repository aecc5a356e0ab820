"""Dataset dispatch by `dataset_type` (src/maxtext/input_pipeline/input_pipeline_interface.py:34-120)."""
from __future__ import annotations


def create_data_iterator(config, data_rank: int = 0, data_world: int = 1, split: str = "train"):
  it = _create(config, data_rank, data_world, split)
  if split == "train" and config.enable_rampup_batch_size:
    it = RampupIterator(config, it, data_world)
  return it


def _create(config, data_rank: int = 0, data_world: int = 1, split: str = "train"):
  t = config.dataset_type
  if t == "synthetic":
    from .synthetic import SyntheticDataIterator
    return SyntheticDataIterator(config, data_rank, data_world)
  if t in ("hf", "grain", "tfds", "c4_mlperf", "olmo_grain"):
    from .file_pipeline import create_file_iterator
    return create_file_iterator(config, data_rank, data_world, split)
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
