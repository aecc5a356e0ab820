"""Prefill packing: several short prompts share one prefill pass (src/maxtext/input_pipeline/packing/prefill_packing.py:46-421).

Requests collect in a bucket until the next one would overflow its token capacity or its row count; the bucket is then
prefilled as ONE packed row (`MaxEngine.prefill_concat`: segment ids keep the prompts apart, positions restart per prompt),
each prompt's slice of the cache is inserted into its decode slot, and the caller is told the first token of every request.
"""
from __future__ import annotations

from typing import Callable

import torch

from .maxengine import DecodeState, MaxEngine


class PrefillBucket:
  """Prompts waiting for one packed pass: at most `capacity` tokens in total."""

  def __init__(self, capacity: int):
    if capacity <= 0:
      raise ValueError("capacity must be a positive number.")
    self.capacity = int(capacity)
    self.clear()

  def clear(self):
    self.slots, self.row_ids, self.token_ids, self.length = [], [], [], 0

  def try_add(self, slot: int, row_id: int, token_ids) -> bool:
    if len(token_ids) > self.unallocated():
      return False
    self.add(slot, row_id, token_ids)
    return True

  def add(self, slot: int, row_id: int, token_ids):
    if len(token_ids) > self.unallocated():
      raise ValueError(f"bucket has {self.unallocated()} tokens left, the prompt has {len(token_ids)}")
    self.slots.append(int(slot))
    self.row_ids.append(row_id)
    self.token_ids.append(token_ids)
    self.length += len(token_ids)

  def is_empty(self) -> bool:
    return not self.slots

  def unallocated(self) -> int:
    return self.capacity - self.length

  def __len__(self):
    return len(self.slots)


class PrefillProcessor:
  """One prompt per pass (the unpacked path, kept for prompts that fill a row on their own)."""

  def __init__(self, engine: MaxEngine):
    self.engine = engine

  def process(self, state: DecodeState, slot: int, tokens, true_length: int | None = None):
    t = torch.as_tensor(tokens, dtype=torch.long)
    prefix, first = self.engine.prefill(t, int(true_length or t.numel()))
    return first, self.engine.insert(prefix, state, int(slot))


class BatchedPrefillProcessor:
  def __init__(self, engine: MaxEngine, max_batch_size: int = 16):
    self.engine, self.max_batch_size = engine, int(max_batch_size)
    self.buckets: dict[int, PrefillBucket] = {}
    self.passes = 0                       # packed passes run so far (each replaces len(bucket) single prefills)

  def process(self, state: DecodeState, slot: int, row_id, tokens, capacity: int,
              done: Callable[[list, DecodeState], None] | None = None) -> DecodeState:
    """Queue one prompt for the bucket of `capacity` tokens; a bucket that cannot take it (tokens or rows) is run first."""
    n = len(tokens)
    if n > capacity:
      raise ValueError(f"prompt of {n} tokens exceeds the bucket capacity {capacity}")
    b = self.buckets.setdefault(int(capacity), PrefillBucket(capacity))
    if len(b) >= self.max_batch_size or n > b.unallocated():
      state = self._run(b, state, done)
    b.add(slot, row_id, tokens)
    return state

  def flush(self, state: DecodeState, done: Callable[[list, DecodeState], None] | None = None) -> DecodeState:
    for b in self.buckets.values():
      if not b.is_empty():
        state = self._run(b, state, done)
    return state

  def _run(self, b: PrefillBucket, state: DecodeState, done) -> DecodeState:
    prompts = [torch.as_tensor(t, dtype=torch.long) for t in b.token_ids]
    prefixes = self.engine.prefill_concat(prompts)
    results = []
    for slot, rid, pf in zip(b.slots, b.row_ids, prefixes):
      state = self.engine.insert(pf, state, slot)
      results.append((rid, pf.first_token))
    self.passes += 1
    b.clear()
    if done is not None:
      done(results, state)
    return state
