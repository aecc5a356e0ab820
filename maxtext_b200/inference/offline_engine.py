"""In-process continuous batching over the decode engine (src/maxtext/inference/offline_engine.py:742-954).

Requests wait in a queue; whenever a slot is free the next prompt is prefilled and inserted, every `generate` call
advances all active slots by one token, finished sequences (EOS or length limit) free their slot at once."""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import torch

from .maxengine import MaxEngine


@dataclass
class Request:
  rid: int
  tokens: list
  max_new_tokens: int = 32
  output: list = field(default_factory=list)
  done: bool = False


class OfflineEngine:
  def __init__(self, engine: MaxEngine, slots: int = 4, eos_id: int = -1, enable_batch_prefill: bool = False,
               batch_prefill_max_batch_size: int = 16):
    """`enable_batch_prefill` packs the prompts that wait for free slots into shared prefill passes
    (src/maxtext/inference/offline_engine.py:749-780, prefill_packing.py)."""
    c = engine.config
    if int(c.max_target_length) - int(c.max_prefill_predict_length) <= 0:
      raise ValueError("Make sure max_target_length - max_prefill_predict_length is greater than 0")      # offline_engine.py:950
    self.eng, self.slots, self.eos_id = engine, slots, eos_id
    self.state = engine.init_decode_state(slots)
    self.queue: deque[Request] = deque()
    self.running: dict[int, Request] = {}
    self.steps = 0
    self.batched = None
    if enable_batch_prefill:
      from .prefill_packing import BatchedPrefillProcessor
      self.batched = BatchedPrefillProcessor(engine, batch_prefill_max_batch_size)

  def submit(self, tokens, max_new_tokens=32) -> Request:
    r = Request(len(self.queue) + len(self.running) + self.steps * 1000, list(tokens), max_new_tokens)
    self.queue.append(r)
    return r

  def _fill_free_slots(self):
    if self.batched is not None:
      return self._fill_free_slots_packed()
    for s in range(self.slots):
      if s in self.running or not self.queue:
        continue
      r = self.queue.popleft()
      t = torch.tensor(r.tokens, dtype=torch.long)
      prefix, first = self.eng.prefill(t, len(r.tokens))
      self.state = self.eng.insert(prefix, self.state, s)
      r.output.append(int(first.data[0, 0]))
      self.running[s] = r
      self._maybe_finish(s)

  def _fill_free_slots_packed(self):
    """All prompts that fit the free slots go through the packing processor; their first tokens arrive by callback."""
    free = [s for s in range(self.slots) if s not in self.running]
    cap = int(self.eng.config.max_prefill_predict_length)
    placed = {}

    def done(results, state):
      for rid, first in results:
        placed[rid].output.append(int(first.reshape(-1)[0]))
    for s in free:
      if not self.queue:
        break
      r = self.queue.popleft()
      placed[r.rid] = r
      self.running[s] = r
      self.state = self.batched.process(self.state, s, r.rid, r.tokens, cap, done)
    self.state = self.batched.flush(self.state, done)
    for s in free:
      self._maybe_finish(s)

  def _maybe_finish(self, s):
    r = self.running.get(s)
    if r is None:
      return
    if len(r.output) >= r.max_new_tokens or r.output[-1] == self.eos_id or not bool(self.state.active[s]):
      r.done = True
      self.eng.free_slot(self.state, s)
      del self.running[s]

  def step(self):
    self._fill_free_slots()
    if not self.running:
      return
    self.state, res = self.eng.generate(self.state)
    self.steps += 1
    for s in list(self.running):
      self.running[s].output.append(int(res.data[s, 0]))
      self._maybe_finish(s)

  def run_until_done(self, max_steps: int = 100000):
    n = 0
    while (self.queue or self.running) and n < max_steps:
      self.step()
      n += 1

  def batch_inference(self, prompts, max_new_tokens=32):
    reqs = [self.submit(p, max_new_tokens) for p in prompts]
    self.run_until_done()
    return [r.output for r in reqs]
