"""Synthetic token batches (dataset_type=synthetic).

Same contract as src/maxtext/input_pipeline/synthetic_data_processing.py:73-132: one fixed batch of
uniform-random token ids of shape (batch, seq+1) drawn from seed 0; inputs = tokens[:, :-1],
targets = tokens[:, 1:], positions = arange, segmentation = ones; the SAME batch is returned every
step. Each rank draws only its slice of the global batch (rows [rank*b, (rank+1)*b) of the global
array) and keeps it in pinned host memory so the per-step copy to the device is asynchronous.
"""
from __future__ import annotations

import torch


class SyntheticDataIterator:
  def __init__(self, config, data_rank: int = 0, data_world: int = 1, batch_size: int | None = None, seed: int = 0,
               pin: bool | None = None):
    self.config = config
    gb = int(batch_size if batch_size is not None else config.global_batch_size_to_load)
    assert gb % data_world == 0, f"global batch {gb} not divisible by {data_world} data shards"
    b = gb // data_world
    S, V = int(config.max_target_length), int(config.vocab_size)
    g = torch.Generator().manual_seed(seed)
    # draw the global array row by row so that every rank sees the same rows regardless of world size
    rows = []
    for r in range(gb):
      row = torch.randint(0, V, (S + 1,), generator=g, dtype=torch.int32)
      if data_rank * b <= r < (data_rank + 1) * b:
        rows.append(row)
    tok = torch.stack(rows)
    pin = torch.cuda.is_available() if pin is None else pin
    def mk(t):
      t = t.contiguous()
      return t.pin_memory() if pin else t
    pos = torch.arange(S, dtype=torch.int32)[None].expand(b, S)
    ones = torch.ones(b, S, dtype=torch.int32)
    self.batch = {
        "inputs": mk(tok[:, :-1]), "targets": mk(tok[:, 1:]),
        "inputs_position": mk(pos), "targets_position": mk(pos),
        "inputs_segmentation": mk(ones), "targets_segmentation": mk(ones),
    }

  def __iter__(self):
    return self

  def __next__(self):
    return self.batch

  def state(self) -> dict:
    return {}

  def load_state(self, state: dict):
    pass
