"""Causal-LM batches -> block-diffusion batches (the role of `BlockDiffusionCorruption` in
src/maxtext/input_pipeline/input_pipeline_utils.py:1027-1068 and of the objective switch in hf_data_processing.py:58-93).

The clean row is what the causal batch calls `inputs`; `targets` becomes that clean row (no shift), `inputs` the corrupted
canvas, and `corruption_mask` / `targets_loss_mask` join the batch. The draw for step n depends on (data_shuffle_seed, rank, n)
only, so a restored iterator continues with the masks it would have produced."""
from __future__ import annotations

import numpy as np
import torch

from .corruption import check_contract, corrupt_tokens


def validate(config):
  """Combinations the objective excludes (hf_data_processing.py:73-80): fine-tuning modes and packing."""
  if bool(getattr(config, "use_sft", False)):
    raise ValueError("block diffusion supports pre-training only (use_sft is set)")
  if bool(getattr(config, "use_dpo", False)):
    raise ValueError("block-diffusion pre-training is not compatible with DPO")
  if bool(getattr(config, "packing", False)) and config.dataset_type != "synthetic":
    raise ValueError("block-diffusion pre-training requires packing=false")
  check_contract(int(config.causal_block_size), int(config.block_diffusion_mask_id), float(config.block_diffusion_min_noise),
                 str(config.block_diffusion_logit_alignment), str(config.block_diffusion_canvas_policy))


class BlockDiffusionIterator:
  def __init__(self, config, inner, data_rank: int = 0):
    validate(config)
    self.c, self.inner, self.rank, self.n = config, inner, int(data_rank), 0

  def __iter__(self):
    return self

  def __next__(self):
    b = dict(next(self.inner))
    c = self.c
    clean = b["inputs"].numpy() if torch.is_tensor(b["inputs"]) else np.asarray(b["inputs"])
    seg = b.get("inputs_segmentation")
    valid = (seg.numpy() if torch.is_tensor(seg) else np.asarray(seg)) != 0 if seg is not None else np.ones_like(clean, dtype=bool)
    rng = np.random.default_rng([int(c.data_shuffle_seed), self.rank, self.n])
    self.n += 1
    r = corrupt_tokens(clean, valid, rng, block_size=int(c.causal_block_size), mask_id=int(c.block_diffusion_mask_id),
                       min_noise=float(c.block_diffusion_min_noise), logit_alignment=str(c.block_diffusion_logit_alignment),
                       canvas_policy=str(c.block_diffusion_canvas_policy), axis=1)
    b["targets"] = torch.from_numpy(clean.astype(np.int32))
    b["inputs"] = torch.from_numpy(r.inputs.astype(np.int32))
    b["targets_segmentation"] = torch.from_numpy(valid.astype(np.int32)) if seg is None else torch.as_tensor(seg).to(torch.int32)
    if "inputs_position" in b:
      b["targets_position"] = b["inputs_position"]
    b["corruption_mask"] = torch.from_numpy(r.corruption_mask.astype(np.int32))
    b["targets_loss_mask"] = torch.from_numpy(r.targets_loss_mask.astype(np.int32))
    return b

  def state(self):
    inner = self.inner.state() if hasattr(self.inner, "state") else {}
    return {"inner": inner, "draws": self.n}

  def load_state(self, st):
    self.n = int(st.get("draws", 0))
    if hasattr(self.inner, "load_state"):
      self.inner.load_state(st.get("inner", {}))

  def __getattr__(self, name):
    return getattr(self.inner, name)
