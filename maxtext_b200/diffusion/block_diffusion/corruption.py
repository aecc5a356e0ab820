"""Forward noising of block diffusion (src/maxtext/diffusion/block_diffusion/corruption.py:34-110).

The sequence axis is cut into blocks of `block_size` slots. Every block draws its own noise level u ~ U(min_noise, 1) and
masks each of its eligible slots with probability u; a block that has eligible slots but drew none masks one of them at
random, so every such block is supervised. Eligible = valid (not padding) and, under the "seed_and_mask" canvas, not the
first slot of its block: that slot stays clean as the seed the shifted logits start from, and it is itself a target of the
block before it (except in the first block).

Two pairings are defined: ("same_position", "all_masked") and ("shifted", "seed_and_mask"); anything else is an error.
"""
from __future__ import annotations

from typing import NamedTuple

import numpy as np

CONTRACTS = (("same_position", "all_masked"), ("shifted", "seed_and_mask"))


class Corruption(NamedTuple):
  inputs: np.ndarray                 # the canvas: clean tokens with mask_id at the corrupted slots
  corruption_mask: np.ndarray        # True where a slot was replaced
  targets_loss_mask: np.ndarray      # True where the clean token is a training target (corrupted slots, plus seeds)


def check_contract(block_size: int, mask_id: int, min_noise: float, logit_alignment: str, canvas_policy: str):
  if block_size <= 0:
    raise ValueError(f"block_size must be positive, got {block_size}")
  if mask_id < 0:
    raise ValueError(f"mask_id must be nonnegative, got {mask_id}")
  if not 0.0 < min_noise <= 1.0:
    raise ValueError(f"min_noise must lie in (0, 1], got {min_noise}")
  if (logit_alignment, canvas_policy) not in CONTRACTS:
    raise ValueError(f"block diffusion pairs same_position with all_masked and shifted with seed_and_mask; got {logit_alignment}/{canvas_policy}")
  if canvas_policy == "seed_and_mask" and block_size < 2:
    raise ValueError("seed_and_mask needs blocks of at least 2 slots")


def corrupt_tokens(inputs, validity_mask, rng: np.random.Generator, *, block_size: int, mask_id: int, min_noise: float = 1e-3,
                   logit_alignment: str = "same_position", canvas_policy: str = "all_masked", axis: int = 1) -> Corruption:
  """inputs, validity_mask: same shape, sequence along `axis`. Returns arrays of that shape."""
  tokens = np.asarray(inputs)
  valid = np.asarray(validity_mask).astype(bool)
  if tokens.shape != valid.shape:
    raise ValueError(f"inputs and validity_mask must have identical shapes, got {tokens.shape} and {valid.shape}")
  if tokens.ndim == 0 or not -tokens.ndim <= axis < tokens.ndim:
    raise ValueError(f"axis {axis} is invalid for {tokens.ndim} dimensions")
  if tokens.shape[axis] == 0:
    raise ValueError("the sequence axis must be nonempty")
  check_contract(block_size, mask_id, min_noise, logit_alignment, canvas_policy)
  axis %= tokens.ndim
  S = tokens.shape[axis]
  v = np.moveaxis(valid, axis, -1)
  lead = v.shape[:-1]
  nb = -(-S // block_size)
  elig = np.zeros((int(np.prod(lead, dtype=np.int64)), nb * block_size), dtype=bool)
  elig[:, :S] = v.reshape(-1, S)
  elig = elig.reshape(-1, nb, block_size)
  seeds = np.zeros_like(elig)
  if canvas_policy == "seed_and_mask":
    seeds[:, 1:, 0] = elig[:, 1:, 0]
    elig[:, :, 0] = False
  level = rng.uniform(min_noise, 1.0, size=elig.shape[:2] + (1,))
  chosen = elig & (rng.random(size=elig.shape) < level)
  # an eligible block without a drawn slot gets one eligible slot, uniformly
  tie = np.where(elig, rng.random(size=elig.shape), -1.0)
  empty = elig.any(-1) & ~chosen.any(-1)
  pick = np.zeros_like(elig)
  np.put_along_axis(pick, tie.argmax(-1)[..., None], True, axis=-1)
  chosen |= pick & empty[..., None]

  def back(m):
    return np.moveaxis(m.reshape(-1, nb * block_size)[:, :S].reshape(lead + (S,)), -1, axis)
  cm, lm = back(chosen), back(chosen | seeds)
  return Corruption(np.where(cm, tokens.dtype.type(mask_id), tokens), cm, lm)
