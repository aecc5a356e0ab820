"""Which output position predicts which clean token (src/maxtext/diffusion/block_diffusion/target_alignment.py:21-54), and
the attention pattern of block diffusion (src/maxtext/layers/attention_op.py:1130-1140).

"same_position": the hidden state of a slot predicts that slot's clean token. "shifted": the state of the slot that holds
the PREVIOUS position of the same row predicts it (a next-token head); position 0 falls back to index 0. With explicit
`positions` the previous position is looked up among the valid slots, so rows whose slots are not in position order work too.
"""
from __future__ import annotations

import torch


def source_indices(alignment: str, seq_len: int, positions: torch.Tensor | None = None, validity_mask: torch.Tensor | None = None,
                   batch: int = 1, device=None) -> torch.Tensor | None:
  """[B, S] index of the output slot that scores each target slot, or None when every slot scores itself."""
  if alignment == "same_position":
    return None
  if alignment != "shifted":
    raise ValueError(f"unsupported block-diffusion logit alignment: {alignment}")
  if positions is None:
    idx = (torch.arange(seq_len, device=device) - 1).clamp_(min=0)
    return idx[None].expand(batch, seq_len)
  pos = positions.long()
  if pos.dim() != 2 or pos.shape[1] != seq_len:
    raise ValueError(f"positions must be [batch, {seq_len}], got {tuple(pos.shape)}")
  valid = torch.ones_like(pos, dtype=torch.bool) if validity_mask is None else validity_mask.bool()
  B, S = pos.shape
  # slot_of[b, p] = 1 + the last valid slot that holds position p (0: none)
  slot = torch.where(valid, torch.arange(1, S + 1, device=pos.device)[None].expand(B, S), torch.zeros_like(pos))
  slot_of = torch.zeros(B, S, dtype=torch.long, device=pos.device).scatter_reduce(1, pos.clamp(0, S - 1), slot, reduce="amax")
  prev = (pos - 1).clamp(0, S - 1)
  return (slot_of.gather(1, prev) - 1).clamp_(min=0)


def align_to_targets(x: torch.Tensor, alignment: str, positions=None, validity_mask=None) -> torch.Tensor:
  """x [B, S, ...] (logits or hidden states) re-ordered so that row s is the one that predicts target s."""
  idx = source_indices(alignment, x.shape[1], positions, validity_mask, x.shape[0], x.device)
  if idx is None:
    return x
  return x.gather(1, idx.reshape(idx.shape + (1,) * (x.dim() - 2)).expand(x.shape))


def same_block_mask(positions: torch.Tensor, block_size: int, segment_ids: torch.Tensor | None = None) -> torch.Tensor:
  """[B, 1, S, S] bool: query and key lie in the same diffusion block (and segment). OR-ed with the causal mask it gives the
  block-causal pattern block(q) >= block(k): earlier blocks are fixed context, the active block sees itself in both directions."""
  if block_size <= 0:
    raise ValueError("causal_block_size must be positive for block-diffusion attention")
  blk = positions.long() // int(block_size)
  m = blk[:, :, None] == blk[:, None, :]
  if segment_ids is not None:
    m &= (segment_ids[:, :, None] == segment_ids[:, None, :]) & (segment_ids[:, None, :] != 0)
  return m[:, None]
