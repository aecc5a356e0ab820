"""Model-independent helpers of the multimodal path (src/maxtext/multimodal/utils.py:100-200,
src/maxtext/layers/attention_op.py:319-352)."""
from __future__ import annotations

import torch


def merge_mm_embeddings(text_embeddings: torch.Tensor, mm_embeddings: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
  """Put the rows of `mm_embeddings` ([B, N, K, D] or [B, N*K, D]) at the positions where `mask` [B, S] is set, in order.

  Rows of a sequence whose mask has fewer set positions than there are soft tokens use the first ones; a mask with more
  set positions than soft tokens is an error (the prompt promised an image that was not supplied)."""
  B, S, D = text_embeddings.shape
  flat = mm_embeddings.reshape(B, -1, D)
  mask = mask.bool()
  need = int(mask.sum(1).max()) if mask.numel() else 0
  if need > flat.shape[1]:
    raise ValueError(f"{need} image positions in the prompt but only {flat.shape[1]} image embeddings")
  # k-th set position of a row takes the k-th soft token
  order = (mask.long().cumsum(1) - 1).clamp_(min=0)
  picked = torch.gather(flat, 1, order[:, :, None].expand(B, S, D))
  return torch.where(mask[:, :, None], picked.to(text_embeddings.dtype), text_embeddings)


def bidirectional_block_mask(image_mask: torch.Tensor) -> torch.Tensor:
  """[B, S] bool (True at image soft tokens) -> [B, 1, S, S] bool: True where query and key lie in the same contiguous run
  of image tokens. OR-ed with the causal mask this lets the tokens of one image see each other in both directions."""
  m = image_mask.bool()
  prev = torch.nn.functional.pad(m[:, :-1], (1, 0), value=False)
  block = (m & ~prev).long().cumsum(1) * m.long()            # 0 outside images, 1.. for successive runs
  same = (block[:, :, None] == block[:, None, :]) & (block[:, :, None] > 0)
  return same[:, None]


def expand_image_placeholders(tokens: list[int], placeholder_id: int, soft_id: int, n_soft: int, begin_id: int | None = None,
                              end_id: int | None = None) -> list[int]:
  """Replace every placeholder token by [begin] + n_soft soft-token ids + [end] (the Gemma-3 prompt convention: the
  tokenizer sees `<start_of_image>` once per image, the model wants 256 positions to write the image into)."""
  out = []
  for t in tokens:
    if t == placeholder_id:
      if begin_id is not None:
        out.append(begin_id)
      out.extend([soft_id] * n_soft)
      if end_id is not None:
        out.append(end_id)
    else:
      out.append(t)
  return out
