"""Gemma-3 prompt and image conventions (src/maxtext/multimodal/processor_gemma3.py:25-260).

The tokenizer emits one `<start_of_image>` (255999) per image in the prompt text. Before the model runs, each of them
becomes  "\\n\\n" <start_of_image> 256 x soft-token <end_of_image> "\\n\\n"  (260 positions per image). The soft-token id
(262144) lies outside the vocabulary: it only marks where the projected image vectors go, so the ids handed to the
embedding lookup carry 0 there and the positions are returned as a mask."""
from __future__ import annotations

import torch

from .processor import preprocess_images
from .utils import expand_image_placeholders

IMAGE_SIZE = 896
BEGIN_IMAGE_TOKEN = 255999
END_IMAGE_TOKEN = 256000
NEW_LINE_TOKEN = 108
SOFT_TOKEN = 262144
SOFT_TOKENS_PER_IMAGE = 256
TOKENS_PER_IMAGE = SOFT_TOKENS_PER_IMAGE + 4


def insert_image_tokens(tokens: list[int]) -> tuple[list[int], list[bool]]:
  """-> (ids for the embedding lookup, mask of soft-token positions)."""
  out = []
  for t in tokens:
    if t == BEGIN_IMAGE_TOKEN:
      out.append(NEW_LINE_TOKEN)
      out.extend(expand_image_placeholders([t], BEGIN_IMAGE_TOKEN, SOFT_TOKEN, SOFT_TOKENS_PER_IMAGE, BEGIN_IMAGE_TOKEN, END_IMAGE_TOKEN))
      out.append(NEW_LINE_TOKEN)
    else:
      out.append(t)
  mask = [t == SOFT_TOKEN for t in out]
  return [0 if m else t for t, m in zip(out, mask)], mask


def prepare(tokens: list[int], images, image_size: int = IMAGE_SIZE):
  """Prompt ids and raw images -> (ids [S], image_mask [S], pixel values [N, 3, H, W])."""
  ids, mask = insert_image_tokens(tokens)
  pix = preprocess_images(images, image_size)
  assert sum(mask) == SOFT_TOKENS_PER_IMAGE * pix.shape[0], "the prompt needs one <start_of_image> per image"
  return torch.tensor(ids), torch.tensor(mask), pix
