"""Image preprocessing (src/maxtext/multimodal/processor.py, processor_gemma3.py): load, resize, rescale, normalise.

Gemma-3 resizes every image to image_size_for_vit x image_size_for_vit (bilinear, antialiased), scales to [0, 1] and
normalises with mean = std = 0.5 per channel; the result is [N, 3, H, W] float32 (channels first, the layout the vision
tower's patch cutter expects)."""
from __future__ import annotations

import numpy as np
import torch

GEMMA3_MEAN = (0.5, 0.5, 0.5)
GEMMA3_STD = (0.5, 0.5, 0.5)


def load_image(path: str) -> np.ndarray:
  from PIL import Image
  with Image.open(path) as im:
    return np.asarray(im.convert("RGB"))


def preprocess_images(images, size: int, mean=GEMMA3_MEAN, std=GEMMA3_STD) -> torch.Tensor:
  """images: list of paths or HWC uint8 / float arrays -> [N, 3, size, size] float32."""
  out = []
  for im in images:
    if isinstance(im, str):
      im = load_image(im)
    t = torch.as_tensor(np.asarray(im)).float()
    if t.dim() == 2:
      t = t[:, :, None].expand(-1, -1, 3)
    if np.asarray(im).dtype == np.uint8:
      t = t / 255.0
    t = t.permute(2, 0, 1)[None]
    if t.shape[-2:] != (size, size):
      t = torch.nn.functional.interpolate(t, size=(size, size), mode="bilinear", antialias=True, align_corners=False)
    m = torch.tensor(mean).view(1, 3, 1, 1)
    s = torch.tensor(std).view(1, 3, 1, 1)
    out.append(((t - m) / s)[0])
  return torch.stack(out)


def config_images(config) -> torch.Tensor | None:
  """Images named by `image_path` (comma separated), preprocessed for the configured tower; None when there are none."""
  paths = [p for p in str(getattr(config, "image_path", "") or "").split(",") if p]
  if not paths:
    return None
  return preprocess_images(paths, int(config.image_size_for_vit))
