"""Llama-4 image conventions (src/maxtext/multimodal/processor_llama4.py:25-520).

An image is resized (aspect ratio kept, padded) onto the canvas of `h x w` tiles (tile = 336 pixels, at most 16 tiles)
whose size is closest to the image, cut into those tiles, and a global view (the whole image resized to one tile) is
appended when there is more than one tile. Every tile becomes `(tile / patch * shuffle_ratio)^2` soft tokens (144 for
336 / 14 * 0.5). In the prompt an `<|image|>` placeholder is replaced by

  <|image_start|>  [ patch x n  <|tile_x_separator|> ... <|tile_y_separator|> ]  <|image|>  patch x n  <|image_end|>

where the bracketed rows of local tiles appear only for multi-tile images and the last n patch tokens hold the global
view. `<|patch|>` positions are the ones the projected vision features overwrite."""
from __future__ import annotations

import numpy as np
import torch

TILE_SIZE = 336
MAX_TILES = 16
PATCH_SIZE = 14
PIXEL_SHUFFLE_RATIO = 0.5
IMAGE_MEAN = (0.5, 0.5, 0.5)
IMAGE_STD = (0.5, 0.5, 0.5)
IMAGE_TOKEN = 200090          # <|image|>
BEGIN_IMAGE_TOKEN = 200080    # <|image_start|>
END_IMAGE_TOKEN = 200081      # <|image_end|>
PATCH_TOKEN = 200092          # <|patch|>
TILE_X_SEPARATOR_TOKEN = 200084
TILE_Y_SEPARATOR_TOKEN = 200085


def supported_grids(max_tiles: int = MAX_TILES) -> list[tuple[int, int]]:
  """Every (rows, columns) of tiles with rows * columns <= max_tiles."""
  return [(h, n // h) for n in range(max_tiles, 0, -1) for h in range(1, n + 1) if n % h == 0]


def best_grid(height: int, width: int, tile: int = TILE_SIZE, max_tiles: int = MAX_TILES) -> tuple[int, int]:
  """The canvas whose pixel size is closest (L1) to the image; ties go to the first in `supported_grids` order."""
  return min(supported_grids(max_tiles), key=lambda g: abs(g[0] * tile - height) + abs(g[1] * tile - width))


def tokens_per_tile(tile: int = TILE_SIZE, patch: int = PATCH_SIZE, ratio: float = PIXEL_SHUFFLE_RATIO) -> int:
  return int((tile // patch) * ratio) ** 2


def _resize(t: torch.Tensor, h: int, w: int) -> torch.Tensor:
  return torch.nn.functional.interpolate(t[None], size=(h, w), mode="bilinear", antialias=True, align_corners=False)[0]


def preprocess_image(image, tile: int = TILE_SIZE, max_tiles: int = MAX_TILES) -> tuple[torch.Tensor, tuple[int, int]]:
  """HWC uint8 / float image (or a path) -> (tiles [T, 3, tile, tile] normalised, (rows, columns)); for multi-tile images the
  global view is the last tile."""
  if isinstance(image, str):
    from .processor import load_image
    image = load_image(image)
  arr = np.asarray(image)
  t = torch.as_tensor(arr).float()
  if arr.dtype == np.uint8:
    t = t / 255.0
  t = t.permute(2, 0, 1)
  H, W = t.shape[1:]
  gh, gw = best_grid(H, W, tile, max_tiles)
  ch, cw = gh * tile, gw * tile
  scale = min(ch / H, cw / W)                                      # fit inside the canvas, never distort
  nh, nw = max(1, min(ch, int(round(H * scale)))), max(1, min(cw, int(round(W * scale))))
  canvas = torch.zeros(3, ch, cw)
  canvas[:, :nh, :nw] = _resize(t, nh, nw)
  mean, std = torch.tensor(IMAGE_MEAN).view(3, 1, 1), torch.tensor(IMAGE_STD).view(3, 1, 1)
  canvas = (canvas - mean) / std
  tiles = canvas.view(3, gh, tile, gw, tile).permute(1, 3, 0, 2, 4).reshape(gh * gw, 3, tile, tile)
  if gh * gw > 1:
    tiles = torch.cat([tiles, ((_resize(t, tile, tile) - mean) / std)[None]], dim=0)
  return tiles, (gh, gw)


def image_tokens(grid: tuple[int, int], n: int) -> list[int]:
  """The token run that stands for one image with `grid` local tiles and `n` soft tokens per tile."""
  gh, gw = grid
  out = [BEGIN_IMAGE_TOKEN]
  if gh * gw > 1:
    for _ in range(gh):
      for x in range(gw):
        out += [PATCH_TOKEN] * n
        if x < gw - 1:
          out.append(TILE_X_SEPARATOR_TOKEN)
      out.append(TILE_Y_SEPARATOR_TOKEN)
  out.append(IMAGE_TOKEN)
  out += [PATCH_TOKEN] * n
  out.append(END_IMAGE_TOKEN)
  return out


def prepare(tokens: list[int], images, tile: int = TILE_SIZE, patch: int = PATCH_SIZE, ratio: float = PIXEL_SHUFFLE_RATIO,
            max_tiles: int = MAX_TILES):
  """Prompt ids with one `<|image|>` per image -> (ids [S] for the embedding lookup, image_mask [S], tiles [T, 3, tile, tile]).
  The tiles of all images are concatenated in prompt order, which is the order of the masked positions."""
  n = tokens_per_tile(tile, patch, ratio)
  all_tiles, out = [], []
  it = iter(images)
  for t in tokens:
    if t == IMAGE_TOKEN:
      tl, grid = preprocess_image(next(it), tile, max_tiles)
      all_tiles.append(tl)
      out += image_tokens(grid, n)
    else:
      out.append(t)
  mask = [t == PATCH_TOKEN for t in out]
  pix = torch.cat(all_tiles) if all_tiles else torch.zeros(0, 3, tile, tile)
  assert sum(mask) == n * pix.shape[0]
  return torch.tensor(out), torch.tensor(mask), pix
