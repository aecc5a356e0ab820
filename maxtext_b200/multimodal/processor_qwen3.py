"""Qwen3-VL / Qwen3-Omni / Qwen3.5 image conventions (src/maxtext/multimodal/processor_qwen3_omni.py:38-340, 720-857).

An image is resized so that both sides are multiples of patch_size * spatial_merge_size, the pixel count stays inside
[min_pixels, max_pixels] and the aspect ratio is kept as closely as that allows; pixels are scaled to [-1, 1]
((x - 127.5) / 127.5). In the prompt every image is  <|vision_start|> <|image_pad|> x K <|vision_end|>  with
K = (H / patch / merge) * (W / patch / merge); the pad positions receive the merged vision tokens. Video and audio inputs of
the Omni model are not handled here."""
from __future__ import annotations

import math

import numpy as np
import torch

from .processor import load_image

TOKENS = {
    "qwen3.5": dict(vision_start=248053, vision_end=248054, image_pad=248056, video_pad=248057, audio_start=248070, audio_end=248071,
                    audio_pad=248076),
    # Qwen3-VL and Qwen3-Omni vocabularies
    "": dict(vision_start=151652, vision_end=151653, image_pad=151655, video_pad=151656, audio_start=151669, audio_end=151670, audio_pad=151675),
}
MAX_RATIO = 200


def special_tokens(model_name: str) -> dict:
  return next(v for k, v in TOKENS.items() if str(model_name or "").startswith(k))


def smart_resize(height: int, width: int, factor: int, min_pixels: int, max_pixels: int) -> tuple[int, int]:
  if max(height, width) / min(height, width) > MAX_RATIO:
    raise ValueError(f"aspect ratio {max(height, width) / min(height, width):.0f} exceeds {MAX_RATIO}")
  h, w = max(factor, round(height / factor) * factor), max(factor, round(width / factor) * factor)
  if h * w > max_pixels:
    beta = math.sqrt(height * width / max_pixels)
    h, w = max(factor, math.floor(height / beta / factor) * factor), max(factor, math.floor(width / beta / factor) * factor)
  elif h * w < min_pixels:
    beta = math.sqrt(min_pixels / (height * width))
    h, w = math.ceil(height * beta / factor) * factor, math.ceil(width * beta / factor) * factor
  return h, w


def preprocess_image(image, config, size: tuple[int, int] | None = None) -> torch.Tensor:
  """path or HWC uint8 array -> [3, H, W] float32 in [-1, 1] with H, W multiples of patch * merge."""
  if isinstance(image, str):
    image = load_image(image)
  arr = np.asarray(image)
  if arr.ndim == 2:
    arr = np.repeat(arr[:, :, None], 3, 2)
  factor = int(config.patch_size_for_vit) * int(config.spatial_merge_size_for_vit)
  h, w = size or smart_resize(arr.shape[0], arr.shape[1], factor, 4 * factor * factor, 16384 * factor * factor)
  t = torch.as_tensor(arr).float().permute(2, 0, 1)[None]
  if arr.dtype != np.uint8:
    t = t * 255.0
  if t.shape[-2:] != (h, w):
    t = torch.nn.functional.interpolate(t, size=(h, w), mode="bicubic", antialias=True, align_corners=False).clamp_(0, 255)
  return ((t - 127.5) / 127.5)[0]


def tokens_per_image(h: int, w: int, config) -> int:
  f = int(config.patch_size_for_vit) * int(config.spatial_merge_size_for_vit)
  return (h // f) * (w // f)


def prepare(tokens: list[int], images, config):
  """Prompt ids (one <|image_pad|> or <|vision_start|> per image, or none: images are then appended) and raw images ->
  (ids [S], image_mask [S], pixel values [N, 3, H, W]). All images of one prompt are brought to the size of the first."""
  tk = special_tokens(getattr(config, "model_name", ""))
  pix = []
  for im in images:
    pix.append(preprocess_image(im, config, size=tuple(pix[0].shape[-2:]) if pix else None))
  pix = torch.stack(pix)
  K = tokens_per_image(pix.shape[-2], pix.shape[-1], config)
  block = [tk["vision_start"]] + [tk["image_pad"]] * K + [tk["vision_end"]]
  out, used, i = [], 0, 0
  toks = list(tokens)
  while i < len(toks):
    t = toks[i]
    if t == tk["vision_start"] and used < len(images):
      out.extend(block)
      used += 1
      while i + 1 < len(toks) and toks[i + 1] in (tk["image_pad"], tk["vision_end"]):    # drop the collapsed placeholder run
        i += 1
    elif t == tk["image_pad"] and used < len(images):
      out.extend(block)
      used += 1
    else:
      out.append(t)
    i += 1
  for _ in range(len(images) - used):
    out.extend(block)
  mask = [t == tk["image_pad"] for t in out]
  assert sum(mask) == K * len(images)
  return torch.tensor(out), torch.tensor(mask), pix


def rope_index(image_mask, grids) -> torch.Tensor:
  """(temporal, height, width) positions of a prompt with images (`use_mrope`; src/maxtext/multimodal/processor_qwen3_omni.py:1004-1288).

  image_mask [S] marks the soft-token positions; `grids` lists (rows, columns) of merged tokens per image, in prompt order.
  Text tokens count up with the same number on all three axes. The tokens of an image all carry the temporal position at
  which the image starts, their row and column added to it on the other two axes; the text after an image continues at
  start + max(rows, columns)."""
  m = [bool(v) for v in (image_mask.tolist() if hasattr(image_mask, "tolist") else image_mask)]
  out, cur, i, g = [], 0, 0, 0
  while i < len(m):
    if not m[i]:
      out.append((cur, cur, cur))
      cur += 1
      i += 1
      continue
    rows, cols = grids[g]
    g += 1
    n = rows * cols
    assert all(m[i:i + n]) and len(m[i:i + n]) == n, "an image's soft tokens must be one contiguous run of rows * columns positions"
    for r in range(rows):
      for c in range(cols):
        out.append((cur, cur + r, cur + c))
    cur += max(rows, cols)
    i += n
  return torch.tensor(out, dtype=torch.long)


def read_wav(path: str):
  """16-bit PCM .wav -> float32 mono in [-1, 1] and its sampling rate (standard library reader; other formats need converting)."""
  import wave
  import numpy as np
  with wave.open(path, "rb") as fh:
    if fh.getsampwidth() != 2:
      raise ValueError(f"{path}: only 16-bit PCM is read, got {8 * fh.getsampwidth()}-bit samples")
    sr, ch, n = fh.getframerate(), fh.getnchannels(), fh.getnframes()
    data = np.frombuffer(fh.readframes(n), dtype="<i2").astype(np.float32) / 32768.0
  return (data.reshape(-1, ch).mean(1) if ch > 1 else data), sr


def prepare_audio_prompt(ids, waveform, config, model_name: str | None = None):
  """Expand the prompt for one audio clip: `<|audio_start|> <|audio_pad|> x K <|audio_end|>` (appended when the prompt has no
  audio placeholder), K = the number of soft tokens of the clip. Returns (ids, audio_mask, features [mel, frames])."""
  import torch
  from .audio_features import prepare_audio
  tk = special_tokens(model_name or str(config.model_name))
  feats, k = prepare_audio(waveform, config)
  ids = list(ids)
  block = [tk["audio_start"]] + [tk["audio_pad"]] * k + [tk["audio_end"]]
  if tk["audio_pad"] in ids:
    i = ids.index(tk["audio_pad"])
    lo = i - 1 if i > 0 and ids[i - 1] == tk["audio_start"] else i
    hi = i + 2 if i + 1 < len(ids) and ids[i + 1] == tk["audio_end"] else i + 1
    ids = ids[:lo] + block + ids[hi:]
  else:
    ids = ids + block
  t = torch.tensor(ids, dtype=torch.long)
  return t, t == tk["audio_pad"], feats


def prepare_video(ids, frames, config, model_name: str | None = None, size: tuple[int, int] | None = None):
  """frames: [T, H, W, 3] uint8 (already sampled at the wanted rate). Frames are resized like images, grouped into temporal
  patches of `temporal_patch_size_for_vit` frames (the last one repeated to fill a patch), and every patch becomes
  `<|vision_start|> <|video_pad|> x K <|vision_end|>` in the prompt, in place of a `<|video_pad|>` placeholder or appended.
  Returns (ids, mask over the pad positions, pixel tensor [T / TP, TP, 3, H', W']); the tower treats each temporal patch as one
  image whose frames differ (attention stays inside a patch, as for the published model)."""
  tk = special_tokens(model_name or str(config.model_name))
  tp = int(config.temporal_patch_size_for_vit)
  frames = np.asarray(frames)
  if frames.ndim != 4 or frames.shape[-1] != 3:
    raise ValueError(f"frames must be [T, H, W, 3], got {frames.shape}")
  first = preprocess_image(frames[0], config, size)
  pix = [first] + [preprocess_image(f, config, tuple(first.shape[1:])) for f in frames[1:]]
  while len(pix) % tp:
    pix.append(pix[-1])
  video = torch.stack(pix).view(len(pix) // tp, tp, *first.shape)
  unit = int(config.patch_size_for_vit) * int(config.spatial_merge_size_for_vit)
  k = (first.shape[1] // unit) * (first.shape[2] // unit)
  block = []
  for _ in range(video.shape[0]):
    block += [tk["vision_start"]] + [tk["video_pad"]] * k + [tk["vision_end"]]
  ids = list(ids)
  if tk["video_pad"] in ids:
    i = ids.index(tk["video_pad"])
    lo = i - 1 if i > 0 and ids[i - 1] == tk["vision_start"] else i
    hi = i + 2 if i + 1 < len(ids) and ids[i + 1] == tk["vision_end"] else i + 1
    ids = ids[:lo] + block + ids[hi:]
  else:
    ids = ids + block
  t = torch.tensor(ids, dtype=torch.long)
  return t, t == tk["video_pad"], video
