"""4-bit NormalFloat quantisation of frozen base weights for QLoRA (`lora.lora_weight_qtype: nf4`, `lora.lora_tile_size`;
src/maxtext/configs/types.py:1590-1598, src/maxtext/utils/lora_utils.py:470-490).

A weight is cut into tiles of `tile` consecutive input-dimension elements; every tile stores its absolute maximum (fp32) and
one 4-bit code per element: the index of the nearest of 16 levels that are the quantiles of a standard normal distribution
rescaled to [-1, 1] (Dettmers et al., "QLoRA", 2023). Two codes share a byte.

`snap_store` rounds every adapted base weight of a parameter store to that grid, so the forward pass computes exactly what a
4-bit base would give; the store keeps its usual fp32 / bf16 copies (frozen parameters are not re-packed), so the memory
saving of a real 4-bit layout is not realised here. `pack` / `unpack` give the 4-bit form for export."""
from __future__ import annotations

import torch

LEVELS = torch.tensor([-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635, -0.18477343022823334,
                       -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725, 0.24611230194568634, 0.33791524171829224,
                       0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0])
DEFAULT_TILE = 64


def _tiles(w: torch.Tensor, tile: int) -> torch.Tensor:
  n = w.shape[-1]
  if n % tile != 0:
    raise ValueError(f"the input dimension ({n}) must be a multiple of lora_tile_size ({tile})")
  return w.reshape(-1, tile)


def quantize(w: torch.Tensor, tile: int = DEFAULT_TILE):
  """w [..., in] -> (codes uint8 [numel] in 0..15, absmax fp32 [numel / tile])."""
  t = _tiles(w.float(), tile)
  absmax = t.abs().amax(1).clamp_min(1e-12)
  x = t / absmax[:, None]
  lv = LEVELS.to(x.device)
  mid = (lv[1:] + lv[:-1]) / 2                       # nearest level = number of midpoints below the value
  codes = torch.bucketize(x, mid).to(torch.uint8)
  return codes.reshape(-1), absmax


def dequantize(codes: torch.Tensor, absmax: torch.Tensor, shape, tile: int = DEFAULT_TILE, dtype=torch.float32) -> torch.Tensor:
  v = LEVELS.to(codes.device)[codes.long()].reshape(-1, tile) * absmax[:, None]
  return v.reshape(shape).to(dtype)


def pack(codes: torch.Tensor) -> torch.Tensor:
  """Two 4-bit codes per byte (even index in the high nibble)."""
  c = codes.reshape(-1, 2)
  return (c[:, 0] << 4 | c[:, 1]).to(torch.uint8)


def unpack(packed: torch.Tensor) -> torch.Tensor:
  return torch.stack([packed >> 4, packed & 0xF], 1).reshape(-1)


def snap(w: torch.Tensor, tile: int = DEFAULT_TILE) -> torch.Tensor:
  codes, absmax = quantize(w, tile)
  return dequantize(codes, absmax, w.shape, tile, w.dtype)


def snap_store(store, config) -> int:
  """Round the base weight of every linear that carries an adapter to the NF4 grid; returns the number of weights changed.
  A no-op unless `lora.lora_weight_qtype` is 'nf4'."""
  d = getattr(config, "lora", None) or {}
  q = str(d.get("lora_weight_qtype") or "").lower() if isinstance(d, dict) else ""
  if not q or q == "none":
    return 0
  if q != "nf4":
    raise ValueError(f"lora_weight_qtype={q!r} is not supported (nf4)")
  tile = int(d.get("lora_tile_size") or DEFAULT_TILE)
  from .lora_utils import adapted
  n = 0
  for p, _, _, _ in adapted(store):
    w = store.full_master(p).float()                 # internal layout [out, in]: tiles run along the input dimension
    store.load_full(p.name, p.pdef.local_slice(snap(w, tile).view(p.pdef.global_shape())))
    n += 1
  if n:
    store.sync_compute_from_master()
  return n
