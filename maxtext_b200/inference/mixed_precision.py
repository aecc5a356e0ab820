"""Per-matrix weight quantisation maps for serving (`quantization=intmp`, `quant_cfg_path`): the role of
src/maxtext/layers/quantizations.py:567-617 (`_get_mixed_precision_quant_config`) and the JSON files of
src/maxtext/configs/quantization/."""
from __future__ import annotations

import json
import re

import torch

DEFAULT = "__default__"
_BASE = {"w_bits": 8, "a_bits": None, "tile_size": -1, "w_scale": 1.0}


def load_quant_map(path: str) -> list[tuple[str, dict]]:
  """JSON file -> [(pattern, settings)] in file order, `__default__` last; every entry is completed from the defaults."""
  with open(path, "rt", encoding="utf8") as f:
    raw = json.load(f)
  base = dict(_BASE)
  base.update(raw.get(DEFAULT, {}) or {})
  out = []
  for pat, cfg in raw.items():
    if pat == DEFAULT:
      continue
    unknown = set(cfg) - set(_BASE)
    if unknown:
      raise ValueError(f"{path}: unknown keys {sorted(unknown)} for pattern {pat!r}")
    full = dict(base)
    full.update(cfg)
    re.compile(pat)
    out.append((pat, full))
  out.append((DEFAULT, base))
  for _, cfg in out:
    if int(cfg["w_bits"]) not in (4, 8):
      raise ValueError(f"{path}: w_bits must be 4 or 8, got {cfg['w_bits']}")
  return out


def settings_for(name: str, qmap: list[tuple[str, dict]]) -> dict:
  """Settings of the parameter called `name` (its path without the trailing /kernel also matches)."""
  stem = name[:-len("/kernel")] if name.endswith("/kernel") else name
  for pat, cfg in qmap:
    if pat == DEFAULT or re.fullmatch(pat, name) or re.fullmatch(pat, stem):
      return cfg
  return dict(_BASE)


def quantize_weight(w: torch.Tensor, cfg: dict):
  """w [..., out, in] fp32 -> (integers as int8, scales, de-quantised fp32). One scale per output row, or per `tile_size`
  stretch of the contraction dimension when set (scales then have a trailing tile axis)."""
  bits, tile, clip = int(cfg["w_bits"]), int(cfg.get("tile_size", -1) or -1), float(cfg.get("w_scale", 1.0) or 1.0)
  qmax = float(2 ** (bits - 1) - 1)
  n_in = w.shape[-1]
  if tile > 0 and n_in % tile == 0 and tile < n_in:
    wt = w.reshape(*w.shape[:-1], n_in // tile, tile)
  else:
    wt = w.unsqueeze(-2)
  scale = (wt.abs().amax(dim=-1, keepdim=True) * clip).clamp_(min=1e-12) / qmax
  q = torch.clamp(torch.round(wt / scale), -qmax, qmax)
  deq = (q * scale).reshape(w.shape)
  return q.reshape(w.shape).to(torch.int8), scale.squeeze(-1).squeeze(-1) if wt.shape[-2] == 1 else scale.squeeze(-1), deq
