"""Token sampling: greedy, weighted (temperature), top-k, nucleus and composite (top-k -> top-p -> temperature)
(src/maxtext/inference/inference_utils.py:125-243)."""
from __future__ import annotations

import torch


def _mask_topk(logits, k):
  if k <= 0 or k >= logits.shape[-1]:
    return logits
  kth = logits.topk(k, dim=-1).values[..., -1:]
  return logits.masked_fill(logits < kth, float("-inf"))


def _mask_nucleus(logits, p):
  if p <= 0 or p >= 1:
    return logits
  sl, idx = logits.sort(dim=-1, descending=True)
  probs = torch.softmax(sl, -1)
  cum = probs.cumsum(-1)
  drop = (cum - probs) >= p                       # keep the smallest prefix whose mass reaches p
  sl = sl.masked_fill(drop, float("-inf"))
  return torch.full_like(logits, float("-inf")).scatter(-1, idx, sl)


def sampling(logits: torch.Tensor, strategy: str = "greedy", topk: int = 0, nucleus_p: float = -1.0, temperature: float = 1.0,
             generator: torch.Generator | None = None) -> torch.Tensor:
  """logits [..., V] -> token ids [...]. On a GPU every strategy is one launch of the sampling kernel (`csrc/sampling_sm100.cu`:
  radix select for top-k, mass select for the nucleus, inverse CDF against one uniform number per row)."""
  if strategy not in ("greedy", "weighted", "topk", "nucleus", "composite"):
    raise ValueError(f"unknown decode_sampling_strategy {strategy}")
  if logits.is_cuda and logits.dtype in (torch.float32, torch.bfloat16):
    from ..ops import backend
    E = backend.ext(required=True)
    flat = logits.reshape(-1, logits.shape[-1])
    flat = flat if flat.is_contiguous() else flat.contiguous()
    greedy = strategy == "greedy"
    u = None if greedy else torch.rand(flat.shape[0], device=flat.device, generator=generator)
    k = int(topk) if strategy in ("topk", "composite") else 0
    p = float(nucleus_p) if strategy in ("nucleus", "composite") else -1.0
    return E.sample_tokens(flat, u, k, p, float(temperature), greedy).reshape(logits.shape[:-1])
  lf = logits.float()
  if strategy == "greedy":
    return lf.argmax(-1)
  t = max(float(temperature), 1e-6)
  if strategy == "weighted":
    pass
  elif strategy == "topk":
    lf = _mask_topk(lf, topk)
  elif strategy == "nucleus":
    lf = _mask_nucleus(lf, nucleus_p)
  elif strategy == "composite":
    lf = _mask_nucleus(_mask_topk(lf, topk), nucleus_p)
  else:
    raise ValueError(f"unknown decode_sampling_strategy {strategy}")
  probs = torch.softmax(lf / t, -1)
  flat = probs.reshape(-1, probs.shape[-1])
  out = torch.multinomial(flat, 1, generator=generator).reshape(probs.shape[:-1])
  return out


def log_prob_of(logits: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
  return torch.log_softmax(logits.float(), -1).gather(-1, tokens.unsqueeze(-1)).squeeze(-1)
