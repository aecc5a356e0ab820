"""Engram: conditional memory by hashed n-gram lookup (src/maxtext/layers/engram.py; DeepSeek-AI, "Conditional Memory via
Scalable Lookup", 2026).

  ids -> canonical ids (case / accent / whitespace variants of a token share one id)            CompressedTokenizer
      -> per layer, for every n-gram order 2..N and every head: ((t0*m0) ^ (t1*m1) ^ ...) mod p    NgramHashMapping
         (odd multipliers drawn per layer, a distinct prime modulus per head)
      -> rows of ONE flat embedding table (head offsets added), concatenated                      Engram
      -> key_g = RMSNorm_g(W_k e), query_g = RMSNorm_g(h_g), gate_g = sigmoid(signed sqrt(q.k / sqrt(D)))
      -> out_g = v + SiLU(causal depthwise conv(RMSNorm_g(v))),  v = gate_g * (W_v e)
for each of the G residual streams (G = mhc_expansion_rate; 1 without hyper-connections). The hashing is integer arithmetic
with 32-bit wrap-around, done on the device of the token ids.
"""
from __future__ import annotations

import math
import re
import unicodedata

import numpy as np
import torch

from . import blocks as L


def _is_prime(n: int) -> bool:
  if n < 2:
    return False
  if n % 2 == 0:
    return n == 2
  r = int(math.isqrt(n))
  for d in range(3, r + 1, 2):
    if n % d == 0:
      return False
  return True


def normalize_token_text(text: str) -> str:
  """NFKC -> NFD -> drop combining marks -> lower case -> runs of blanks to one space -> strip (a lone space survives)."""
  t = unicodedata.normalize("NFD", unicodedata.normalize("NFKC", text))
  t = "".join(ch for ch in t if unicodedata.category(ch) != "Mn").lower()
  t = re.sub(r"[ \t\r\n]+", " ", t)
  return " " if t == " " else t.strip()


class CompressedTokenizer:
  """original id -> canonical id (many to one). `tokenizer` needs `vocab_size` and `decode([id])`."""

  def __init__(self, tokenizer):
    n = int(tokenizer.vocab_size)
    table = np.empty(n, dtype=np.int64)
    key2new: dict[str, int] = {}
    for tid in range(n):
      try:
        text = tokenizer.decode([tid])
      except Exception:  # pylint: disable=broad-except
        text = f"<{tid}>"
      if "�" in text:
        key = f"<raw:{tid}>"                       # not valid text on its own (a byte of a multi-byte character): keep it apart
      else:
        key = normalize_token_text(text) or text or f"<empty:{tid}>"
      table[tid] = key2new.setdefault(key, len(key2new))
    self.table_np = table
    self.size = len(key2new)
    self._dev = {}

  def __len__(self):
    return self.size

  def __call__(self, ids: torch.Tensor) -> torch.Tensor:
    t = self._dev.get(ids.device)
    if t is None:
      t = self._dev[ids.device] = torch.from_numpy(self.table_np).to(ids.device)
    ids = ids.long()
    safe = ids.clamp(min=0, max=len(self.table_np) - 1)
    return torch.where(ids < 0, ids, t[safe]).to(torch.int32)


class NgramHashMapping:
  """Hash ids of all engram layers: {layer: [B, S, heads * (N - 1)] int32 in [0, prime of that head)}."""

  LAYER_PRIME_OFFSET = 10007

  def __init__(self, vocab_bases, max_ngram_size: int, num_heads: int, layer_ids, tokenizer, pad_id: int, seed: int):
    self.bases, self.N, self.H, self.layer_ids = [int(v) for v in vocab_bases], int(max_ngram_size), int(num_heads), [int(i) for i in layer_ids]
    assert len(self.bases) >= self.N - 1, "engram_vocab_bases needs one entry per n-gram order (2..max)"
    self.ct = CompressedTokenizer(tokenizer)
    self.pad = int(self.ct.table_np[int(pad_id)])
    m_max = int(np.iinfo(np.int32).max // max(1, len(self.ct)))
    half = max(1, m_max // 2)
    self.multipliers = {}
    for lid in self.layer_ids:
      rng = np.random.default_rng(int(seed + self.LAYER_PRIME_OFFSET * lid))
      self.multipliers[lid] = (rng.integers(low=0, high=half, size=(self.N,), dtype=np.int32) * 2 + 1).astype(np.int32)
    seen, self.primes = set(), {}
    for lid in self.layer_ids:
      per_order = []
      for n in range(2, self.N + 1):
        start, heads = self.bases[n - 2] - 1, []
        for _ in range(self.H):
          c = start + 1
          while c in seen or not _is_prime(c):
            c += 1
          seen.add(c)
          heads.append(c)
          start = c
        per_order.append(heads)
      self.primes[lid] = per_order

  def vocab_sizes(self, layer_id: int) -> list[int]:
    return [p for order in self.primes[layer_id] for p in order]

  def hashes(self, compressed: torch.Tensor, layer_id: int) -> torch.Tensor:
    x = compressed.to(torch.int32)
    B, S = x.shape
    mult = torch.from_numpy(self.multipliers[layer_id]).to(x.device)
    shifted = [x]
    for k in range(1, self.N):
      shifted.append(torch.cat([torch.full((B, min(k, S)), self.pad, dtype=torch.int32, device=x.device), x[:, :max(S - k, 0)]], dim=1))
    h = shifted[0] * mult[0]                         # int32 products wrap around, as in the published hash
    out = []
    for n in range(2, self.N + 1):
      h = torch.bitwise_xor(h, shifted[n - 1] * mult[n - 1])
      mods = torch.tensor(self.primes[layer_id][n - 2], dtype=torch.int32, device=x.device)
      out.append(torch.remainder(h[..., None], mods))  # sign of the divisor: always a valid row
    return torch.cat(out, dim=2)

  def __call__(self, ids: torch.Tensor) -> dict[int, torch.Tensor]:
    c = self.ct(ids)
    return {lid: self.hashes(c, lid) for lid in self.layer_ids}


class Engram:
  """Parameters follow the reference module tree: multi_head_embedding/embedding, key_proj, k_norm, q_norm, value_proj,
  short_conv/{norm, conv}."""

  def __init__(self, b: L.Builder, config, vocab_sizes, name="engram"):
    c = config
    self.c = c
    self.G, self.D = int(getattr(c, "mhc_expansion_rate", 1) or 1), int(c.emb_dim)
    self.N, self.K = int(c.engram_max_ngram_size), int(c.engram_kernel_size)
    self.head_dim = int(c.engram_head_dim)
    self.E = self.head_dim * int(c.engram_num_heads) * (self.N - 1)
    eb = b.sub(name)
    self.offsets_np = np.cumsum([0] + list(vocab_sizes[:-1])).astype(np.int64)
    self.table = eb.sub("multi_head_embedding", "embedding").table("embedding", (int(sum(vocab_sizes)), self.head_dim), ("vocab", "embed"))
    G, D = self.G, self.D
    self.key_proj = eb.sub("key_proj").linear("kernel", (self.E,), (G, D), ("engram_dim", "mhc", "embed"), init="fan_in_normal")
    self.key_bias = eb.sub("key_proj").table("bias", (G, D), ("mhc", "embed"), init="zeros")
    self.k_scale = eb.sub("k_norm").table("scale", (G, D), (None, "norm"), init="ones")
    self.q_scale = eb.sub("q_norm").table("scale", (G, D), (None, "norm"), init="ones")
    self.value_proj = eb.sub("value_proj").linear("kernel", (self.E,), (D,), ("engram_dim", "embed"), init="fan_in_normal")
    self.value_bias = eb.sub("value_proj").vector("bias", D, axes=("embed",), init="zeros")
    self.conv_scale = eb.sub("short_conv", "norm").table("scale", (G, D), (None, "norm"), init="ones")
    self.conv_kernel = eb.sub("short_conv", "conv").table("kernel", (self.K, 1, G * D), (None, None, "embed"), init="zeros")
    self._off = {}

  def _rms(self, x, scale):
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.c.normalization_layer_epsilon) * scale.float()

  def __call__(self, hidden: torch.Tensor, hash_ids: torch.Tensor) -> torch.Tensor:
    """hidden [B, S, G, D] (or [B, S, D] when G = 1), hash_ids [B, S, heads_total] -> same shape as `hidden`."""
    squeeze = hidden.dim() == 3
    if squeeze:
      hidden = hidden.unsqueeze(2)
    B, S, G, D = hidden.shape
    off = self._off.get(hidden.device)
    if off is None:
      off = self._off[hidden.device] = torch.from_numpy(self.offsets_np).to(hidden.device)
    e = self.table.leaf()[(hash_ids.long() + off)].reshape(B, S, self.E)
    key = torch.matmul(e, self.key_proj.leaf().t().to(e.dtype)).view(B, S, G, D) + self.key_bias.leaf().to(e.dtype)
    key = self._rms(key, self.k_scale.leaf())
    query = self._rms(hidden, self.q_scale.leaf())
    gate = (query * key).sum(-1) / math.sqrt(D)
    gate = torch.sigmoid(torch.sqrt(gate.abs().clamp(min=1e-6)) * torch.sign(gate))                      # [B, S, G]
    value = torch.matmul(e, self.value_proj.leaf().t().to(e.dtype)) + self.value_bias.leaf().to(e.dtype)
    gated = gate.unsqueeze(-1) * value.float().unsqueeze(2)                                                # [B, S, G, D]
    # causal depthwise convolution over time, dilation = max n-gram size, on the per-stream normalised values
    xn = self._rms(gated, self.conv_scale.leaf()).reshape(B, S, G * D)
    w = self.conv_kernel.leaf().float().reshape(self.K, G * D)
    dil = self.N
    y = torch.zeros_like(xn)
    for j in range(self.K):
      sh = (self.K - 1 - j) * dil                  # tap j looks `sh` steps back
      if sh < S:
        y = y + torch.nn.functional.pad(xn[:, :S - sh], (0, 0, sh, 0)) * w[j]
    out = (gated + torch.nn.functional.silu(y).view(B, S, G, D)).to(hidden.dtype)
    return out.squeeze(2) if squeeze else out
