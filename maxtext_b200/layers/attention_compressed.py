"""DeepSeek-V4 compressed attention (src/maxtext/layers/attention_compressed.py:428-1663).

Every layer attends, with one shared key/value head (key = value), over
  * its own tokens inside a sliding window (causal), and, depending on the layer's `compress_ratio` r,
  * r = 128 (HCA): one pooled entry per closed block of r tokens, visible once the whole block lies in the past;
  * r = 4 (CSA): one pooled entry per block of r tokens, pooled over an overlapping window of 2r tokens (the block and the
    one before it), of which an indexer picks the `indexer_topk` best per query;
  * r = 0: nothing more (sliding window only).
A learned per-head sink logit joins the softmax denominator. Pooling is a softmax gate over the tokens of a window (per
channel, with a learned per-slot bias), followed by an RMS norm and the rotary embedding at the block's first position.
Because values carry the rotary embedding too, the attention output is rotated back by the query's position before the
two-step output projection (grouped low-rank map, then a dense map).

Rotary embedding (src/maxtext/layers/embeddings.py:1985-2128): the trailing `qk_rope_head_dim` channels are rotated in
adjacent pairs (2i, 2i + 1); layers with compression use `compressed_rope_max_timescale`, the others `rope_max_timescale`.

Training and cache-free prefill form logits over [window keys | pooled entries] per chunk of queries, so the work is
O(S * (window + chunk + S / r)) and no [S, S] tensor exists. Decoding keeps, per slot, the rotated key = value vectors and the
per-token pooling projections (`CompressedLayerCache`) and rebuilds the pooled entries of complete blocks from them.
"""
from __future__ import annotations

import math

import torch
import torch.utils.checkpoint

from ..ops import functional as F
from . import blocks as L

Q_CHUNK = 1024


def rope_pairs(x: torch.Tensor, positions: torch.Tensor, theta: float, rope_dim: int, reverse: bool = False) -> torch.Tensor:
  """x [B, S, ..., D] (any number of axes between S and D), positions [B, S]: rotate the last `rope_dim` channels in
  adjacent pairs by position * theta^(-2i / rope_dim); `reverse` rotates back."""
  half = rope_dim // 2
  inv = theta ** (-2.0 * torch.arange(half, device=x.device, dtype=torch.float32) / rope_dim)
  ang = positions.float()[..., None] * inv                                   # [B, S, half]
  ang = ang.reshape(ang.shape[:2] + (1,) * (x.dim() - 3) + (half,))
  cos, sin = torch.cos(ang), torch.sin(ang)
  if reverse:
    sin = -sin
  r = x[..., -rope_dim:].float()
  even, odd = r[..., 0::2], r[..., 1::2]
  rot = torch.stack((even * cos - odd * sin, odd * cos + even * sin), dim=-1).flatten(-2)
  return torch.cat([x[..., :-rope_dim], rot.to(x.dtype)], dim=-1)


class _Pool:
  """Projections shared by the pooling modules: kv and gate maps to `mult * dim` channels, a per-slot gate bias and the norm
  of the pooled entry (BaseDeepseekCompressor, attention_compressed.py:428-501)."""

  def __init__(self, b: L.Builder, c, ratio: int, dim: int, mult: int):
    self.c, self.r, self.dim, self.mult = c, int(ratio), int(dim), int(mult)
    self.kv_proj = b.sub("kv_proj").linear("kernel", (c.emb_dim,), (mult * dim,), ("embed", "kv"))
    self.gate_proj = b.sub("gate_proj").linear("kernel", (c.emb_dim,), (mult * dim,), ("embed", "kv"))
    self.position_bias = b.table("position_bias", (self.r, mult * dim), (None, None), init="zeros")
    self.kv_norm = L.Norm(b, "kv_norm", dim, c.normalization_layer_epsilon)

  def project(self, x):
    """x [B, S, D] -> per-token (kv, gate) [B, S, mult * dim] in fp32 (the gate without its slot bias)."""
    return F.linear(x, self.kv_proj).float(), F.linear(x, self.gate_proj).float()

  def windows(self, kv_tok, gate_tok):
    """Per-token projections -> kv, gate [B, n, r, mult * dim] over the whole blocks (gate with its slot bias)."""
    B, S, _ = kv_tok.shape
    n = S // self.r
    use = n * self.r
    kv = kv_tok[:, :use].reshape(B, n, self.r, -1)
    gate = gate_tok[:, :use].reshape(B, n, self.r, -1) + self.position_bias.leaf().float()
    return kv, gate

  def closed(self, x, positions, theta, rope_dim):
    return self.closed_from(*self.project(x), positions, theta, rope_dim, x.dtype)

  def overlapping(self, x, positions, theta, rope_dim):
    return self.overlapping_from(*self.project(x), positions, theta, rope_dim, x.dtype)

  def closed_from(self, kv_tok, gate_tok, positions, theta, rope_dim, dtype):
    """Non-overlapping pooling: [B, n, dim], rotated at each block's first position."""
    kv, gate = self.windows(kv_tok, gate_tok)
    if kv.shape[1] == 0:
      return kv_tok.new_zeros(kv_tok.shape[0], 0, self.dim).to(dtype)
    pooled = (kv * torch.softmax(gate, dim=2)).sum(2)
    pooled = self.kv_norm(pooled.to(dtype))
    return rope_pairs(pooled, positions[:, :kv.shape[1] * self.r:self.r], theta, rope_dim)

  def overlapping_from(self, kv_tok, gate_tok, positions, theta, rope_dim, dtype):
    """Stride-r, width-2r pooling (csa_overlap_pooling, attention_compressed.py:60-161): the first half of the channels of
    block i - 1 and the second half of the channels of block i are gated together. A block that starts a new document
    (its first position does not continue the previous block) pools itself only."""
    kv, gate = self.windows(kv_tok, gate_tok)
    B, n = kv.shape[:2]
    if n == 0:
      return kv_tok.new_zeros(B, 0, self.dim).to(dtype)
    d = self.dim
    start = positions[:, :n * self.r:self.r]
    cont = torch.ones(B, n, dtype=torch.bool, device=kv.device)
    cont[:, 0] = False                                                         # nothing precedes the first block
    cont[:, 1:] = start[:, 1:] == start[:, :-1] + self.r
    prev_kv = torch.cat([kv.new_zeros(B, 1, self.r, d), kv[:, :-1, :, :d]], 1)
    prev_gate = torch.cat([gate.new_full((B, 1, self.r, d), -math.inf), gate[:, :-1, :, :d]], 1)
    prev_kv = torch.where(cont[:, :, None, None], prev_kv, torch.zeros_like(prev_kv))
    prev_gate = torch.where(cont[:, :, None, None], prev_gate, torch.full_like(prev_gate, -math.inf))
    both_kv = torch.cat([prev_kv, kv[..., d:]], 2)                             # [B, n, 2r, d]
    both_gate = torch.cat([prev_gate, gate[..., d:]], 2)
    pooled = (both_kv * torch.softmax(both_gate, dim=2)).sum(2)
    pooled = self.kv_norm(pooled.to(dtype))
    return rope_pairs(pooled, start, theta, rope_dim)


def block_visible(positions: torch.Tensor, n: int, r: int) -> torch.Tensor:
  """[B, S, n] bool: block j (first position p_j) is visible to a query at position p once p_j + r <= p + 1."""
  start = positions[:, :n * r:r]
  return (start[:, None, :] + r) <= (positions[:, :, None] + 1)


def block_visible_at(query_positions: torch.Tensor, n: int, r: int) -> torch.Tensor:
  """As `block_visible` for rows whose cached tokens sit at positions 0, 1, 2, ...: block j starts at j * r."""
  start = torch.arange(n, device=query_positions.device) * r
  return (start[None, None, :] + r) <= (query_positions[:, :, None] + 1)


def block_segments(segment_ids: torch.Tensor | None, n: int, r: int):
  """[B, n] segment of each block, -1 where a block spans two documents (attention_compressed.py:1524-1541)."""
  if segment_ids is None:
    return None
  s = segment_ids[:, :n * r].reshape(segment_ids.shape[0], n, r)
  lo, hi = s.min(-1).values, s.max(-1).values
  return torch.where(lo == hi, lo, torch.full_like(lo, -1))


class V4Indexer:
  """Scores pooled index entries against every query and keeps the best k (DeepseekV4Indexer, attention_compressed.py:665-914)."""

  def __init__(self, b: L.Builder, c, ratio: int):
    self.c, self.r = c, int(ratio)
    self.h, self.d, self.topk = int(c.indexer_n_heads), int(c.indexer_head_dim), int(c.indexer_topk)
    self.q_proj = b.sub("q_proj").linear("kernel", (c.q_lora_rank,), (self.h * self.d,), ("q_lora", "indexer_q"))
    self.pool = _Pool(b, c, ratio, self.d, 2)
    self.weights_proj = b.sub("weights_proj").linear("kernel", (c.emb_dim,), (self.h,), ("embed", "indexer_weights"))

  def scores(self, x, q_latent, positions, theta, rope_dim, keys=None):
    """[B, S, n] fp32 relevance of every pooled block for every query (before masking). `keys` [B, n, d]: pooled index
    entries that the caller already has (decoding from a cache); by default they are pooled from x."""
    B, S, _ = x.shape
    keys = (self.pool.overlapping(x, positions, theta, rope_dim) if keys is None else keys).float()       # [B, n, d]
    q = F.linear(q_latent, self.q_proj).view(B, S, self.h, self.d)
    q = rope_pairs(q, positions, theta, rope_dim).float()
    s = torch.relu(torch.einsum("bshd,bnd->bshn", q, keys)) * self.d ** -0.5
    w = F.linear(x, self.weights_proj).float() * self.h ** -0.5
    return torch.einsum("bshn,bsh->bsn", s, w)

  def select(self, x, q_latent, positions, allowed, theta, rope_dim, keys=None):
    """allowed [B, S, n] bool -> [B, S, n] bool: the (at most) top-k allowed blocks of every query."""
    n = allowed.shape[-1]
    if n == 0:
      return allowed
    with torch.no_grad():
      sc = self.scores(x, q_latent, positions, theta, rope_dim, keys).masked_fill(~allowed, -math.inf)
      k = min(self.topk, n)
      idx = sc.topk(k, dim=-1).indices
      chosen = torch.zeros_like(allowed).scatter_(-1, idx, True)
    return chosen & allowed


class CompressedAttention:
  def __init__(self, b: L.Builder, c, name: str, compress_ratio: int, window: int):
    if b.tp_size > 1:
      raise NotImplementedError("compressed attention is not split over the tensor axis")
    self.c, self.r, self.window = c, int(compress_ratio), int(window)
    D, H, dh, rq = c.emb_dim, c.num_query_heads, c.head_dim, int(c.q_lora_rank)
    self.H, self.dh = H, dh
    self.rope_dim = int(c.qk_rope_head_dim)
    assert 0 < self.rope_dim <= dh and self.rope_dim % 2 == 0, "qk_rope_head_dim must be an even number of channels within head_dim"
    self.theta = float(c.compressed_rope_max_timescale if self.r > 0 else c.rope_max_timescale)
    eps = c.normalization_layer_epsilon
    ab = b.sub(name)
    self.wq_a = ab.sub("wq_a").linear("kernel", (D,), (rq,), ("embed", "q_lora"))
    self.q_norm = L.Norm(ab, "q_norm", rq, eps)
    self.wq_b = ab.sub("wq_b").linear("kernel", (rq,), (H, dh), ("q_lora", "q_heads", "kv"))
    self.q_up_norm = L.Norm(ab, "q_up_norm", dh, eps, with_scale=False)
    self.wkv = ab.sub("wkv").linear("kernel", (D,), (1, dh), ("embed", "kv_heads", "kv_head_dim"))
    self.kv_norm = L.Norm(ab, "kv_norm", dh, eps)
    self.sinks = ab.vector("sinks", H, (None,), init="zeros")
    self.g, self.o_rank = int(c.o_groups), int(c.o_lora_rank)
    self.per_group = H * dh // self.g
    # grouped low-rank output map, reference layout [groups, in per group, rank] (src/maxtext/layers/linears.py:690-773)
    shape = (self.g, self.per_group, self.o_rank)
    self.o_a = ab.sub("o_a_proj")._add("kernel", shape=shape, ref_shape=shape, logical_axes=("o_groups", "q_heads", "o_lora_up_proj"), kind="same",
                                       init="fan_in_normal", init_scale=math.sqrt(self.g / self.per_group))       # variance 1 / (inputs per group)
    self.o_b = ab.sub("o_b_proj").linear("kernel", (self.g * self.o_rank,), (D,), ("o_lora_up_proj", "embed"))
    self.hca = self.csa = self.indexer = None
    if self.r > 4:
      self.hca = _Pool(ab.sub("hca_compressor"), c, self.r, dh, 1)
    elif self.r == 4:
      cb = ab.sub("csa_compressor")
      self.csa = _Pool(cb, c, self.r, dh, 2)
      self.indexer = V4Indexer(cb.sub("indexer"), c, self.r)

  # ---- pieces
  def project(self, x, positions):
    B, S, _ = x.shape
    qn = self.q_norm(F.linear(x, self.wq_a))
    q = self.q_up_norm(F.linear(qn, self.wq_b).view(B, S, self.H, self.dh))
    q = rope_pairs(q, positions, self.theta, self.rope_dim) * self.dh ** -0.5
    kv = self.kv_norm(F.linear(x, self.wkv))
    return q, rope_pairs(kv, positions, self.theta, self.rope_dim), qn

  def pooled(self, x, qn, positions, segment_ids):
    """(entries [B, n, dh], allowed [B, S, n] bool) or (None, None)."""
    if self.r == 0:
      return None, None
    n = x.shape[1] // self.r
    pool = self.hca if self.hca is not None else self.csa
    ent = pool.closed(x, positions, self.theta, self.rope_dim) if self.hca is not None else \
        pool.overlapping(x, positions, self.theta, self.rope_dim)
    allowed = block_visible(positions, n, self.r)
    bs = block_segments(segment_ids, n, self.r)
    if bs is not None:
      allowed = allowed & (segment_ids[:, :, None] == bs[:, None, :]) & (bs[:, None, :] >= 0)
    if self.indexer is not None:
      allowed = self.indexer.select(x, qn, positions, allowed, self.theta, self.rope_dim)
    return ent, allowed

  def _attend(self, q, kv, positions, segment_ids, ent, allowed, s0, s1):
    """Queries s0:s1 over the window keys that can matter to them plus all pooled entries: [B, s1 - s0, H, dh]."""
    k0 = max(0, s0 - self.window + 1) if self.window > 0 else 0
    qp, kp = positions[:, s0:s1, None], positions[:, None, k0:s1]
    m = kp <= qp
    if self.window > 0:
      m = m & (qp - kp < self.window)
    if segment_ids is not None:
      m = m & (segment_ids[:, s0:s1, None] == segment_ids[:, None, k0:s1]) & (segment_ids[:, None, k0:s1] != 0)
    keys = kv[:, k0:s1]
    if ent is not None and ent.shape[1] > 0:
      keys = torch.cat([keys, ent], 1)
      m = torch.cat([m, allowed[:, s0:s1]], -1)
    qf, kf = q[:, s0:s1].float(), keys.float()
    logits = torch.einsum("bshd,bkd->bhsk", qf, kf).masked_fill(~m[:, None], -1e30)
    sink = self.sinks.leaf().float().view(1, -1, 1, 1).expand(logits.shape[0], -1, logits.shape[2], 1)
    p = torch.softmax(torch.cat([logits, sink], -1), -1)[..., :-1]
    p = p.masked_fill(~m[:, None], 0.0)
    return torch.einsum("bhsk,bkd->bshd", p, kf).to(q.dtype)

  def attend(self, q, kv, positions, segment_ids, ent, allowed):
    S = q.shape[1]
    outs = []
    for s0 in range(0, S, Q_CHUNK):
      s1 = min(S, s0 + Q_CHUNK)
      if torch.is_grad_enabled() and S > Q_CHUNK:
        outs.append(torch.utils.checkpoint.checkpoint(self._attend, q, kv, positions, segment_ids, ent, allowed, s0, s1, use_reentrant=False))
      else:
        outs.append(self._attend(q, kv, positions, segment_ids, ent, allowed, s0, s1))
    return outs[0] if len(outs) == 1 else torch.cat(outs, 1)

  def make_cache(self, slots: int, max_len: int, dtype, device) -> "CompressedLayerCache":
    return CompressedLayerCache(self, slots, max_len, dtype, device)

  def _cached(self, x, ctx):
    """Prefill into / decode from a `CompressedLayerCache`: the new tokens' rotated key = value vectors and their pooling
    projections are appended at each row's length; pooled entries are rebuilt from the cached per-token projections of the
    complete blocks, so a decoded token sees exactly what it would see in one full pass."""
    cache = ctx.cache
    if ctx.segment_ids is not None and ctx.mode == "prefill" and bool((ctx.segment_ids != ctx.segment_ids[:, :1]).any()):
      raise NotImplementedError("several prompts packed into one prefill pass are not supported by compressed attention")
    B, S, _ = x.shape
    pos = cache.lengths[:, None] + torch.arange(S, device=x.device)[None]
    q, kv, qn = self.project(x, pos)
    rows = cache.slot_ids[:, None].expand(B, S)
    cache.kv[rows, pos] = kv.to(cache.kv.dtype)
    pool = self.hca if self.hca is not None else self.csa
    if pool is not None:
      pk, pg = pool.project(x)
      cache.pool_kv[rows, pos], cache.pool_gate[rows, pos] = pk, pg
    if self.indexer is not None:
      ik, ig = self.indexer.pool.project(x)
      cache.idx_kv[rows, pos], cache.idx_gate[rows, pos] = ik, ig
    upto = int((cache.lengths.max() + S).item())
    kv_all = cache.kv[cache.slot_ids, :upto]
    kpos = torch.arange(upto, device=x.device)[None].expand(B, upto)
    m = (kpos[:, None, :] <= pos[:, :, None]) & (kpos[:, None, :] < (cache.lengths + S)[:, None, None])
    if self.window > 0:
      m = m & (pos[:, :, None] - kpos[:, None, :] < self.window)
    keys = kv_all
    if pool is not None and upto // self.r > 0:
      n = upto // self.r
      sl = cache.slot_ids
      ent = (pool.closed_from if self.hca is not None else pool.overlapping_from)(
          cache.pool_kv[sl, :upto], cache.pool_gate[sl, :upto], kpos, self.theta, self.rope_dim, x.dtype)
      allowed = block_visible_at(pos, n, self.r)
      if self.indexer is not None:
        ikeys = self.indexer.pool.overlapping_from(cache.idx_kv[sl, :upto], cache.idx_gate[sl, :upto], kpos, self.theta, self.rope_dim, x.dtype)
        allowed = self.indexer.select(x, qn, pos, allowed, self.theta, self.rope_dim, keys=ikeys)
      keys = torch.cat([kv_all, ent], 1)
      m = torch.cat([m, allowed], -1)
    qf, kf = q.float(), keys.float()
    logits = torch.einsum("bshd,bkd->bhsk", qf, kf).masked_fill(~m[:, None], -1e30)
    sink = self.sinks.leaf().float().view(1, -1, 1, 1).expand(B, -1, S, 1)
    p = torch.softmax(torch.cat([logits, sink], -1), -1)[..., :-1].masked_fill(~m[:, None], 0.0)
    out = torch.einsum("bhsk,bkd->bshd", p, kf).to(q.dtype)
    out = rope_pairs(out, pos, self.theta, self.rope_dim, reverse=True)
    grouped = torch.einsum("bsgi,gio->bsgo", out.reshape(B, S, self.g, self.per_group), self.o_a.leaf().to(out.dtype))
    return F.linear(grouped.reshape(B, S, self.g * self.o_rank), self.o_b)

  def __call__(self, x, ctx):
    if ctx.cache is not None:
      return self._cached(x, ctx)
    if ctx.cp_size > 1:
      raise NotImplementedError("compressed attention is not implemented under context parallelism")
    B, S, _ = x.shape
    pos, seg = ctx.positions, ctx.segment_ids
    q, kv, qn = self.project(x, pos)
    ctx.keep("query_proj", q)
    ent, allowed = self.pooled(x, qn, pos, seg)
    out = self.attend(q, kv, pos, seg, ent, allowed)
    out = rope_pairs(out, pos, self.theta, self.rope_dim, reverse=True)       # values carried the rotation: undo it at the query's position
    ctx.keep("context", out)
    grouped = torch.einsum("bsgi,gio->bsgo", out.reshape(B, S, self.g, self.per_group), self.o_a.leaf().to(out.dtype))
    return F.linear(grouped.reshape(B, S, self.g * self.o_rank), self.o_b)


class CompressedLayerCache:
  """Per-slot cache of one compressed-attention layer: the rotated key = value vector of every token, and the per-token
  pooling projections (kv and gate, for the layer's compressor and, in sparse layers, for the indexer) from which the pooled
  entries of complete blocks are rebuilt. `token_buffers` names the [slots, max_len, ...] tensors an engine copies on insert."""

  def __init__(self, attn: CompressedAttention, slots: int, max_len: int, dtype, device):
    self.slots, self.max_len = slots, max_len
    self.kv = torch.zeros(slots, max_len, attn.dh, dtype=dtype, device=device)
    names = ["kv"]
    pool = attn.hca if attn.hca is not None else attn.csa
    if pool is not None:
      w = pool.mult * pool.dim
      self.pool_kv = torch.zeros(slots, max_len, w, dtype=torch.float32, device=device)
      self.pool_gate = torch.zeros(slots, max_len, w, dtype=torch.float32, device=device)
      names += ["pool_kv", "pool_gate"]
    if attn.indexer is not None:
      w = attn.indexer.pool.mult * attn.indexer.pool.dim
      self.idx_kv = torch.zeros(slots, max_len, w, dtype=torch.float32, device=device)
      self.idx_gate = torch.zeros(slots, max_len, w, dtype=torch.float32, device=device)
      names += ["idx_kv", "idx_gate"]
    self.token_buffers = tuple(names)
    self.slot_ids = self.lengths = None

  def bind(self, slot_ids, lengths):
    self.slot_ids, self.lengths = slot_ids, lengths
