"""Key/value caches for prefill and autoregressive decoding.

The reference keeps two caches per layer (prefill and AR) with configurable axis orders and merges the two
attention partials (src/maxtext/inference/kvcache.py:249-1137; attention_op.py:2730). On a GPU one contiguous cache
per layer is simpler and faster: `[slots, max_len, kv_heads, head_dim]`, written in place at each slot's current
length; a prefill result is inserted by copying its rows into a slot. Optional int8 / fp8 storage with per
(token, head) scales mirrors `KVQuant` (kvcache.py:49-150). `MlaKVCache` stores the compressed latent and the
shared RoPE key (kvcache.py:1204) and expands them with `wkv_b` at attention time.
"""
from __future__ import annotations

import torch

from ..ops import reference as ref


class KVQuant:
  def __init__(self, dtype: str = "int8"):
    self.kind = dtype
    self.tdtype = torch.int8 if dtype == "int8" else torch.float8_e4m3fn
    self.maxv = 127.0 if dtype == "int8" else 448.0

  def quantize(self, x: torch.Tensor):
    scale = x.float().abs().amax(dim=-1, keepdim=True).clamp_min(1e-8) / self.maxv
    q = x.float() / scale
    q = q.round().clamp(-127, 127).to(torch.int8) if self.kind == "int8" else q.to(self.tdtype)
    return q, scale.to(torch.float32)

  def dequantize(self, q, scale, dtype):
    return (q.float() * scale).to(dtype)


class LayerKVCache:
  """Cache of one attention layer for `slots` concurrent sequences."""

  def __init__(self, slots, max_len, kv_heads, head_dim, v_dim, dtype, device, quant: KVQuant | None = None, seq_group=None,
               seq_rank: int = 0, seq_size: int = 1):
    """`seq_size` > 1 (the `context_autoregressive` mesh axis, src/maxtext/configs/base.yml `ici_context_autoregressive_parallelism`):
    the cache is split along the sequence, position p lives on rank p mod seq_size at row p div seq_size, every rank attends over
    its own rows and the partial results are merged with their log-sum-exp."""
    self.seq_group, self.seq_rank, self.seq_size = seq_group, int(seq_rank), int(seq_size)
    self.global_len = max_len
    if self.seq_size > 1:
      max_len = -(-max_len // self.seq_size)
    self.slots, self.max_len, self.quant = slots, max_len, quant
    sd = quant.tdtype if quant else dtype
    self.dtype = dtype
    self.k = torch.zeros(slots, max_len, kv_heads, head_dim, dtype=sd, device=device)
    self.v = torch.zeros(slots, max_len, kv_heads, v_dim, dtype=sd, device=device)
    if quant:
      self.ks = torch.ones(slots, max_len, kv_heads, 1, dtype=torch.float32, device=device)
      self.vs = torch.ones(slots, max_len, kv_heads, 1, dtype=torch.float32, device=device)
    self.slot_ids: torch.Tensor | None = None     # which cache rows the current batch maps to
    self.lengths: torch.Tensor | None = None      # tokens already cached per batch row (before this call)

  def bind(self, slot_ids, lengths):
    self.slot_ids, self.lengths = slot_ids, lengths

  def rows_for(self, n: int) -> int:
    """Rows of this rank's part that hold a prompt of n tokens."""
    return n if self.seq_size == 1 else -(-n // self.seq_size)

  def _attend_split(self, q, k, v, ctx, window, soft_cap, sinks):
    """Sequence-split cache: write the new tokens this rank owns, attend over the local rows, merge over the ranks."""
    import torch.distributed as dist
    B, S = q.shape[:2]
    N, r = self.seq_size, self.seq_rank
    pos = self.lengths[:, None] + torch.arange(S, device=q.device)[None]
    mine = (pos % N) == r
    rows = self.slot_ids[:, None].expand(B, S)
    for buf, sbuf, x in ((self.k, getattr(self, "ks", None), k), (self.v, getattr(self, "vs", None), v)):
      if self.quant:
        qx, sx = self.quant.quantize(x)
        buf[rows[mine], (pos // N)[mine]] = qx[mine]
        sbuf[rows[mine], (pos // N)[mine]] = sx[mine]
      else:
        buf[rows[mine], (pos // N)[mine]] = x[mine].to(buf.dtype)
    upto = self.rows_for(int((self.lengths.max() + S).item()))
    K, V = self._read(self.k, getattr(self, "ks", None), upto), self._read(self.v, getattr(self, "vs", None), upto)
    kv_pos = (torch.arange(upto, device=q.device) * N + r)[None].expand(B, upto)
    mask = ref.attention_mask(pos, kv_pos, None, None, True, window) & (kv_pos < (self.lengths + S)[:, None])[:, None, None, :]
    if ctx.segment_ids is not None and ctx.mode == "prefill":
      mask = mask & (ctx.segment_ids[:, None, :, None] != 0)
    sk = sinks.data if (sinks is not None and r == 0) else None            # the sink joins the denominator once
    out, lse = ref.attention(q, K, V, mask, 1.0, soft_cap, sinks=sk, return_lse=True)
    empty = ~mask.any(-1)                                                  # [B, 1, S]: no key of this rank is visible
    lse = lse.masked_fill(empty.expand_as(lse), float("-inf")) if sk is None else lse
    outs = [torch.empty_like(out) for _ in range(N)]
    lses = [torch.empty_like(lse) for _ in range(N)]
    dist.all_gather(outs, out.contiguous(), group=self.seq_group)
    dist.all_gather(lses, lse.contiguous(), group=self.seq_group)
    L = torch.stack(lses)                                                  # [N, B, H, S]
    w = torch.softmax(L, 0).nan_to_num(0.0)
    O = torch.stack(outs).float()                                          # [N, B, S, H, D]
    return (O * w.permute(0, 1, 3, 2)[..., None]).sum(0).to(q.dtype)

  def _write(self, buf, sbuf, x, pos):
    B, S = x.shape[:2]
    rows = self.slot_ids[:, None].expand(B, S)
    if self.quant:
      q, s = self.quant.quantize(x)
      buf[rows, pos] = q
      sbuf[rows, pos] = s
    else:
      buf[rows, pos] = x.to(buf.dtype)

  def _decode_kernel_ok(self, q, S, sinks) -> bool:
    if not (q.is_cuda and S == 1 and self.quant is None and sinks is None and q.dtype == torch.bfloat16 and self.k.dtype == torch.bfloat16):
      return False
    from ..ops import backend
    D, g = q.shape[3], q.shape[2] // self.k.shape[2]
    return (backend.use_cuda_kernels(q) and hasattr(backend.ext(), "decode_attention") and D in (64, 128) and self.v.shape[3] == D
            and g <= 16 and q.shape[2] % self.k.shape[2] == 0)

  def _read(self, buf, sbuf, upto):
    x = buf[self.slot_ids, :upto]
    if self.quant:
      return self.quant.dequantize(x, sbuf[self.slot_ids, :upto], self.dtype)
    return x

  def attend(self, q, k, v, ctx, window=0, soft_cap=0.0, sinks=None):
    """Append k/v of the S new tokens at each row's current length, then attend over everything cached."""
    B, S = q.shape[:2]
    if self.seq_size > 1:
      if getattr(ctx, "bidir", None) is not None:
        raise NotImplementedError("a sequence-split cache does not take bidirectional image blocks")
      return self._attend_split(q, k, v, ctx, window, soft_cap, sinks)
    pos = self.lengths[:, None] + torch.arange(S, device=q.device)[None]           # absolute positions of the new tokens
    self._write(self.k, getattr(self, "ks", None), k, pos)
    self._write(self.v, getattr(self, "vs", None), v, pos)
    if self._decode_kernel_ok(q, S, sinks):
      # one new token per sequence: split-KV decode kernel straight on the cache, lengths stay on the device (no host sync)
      from ..ops import backend
      out = torch.empty(B, q.shape[2], q.shape[3], dtype=q.dtype, device=q.device)
      splits = max(1, min(16, 296 // max(1, B * self.k.shape[2])))
      backend.ext().decode_attention(q[:, 0].contiguous(), self.k, self.v, self.slot_ids.to(torch.int32), (self.lengths + 1).to(torch.int32),
                                     out, 1.0, float(soft_cap), int(window), splits)
      return out[:, None]
    upto = int((self.lengths.max() + S).item()) if ctx.mode != "prefill" else int(S + self.lengths.max().item())
    K, V = self._read(self.k, getattr(self, "ks", None), upto), self._read(self.v, getattr(self, "vs", None), upto)
    kv_pos = torch.arange(upto, device=q.device)[None].expand(B, upto)
    valid_len = (self.lengths + S)[:, None]
    mask = ref.attention_mask(pos, kv_pos, None, None, True, window) & (kv_pos < valid_len)[:, None, None, :]
    if ctx.segment_ids is not None and ctx.mode == "prefill":
      mask = mask & (ctx.segment_ids[:, None, :, None] != 0)
      if ctx.segment_ids.shape[1] == upto:
        # several prompts packed into one prefill pass (prefill_concat): a token sees its own prompt only
        mask = mask & (ctx.segment_ids[:, None, :, None] == ctx.segment_ids[:, None, None, :])
    if getattr(ctx, "bidir", None) is not None and ctx.bidir.shape[-2] == S and ctx.bidir.shape[-1] <= upto:
      # multimodal prefill from an empty cache: the soft tokens of one image see each other in both directions
      extra = torch.zeros_like(mask)
      extra[..., : ctx.bidir.shape[-1]] = ctx.bidir
      mask = mask | (extra & (kv_pos < valid_len)[:, None, None, :])
    return ref.attention(q, K, V, mask, 1.0, soft_cap, sinks=sinks.data if sinks is not None else None)


class MlaLayerCache(LayerKVCache):
  """Latent cache: kv_lora_rank + rope_dim numbers per token instead of heads x (qk + v)."""

  def __init__(self, slots, max_len, kv_lora_rank, rope_dim, dtype, device):
    self.slots, self.max_len, self.quant, self.dtype = slots, max_len, None, dtype
    self.seq_group, self.seq_rank, self.seq_size, self.global_len = None, 0, 1, max_len        # latent caches are not split along the sequence
    self.latent = torch.zeros(slots, max_len, kv_lora_rank, dtype=dtype, device=device)
    self.k_rope = torch.zeros(slots, max_len, rope_dim, dtype=dtype, device=device)
    self.slot_ids = self.lengths = None

  def attend_mla(self, q, latent, k_rope, mla, ctx):
    from ..ops import functional as F
    B, S = q.shape[:2]
    pos = self.lengths[:, None] + torch.arange(S, device=q.device)[None]
    rows = self.slot_ids[:, None].expand(B, S)
    self.latent[rows, pos] = latent.to(self.dtype)
    self.k_rope[rows, pos] = k_rope.reshape(B, S, -1).to(self.dtype)
    upto = int((self.lengths.max() + S).item())
    lat, kr = self.latent[self.slot_ids, :upto], self.k_rope[self.slot_ids, :upto]
    kv = F.linear(lat, mla.wkv_b).view(B, upto, mla.h, mla.nope + mla.vd)
    k = torch.cat([kv[..., :mla.nope], kr[:, :, None, :].expand(B, upto, mla.h, mla.rope_d)], dim=-1)
    v = kv[..., mla.nope:]
    kv_pos = torch.arange(upto, device=q.device)[None].expand(B, upto)
    mask = ref.attention_mask(pos, kv_pos) & (kv_pos < (self.lengths + S)[:, None])[:, None, None, :]
    if ctx.segment_ids is not None and ctx.mode == "prefill" and ctx.segment_ids.shape[1] == upto:
      mask = mask & (ctx.segment_ids[:, None, :, None] == ctx.segment_ids[:, None, None, :])      # packed prompts (prefill_concat)
    return ref.attention(q, k, v, mask, 1.0)


def make_caches(model, slots: int, max_len: int, device, quantize: bool = False):
  """One cache per attention block of the model, in layer order."""
  c = model.config
  dt = model.store.compute_dtype
  quant = KVQuant(c.kv_quant_dtype) if (quantize or c.quantize_kvcache) else None
  mesh = getattr(model, "mesh", None)
  seq_size = mesh.axis_size("context_autoregressive") if mesh is not None else 1
  seq = dict(seq_group=mesh.group("context_autoregressive"), seq_rank=mesh.axis_index("context_autoregressive"), seq_size=seq_size) if seq_size > 1 else {}
  out = []
  for layer in model.layers:
    per_layer = []
    for blk in layer.blocks:
      if seq_size > 1 and blk.plan.attention in ("mla", "gdn", "compressed"):
        raise NotImplementedError("context_autoregressive parallelism splits plain key / value caches only")
      if blk.plan.attention == "mla":
        per_layer.append(MlaLayerCache(slots, max_len, c.kv_lora_rank, c.qk_rope_head_dim, dt, device))
      elif blk.plan.attention == "compressed":
        per_layer.append(blk.attn.make_cache(slots, max_len, dt, device))
      elif blk.plan.attention == "gdn":
        from ..layers.gdn import GDNState
        a = blk.attn
        per_layer.append(GDNState(slots, a.conv_dim, a.K, a.hv, a.dk, a.dv, device))
      else:
        a = blk.attn
        per_layer.append(LayerKVCache(slots, max_len, a.hkv_l, a.dh, a.dh, dt, device, quant, **seq))
    out.append(per_layer)
  return out
