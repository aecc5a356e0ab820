"""Decoder building blocks: GQA attention, MLA, dense gated MLP, routed MoE.

Parameter names, reference shapes and logical axes follow MaxText so that checkpoints and sharding
rules carry over (attention kernels src/maxtext/layers/attentions.py:660-830, MLP
src/maxtext/layers/linears.py:422-625, MoE src/maxtext/layers/moe.py:395-615, MLA
src/maxtext/layers/attention_mla.py:785-1115). Storage is `[out, in]` per matrix; q|k|v and
wi_0|wi_1 are adjacent in the unit's flat buffer and are consumed as single fused GEMM operands.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..ops import functional as F
from ..parallel import tp_fused
from ..ops import reference as ref
from ..parallel.param_store import Param, ParamDef, ALIGN


# ------------------------------------------------------------------------------------------ param helpers
class LoraSpec:
  """Which linears get a low-rank adapter (`lora: {enable_lora, lora_rank, lora_alpha, lora_module_path}`,
  src/maxtext/configs/types.py:1575-1600). `lora_module_path` is a regular expression searched in the module path,
  e.g. `layers/.*(self_attention/(query|out)|mlp/(wi_0|wo))`; empty selects the attention and dense-MLP projections."""

  DEFAULT = r"(self_attention|attention)/(query|key|value|out)|mlp/(wi_0|wi_1|wo)"

  def __init__(self, d: dict):
    import re
    self.rank = int(d.get("lora_rank", 0))
    self.alpha = float(d.get("lora_alpha", 0.0)) or float(self.rank)
    self.pattern = re.compile(d.get("lora_module_path") or self.DEFAULT)
    assert self.rank > 0, "enable_lora needs lora_rank > 0"

  def matches(self, b: "Builder", leaf: str) -> bool:
    if leaf != "kernel" or b.layer is None:
      return False
    path = "/".join((str(b.stack),) + tuple(b.prefix))
    return self.pattern.search(path) is not None


def lora_spec(config) -> LoraSpec | None:
  d = getattr(config, "lora", None) or {}
  if not isinstance(d, dict) or not d.get("enable_lora"):
    return None
  s = getattr(config, "_lora_spec", None)
  if s is None:
    s = LoraSpec(d)
    try:
      object.__setattr__(config, "_lora_spec", s)
    except Exception:  # pylint: disable=broad-except
      pass
  return s


class Builder:
  """Collects ParamDefs for one unit while layers are constructed."""

  def __init__(self, config, unit: str, layer: int | None, stack: str | None, tp_size=1, tp_rank=0, ep_size=1, ep_rank=0,
               prefix: tuple = ()):
    self.config, self.unit, self.layer, self.stack = config, unit, layer, stack
    self.tp_size, self.tp_rank, self.ep_size, self.ep_rank = tp_size, tp_rank, ep_size, ep_rank
    self.prefix = tuple(prefix)
    self.params: list[Param] = []

  def sub(self, *names) -> "Builder":
    b = Builder(self.config, self.unit, self.layer, self.stack, self.tp_size, self.tp_rank, self.ep_size, self.ep_rank,
                self.prefix + tuple(names))
    b.params = self.params
    return b

  def _add(self, leaf: str, **kw) -> Param:
    path = self.prefix + (leaf,)
    name = "/".join(((f"{self.stack}_{self.layer}",) if self.layer is not None else ()) + path)
    p = Param(ParamDef(name=name, unit=self.unit, ref_path=path, layer=self.layer, stack=self.stack, tp_rank=self.tp_rank,
                       tp_size=self.tp_size, ep_rank=self.ep_rank, ep_size=self.ep_size, **kw))
    self.params.append(p)
    return p

  def linear(self, leaf, in_shape, out_shape, axes, init="fan_in_trunc", init_scale=1.0, tp: str | None = None) -> Param:
    """Matrix with reference layout [in..., out...]; internal [prod(out), prod(in)].
    tp = "col" splits the first out dim, "row" the first in dim over the tensor-parallel group."""
    in_shape, out_shape = tuple(in_shape), tuple(out_shape)
    n_in, n_out = int(math.prod(in_shape)), int(math.prod(out_shape))
    lo, li = n_out, n_in
    tp_dim = None
    if tp == "col" and self.tp_size > 1:
      assert out_shape[0] % self.tp_size == 0, f"{leaf}: {out_shape} not divisible by tp {self.tp_size}"
      lo, tp_dim = n_out // self.tp_size, 0
    elif tp == "row" and self.tp_size > 1:
      assert in_shape[0] % self.tp_size == 0
      li, tp_dim = n_in // self.tp_size, 1
    p = self._add(leaf, shape=(lo, li), ref_shape=in_shape + out_shape, logical_axes=tuple(axes), kind="linear",
                  n_in_dims=len(in_shape), init=init, init_scale=init_scale, tp_dim=tp_dim)
    spec = lora_spec(self.config)
    if spec is not None and spec.matches(self, leaf):
      # W x + (alpha / r) B (A x): A [r, in] drawn like a dense kernel, B [out, r] zero, so training starts at the base model.
      # Under tensor parallelism the adapter follows its weight: a column-split W (outputs divided) gets a whole A and a B split
      # along the outputs; a row-split W (inputs divided) gets an A split along the inputs and a whole B, whose product is a
      # partial sum that joins W's own all-reduce. The whole factor sees rank-local data, so its gradient is a partial sum.
      r = spec.rank
      col = tp == "col" and self.tp_size > 1
      row = tp == "row" and self.tp_size > 1
      a = self._add(leaf + "_lora_a", shape=(r, li), ref_shape=in_shape + (r,), logical_axes=tuple(axes[:len(in_shape)]) + (None,),
                    kind="linear", n_in_dims=len(in_shape), init="fan_in_normal", tp_dim=1 if row else None)
      b = self._add(leaf + "_lora_b", shape=(lo, r), ref_shape=(r,) + out_shape, logical_axes=(None,) + tuple(axes[len(in_shape):]),
                    kind="linear", n_in_dims=1, init="zeros", tp_dim=0 if col else None)
      if col:
        a.pdef.tp_partial = True
      if row:
        b.pdef.tp_partial = True
      p.lora = (a, b, spec.alpha / r)
    return p

  def vector(self, leaf, n, axes=("norm",), init="ones", tp=False) -> Param:
    ln = n // self.tp_size if tp and self.tp_size > 1 else n
    return self._add(leaf, shape=(ln,), ref_shape=(n,), logical_axes=tuple(axes), kind="same", init=init,
                     tp_dim=0 if (tp and self.tp_size > 1) else None)

  def table(self, leaf, shape, axes, init="embed") -> Param:
    return self._add(leaf, shape=tuple(shape), ref_shape=tuple(shape), logical_axes=tuple(axes), kind="same", init=init)

  def experts(self, leaf, num_experts, d_in, d_out, axes, tp: str | None = None) -> Param:
    """Expert weights, reference [E, in, out]; internal [E_local, out, in]."""
    assert num_experts % self.ep_size == 0
    el = num_experts // self.ep_size
    lo, li = d_out, d_in
    if tp == "col" and self.tp_size > 1:
      lo = d_out // self.tp_size
    elif tp == "row" and self.tp_size > 1:
      li = d_in // self.tp_size
    return self._add(leaf, shape=(el, lo, li), ref_shape=(num_experts, d_in, d_out), logical_axes=tuple(axes),
                     kind="expert_linear", init="fan_in_trunc", ep_dim=0 if self.ep_size > 1 else None,
                     tp_dim=(1 if tp == "col" else 2) if (tp and self.tp_size > 1) else None)


class FusedParam:
  """Several parameters that sit back to back in the flat unit buffer, seen as one [sum(out), in] matrix."""

  def __init__(self, parts: list[Param]):
    self.parts = parts
    self.rows = [p.shape[0] for p in parts]

  @staticmethod
  def possible(parts: list[Param]) -> bool:
    cols = parts[0].shape[-1]
    if any(p.lora is not None for p in parts) or len({p.pdef.frozen for p in parts}) > 1:
      return False                           # adapters are per projection; a run is trained or frozen as a whole
    return all(len(p.shape) == 2 and p.shape[1] == cols and p.pdef.numel % ALIGN == 0 for p in parts)

  @property
  def frozen(self):
    return self.parts[0].pdef.frozen

  def _span(self, attr):
    first = getattr(self.parts[0], attr)
    if first is None:
      return None
    total = sum(self.rows)
    cols = self.parts[0].shape[1]
    # verify adjacency (cheap pointer arithmetic)
    ptr, esz = first.data_ptr(), first.element_size()
    for p, r in zip(self.parts, self.rows):
      t = getattr(p, attr)
      if t is None or t.data_ptr() != ptr:
        return None
      ptr += r * cols * esz
    return torch.as_strided(first, (total, cols), (cols, 1))

  @property
  def data(self):
    return self._span("data")

  def fusable(self) -> bool:
    """Do the parts sit back to back in their unit? Answered from the static layout, so that asking does not read `.data`
    (reading it would trigger the stand-alone all-gather of a unit whose gather is meant to ride inside this GEMM)."""
    f = getattr(self, "_fusable", None)
    if f is None:
      u = self.parts[0].unit
      if u is None:
        return self.data is not None
      if any(p.unit is not u for p in self.parts):
        f = False
      else:
        offs = [u.offsets[u.params.index(p)] for p in self.parts]
        f = all(offs[i + 1] == offs[i] + self.parts[i].pdef.numel for i in range(len(offs) - 1))
      self._fusable = f
    return f

  def pending_unit(self):
    return self.parts[0].pending_unit()

  @property
  def main_grad(self):
    return self._span("main_grad")

  @property
  def grad_written(self):
    return all(p.grad_written for p in self.parts)

  @grad_written.setter
  def grad_written(self, v):
    for p in self.parts:
      p.grad_written = v

  @property
  def shape(self):
    return (sum(self.rows), self.parts[0].shape[1])


# ------------------------------------------------------------------------------------------ tensor-parallel glue
class _CopyToTP(torch.autograd.Function):
  """Identity forward, all-reduce backward (input of a column-parallel linear)."""
  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return x

  @staticmethod
  def backward(ctx, dy):
    dy = dy.contiguous()
    dist.all_reduce(dy, group=ctx.group)
    return dy, None


class _ReduceFromTP(torch.autograd.Function):
  """All-reduce forward, identity backward (output of a row-parallel linear)."""
  @staticmethod
  def forward(ctx, x, group):
    x = x.contiguous()
    dist.all_reduce(x, group=group)
    return x

  @staticmethod
  def backward(ctx, dy):
    return dy, None


def sp_enabled(config) -> bool:
  """True when the mesh has a `tensor_sequence` axis: tensor parallelism with a sequence-split residual stream."""
  return int(getattr(config, "ici_tensor_sequence_parallelism", 1)) * int(getattr(config, "dcn_tensor_sequence_parallelism", 1)) > 1


def tp_enter(x, ctx):
  if ctx.tp_size > 1 and ctx.sp:
    from ..parallel import sequence_parallel as sp
    return sp.gather(x, ctx.tp_group)
  return _CopyToTP.apply(x, ctx.tp_group) if ctx.tp_size > 1 and torch.is_grad_enabled() else x


def tp_exit(x, ctx):
  if ctx.tp_size <= 1:
    return x
  if ctx.sp and x.dim() == 3:
    from ..parallel import sequence_parallel as sp
    return sp.reduce_scatter(x, ctx.tp_group)
  if torch.is_grad_enabled():
    return _ReduceFromTP.apply(x, ctx.tp_group)
  x = x.contiguous()
  dist.all_reduce(x, group=ctx.tp_group)
  return x


# ------------------------------------------------------------------------------------------ norms
class Norm:
  def __init__(self, b: Builder, name: str, dim: int, eps: float, offset: float = 0.0, with_scale: bool = True,
               kind: str = "rms", axes=("norm",)):
    self.eps, self.offset, self.kind = eps, offset, kind
    nb = b.sub(name)
    # a scale applied as (offset + scale) starts at zero, so that the effective factor starts at one
    self.scale = nb.vector("scale", dim, axes, init="zeros" if offset else "ones") if with_scale else None
    self.bias = nb.vector("bias", dim, axes, init="zeros") if kind == "layernorm" else None

  def __call__(self, x):
    if self.kind == "layernorm":
      return ref.layernorm(x, self.scale.leaf(), self.bias.leaf(), self.eps)
    if self.scale is None:
      xf = x.float()
      return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype)
    return F.rmsnorm(x, self.scale, self.eps, self.offset)


# ------------------------------------------------------------------------------------------ attention (MHA / GQA / MQA)
class Attention:
  """Multi/grouped-query attention with RoPE; the 1/sqrt(head_dim) factor lives in the query weights
  (src/maxtext/layers/attentions.py:663-677) unless QK-norm or an explicit query scalar is used."""

  def __init__(self, b: Builder, config, name="self_attention", window: int = 0, rope_inv_ts=None, interleaved=False,
               use_rope=True, qk_norm=False, query_scalar: float | None = None, soft_cap: float = 0.0, bias=False,
               rotary_dim=None, sinks=False, l2_qk_norm=False, temperature_tuning=False, chunk=0, out_bias=None, global_qk_norm=False, gated=False, qk_norm_offset=0.0,
               head_dim: int | None = None, num_kv_heads: int | None = None, share_kv: bool = False, v_norm: str = ""):
    c = config
    self.config = c
    # gemma4 global layers have their own head width and key/value head count (src/maxtext/models/gemma4.py:186-196)
    self.hq, self.hkv, self.dh, self.d = c.num_query_heads, int(num_kv_heads or c.num_kv_heads), int(head_dim or c.head_dim), c.emb_dim
    self.share_kv, self.v_norm = bool(share_kv), str(v_norm or "")
    tp = b.tp_size
    self.hq_l = self.hq // tp
    self.hkv_l = max(1, self.hkv // tp) if self.hkv >= tp else self.hkv
    self.window, self.inv_ts, self.interleaved, self.use_rope = window, rope_inv_ts, interleaved, use_rope
    self.qk_norm, self.query_scalar, self.soft_cap, self.rotary_dim = qk_norm, query_scalar, soft_cap, rotary_dim
    self.l2_qk_norm, self.temperature_tuning, self.chunk = l2_qk_norm, temperature_tuning, int(chunk)
    # YaRN "attention scaling" (src/maxtext/layers/embeddings.py:1020-1022): rotated q and k are each multiplied by
    # 0.1 ln(factor) + 1; here the product of the two factors scales the logits
    self.logit_scale = 1.0
    if use_rope and getattr(c, "rope_attention_scaling", False) and str(c.rope_type).lower() == "yarn" and c.rope_factor > 1:
      self.logit_scale = (0.1 * math.log(float(c.rope_factor)) + 1.0) ** 2
    # qwen3-next (src/maxtext/layers/attentions.py:685-686,1266-1270,1360-1362): the query projection is twice as wide,
    # per head [query | gate], and sigmoid(gate) multiplies the attention output before the output projection
    self.gated = bool(gated)
    ab = b.sub(*name.split("/"))
    depth_scale = 1.0 if (qk_norm or (query_scalar is not None and query_scalar != 1.0)) else 1.0 / math.sqrt(self.dh)
    kv_tp = "col" if self.hkv >= tp else None
    self.q = ab.sub("query").linear("kernel", (self.d,), (self.hq, self.dh * (2 if self.gated else 1)), ("embed", "q_heads", "kv"),
                                    "fan_in_normal", depth_scale, tp="col")
    self.k = ab.sub("key").linear("kernel", (self.d,), (self.hkv, self.dh), ("embed", "kv_heads", "kv_head_dim"),
                                  "fan_in_normal", tp=kv_tp)
    # share_kv_projections (src/maxtext/layers/attentions.py:289): the value is the (un-normalised, un-rotated) key projection
    self.v = None if self.share_kv else ab.sub("value").linear("kernel", (self.d,), (self.hkv, self.dh), ("embed", "kv_heads", "kv_head_dim"),
                                                               "fan_in_normal", tp=kv_tp)
    self.o = ab.sub("out").linear("kernel", (self.hq, self.dh), (self.d,), ("heads", "kv", "embed"), "fan_in_normal",
                                  tp="row")
    self.qkv = FusedParam([self.q, self.k, self.v]) if (not self.gated and not self.share_kv and FusedParam.possible([self.q, self.k, self.v])) else None
    self.vn = Norm(ab, "value_norm", self.dh, c.normalization_layer_epsilon, with_scale=(self.v_norm == "scale"), axes=("norm",)) if self.v_norm else None
    self.bq = self.bk = self.bv = None
    if bias:
      self.bq = ab.sub("query").vector("bias", self.hq * self.dh, ("q_heads",), init="zeros", tp=True)
      self.bk = ab.sub("key").vector("bias", self.hkv * self.dh, ("kv_heads",), init="zeros", tp=kv_tp is not None)
      self.bv = ab.sub("value").vector("bias", self.hkv * self.dh, ("kv_heads",), init="zeros", tp=kv_tp is not None)
    # the output projection carries a bias whenever q/k/v do, except for qwen2 (src/maxtext/layers/attentions.py:833)
    self.bo = ab.sub("out").vector("bias", self.d, ("embed",), init="zeros") if (bias if out_bias is None else out_bias) else None
    if self.bo is not None and tp > 1 and sp_enabled(c):
      self.bo.pdef.tp_partial = True           # added after the reduce-scatter: each rank sees its own tokens
    self.qn = self.kn = None
    self.global_qk_norm = bool(global_qk_norm) and qk_norm
    if self.global_qk_norm:
      # olmo3 (src/maxtext/layers/attentions.py:486-494): one RMS statistic over all heads of a token, scale per lane
      assert tp == 1, "the all-head q/k normalisation of olmo3 is not implemented under tensor parallelism"
      self.qn = Norm(ab, "query_norm", self.hq * self.dh, c.normalization_layer_epsilon, axes=("norm",))
      self.kn = Norm(ab, "key_norm", self.hkv * self.dh, c.normalization_layer_epsilon, axes=("norm",))
    elif qk_norm:
      ws = bool(getattr(c, "qk_norm_with_scale", True))         # false: plain RMS normalisation without a learned scale
      self.qn = Norm(ab, "query_norm", self.dh, c.normalization_layer_epsilon, qk_norm_offset, with_scale=ws, axes=("norm",))
      self.kn = Norm(ab, "key_norm", self.dh, c.normalization_layer_epsilon, qk_norm_offset, with_scale=ws, axes=("norm",))
    if tp > 1 and not self.global_qk_norm:
      for n_ in (self.qn, self.kn):
        if n_ is not None and n_.scale is not None:
          n_.scale.pdef.tp_partial = True        # every rank normalises its own heads with the shared per-lane scale
    self.sinks = ab.vector("sinks", self.hq, ("q_heads",), init="zeros", tp=True) if sinks else None

  def _project(self, x, ctx, tp_rt=None):
    B, S, _ = x.shape
    hq, hkv, dh = self.hq_l, self.hkv_l, self.dh
    fused = self.qkv is not None and self.bq is None and self.qkv.fusable()
    if fused:
      saved = ctx.reuse("qkv_proj")
      qkv = F.linear(x, self.qkv, saved_out=saved, tp_reduce_dx=tp_rt)
      if ctx.wants("qkv_proj"):
        ctx.keep("qkv_proj", qkv.clone())      # the rotary embedding below rewrites qkv in place
      return qkv.view(B, S, hq + 2 * hkv, dh), None
    q = ctx.keep("query_proj", F.linear(x, self.q, ctx.reuse("query_proj"), self.bq))
    k = ctx.keep("key_proj", F.linear(x, self.k, ctx.reuse("key_proj"), self.bk))
    v = k if self.share_kv else ctx.keep("value_proj", F.linear(x, self.v, ctx.reuse("value_proj"), self.bv))
    return None, (q.view(B, S, hq, -1), k.view(B, S, hkv, dh), v.view(B, S, hkv, dh))

  def __call__(self, x, ctx):
    B, S, _ = x.shape
    # tensor parallelism: with the fused runtime the two all-reduces of this block run inside GEMM epilogues
    tp_rt = tp_fused.runtime_for(ctx, x, self.d) if ctx.tp_size > 1 else None
    fuse_in = tp_rt is not None and self.qkv is not None and self.bq is None and self.qkv.fusable()
    if not fuse_in:
      x = tp_enter(x, ctx)
      B, S, _ = x.shape                      # sequence parallelism: the gathered length
    packed, sep = self._project(x, ctx, tp_rt if fuse_in else None)
    moba = bool(getattr(self.config, "moba", False)) and ctx.cache is None and ctx.cp_size == 1
    plain = (ctx.positions3 is None and not self.qk_norm and self.vn is None and not self.share_kv and self.sinks is None and self.rotary_dim is None and not self.gated and ctx.bidir is None and not moba and ctx.cache is None and ctx.cp_size == 1
             and not self.l2_qk_norm and not self.temperature_tuning and not (self.chunk and S > self.chunk))
    saved_ctx = ctx.reuse("context")
    if saved_ctx is not None and packed is not None and plain:
      # attention output kept by the remat policy: only the backward of the packed op is needed
      out = F.packed_attention(packed, ctx.positions, ctx.segment_ids, self.inv_ts, self.hq_l, self.hkv_l, self.interleaved,
                               self.logit_scale * (self.query_scalar or 1.0), self.soft_cap, self.window, self.use_rope)
    elif packed is not None and plain:
      out = F.packed_attention(packed, ctx.positions, ctx.segment_ids, self.inv_ts, self.hq_l, self.hkv_l, self.interleaved,
                               self.logit_scale * (self.query_scalar or 1.0), self.soft_cap, self.window, self.use_rope)
    else:
      if sep is None:
        q, k, v = packed[:, :, :self.hq_l], packed[:, :, self.hq_l:self.hq_l + self.hkv_l], packed[:, :, self.hq_l + self.hkv_l:]
      else:
        q, k, v = sep
      gate = None
      if self.gated:
        q, gate = q[..., :self.dh], q[..., self.dh:].reshape(B, S, -1)
      if self.global_qk_norm:
        q = self.qn(q.reshape(B, S, -1)).view(B, S, self.hq_l, self.dh)
        k = self.kn(k.reshape(B, S, -1)).view(B, S, self.hkv_l, self.dh)
      elif self.qk_norm:
        q, k = self.qn(q), self.kn(k)
      if self.vn is not None:
        v = self.vn(v)
      if self.use_rope and ctx.positions3 is not None and bool(getattr(self.config, "use_mrope", False)):
        # multi-axis rotary embedding: image tokens carry (t, h, w) positions (src/maxtext/layers/embeddings.py:1791-1948)
        sec = list(self.config.mrope_section)
        q = ref.apply_mrope(q, ctx.positions3, self.inv_ts, sec, self.rotary_dim)
        k = ref.apply_mrope(k, ctx.positions3, self.inv_ts, sec, self.rotary_dim)
      elif self.use_rope:
        q = F.rope(q, ctx.positions, self.inv_ts, self.interleaved, self.rotary_dim)
        k = F.rope(k, ctx.positions, self.inv_ts, self.interleaved, self.rotary_dim)
      if self.l2_qk_norm:
        # llama4 (src/maxtext/layers/attentions.py:1292-1296): x * rsqrt(mean(x^2) + eps), no learned scale, after RoPE
        eps = self.config.normalization_layer_epsilon
        q = (q.float() * torch.rsqrt(q.float().pow(2).mean(-1, keepdim=True) + eps)).to(q.dtype)
        k = (k.float() * torch.rsqrt(k.float().pow(2).mean(-1, keepdim=True) + eps)).to(k.dtype)
      if (self.query_scalar and self.query_scalar != 1.0) or self.logit_scale != 1.0:
        q = q * ((self.query_scalar or 1.0) * self.logit_scale)
      if self.temperature_tuning and not self.use_rope:
        # llama4 NoPE layers (attentions.py:1302-1308): log(floor((pos + 1) / floor_scale) + 1) * scale + 1
        c_ = self.config
        sc = torch.log(torch.floor((ctx.positions.float() + 1.0) / float(getattr(c_, "temperature_tuning_floor_scale", 8192.0))) + 1.0) \
            * float(getattr(c_, "temperature_tuning_scale", 0.1)) + 1.0
        q = (q.float() * sc[:, :, None, None]).to(q.dtype)
      if moba:
        # mixture-of-block attention: each query attends its own block and the best `moba_topk` earlier key blocks
        seg = None
        if ctx.segment_ids is not None:
          seg = (ctx.segment_ids[:, None, :, None] == ctx.segment_ids[:, None, None, :]) & (ctx.segment_ids[:, None, None, :] != 0)
        out = ref.moba_attention(q, k, v, ctx.positions, int(self.config.moba_chunk_size), int(self.config.moba_topk), 1.0, seg)
      elif ctx.cache is None and ctx.bidir is not None and ctx.cp_size == 1:
        # multimodal prompt: causal (and windowed) as usual, plus both directions inside each image's block of soft tokens
        m = ref.attention_mask(ctx.positions, ctx.positions, ctx.segment_ids, ctx.segment_ids, True, self.window) | ctx.bidir
        out = ref.attention(q, k, v, m, 1.0, self.soft_cap).to(q.dtype)
      elif ctx.cache is None and self.chunk and S > self.chunk and ctx.cp_size == 1:
        out = F.attention(q, k, v, ctx.positions, ctx.segment_ids, 1.0, self.soft_cap, self.window, chunk=self.chunk,
                          sinks=self.sinks.leaf() if self.sinks is not None else None)
      elif ctx.cache is not None:
        out = ctx.cache.attend(q, k, v, ctx, window=self.window, soft_cap=self.soft_cap, sinks=self.sinks)
      elif ctx.cp_size > 1:
        from ..parallel.context_parallel import context_attention
        out = context_attention(q, k, v, ctx.positions, ctx.segment_ids, ctx, 1.0, self.soft_cap, self.window)
      elif self.sinks is not None:
        out = F.attention(q, k, v, ctx.positions, ctx.segment_ids, 1.0, self.soft_cap, self.window, sinks=self.sinks.leaf())
      else:
        out = F.attention(q, k, v, ctx.positions, ctx.segment_ids, 1.0, self.soft_cap, self.window)
    ctx.keep("context", out)
    if self.gated:
      out = (out.reshape(B, S, -1).float() * torch.sigmoid(gate.float())).to(out.dtype)
    if tp_rt is not None and ctx.reuse("out_proj") is None and self.bo is None and self.o.lora is None:
      y = F.linear(out.reshape(B, S, -1), self.o, tp_reduce=tp_rt)
    else:
      y = F.linear(out.reshape(B, S, -1), self.o, ctx.reuse("out_proj"), self.bo if ctx.tp_size == 1 else None)
      if ctx.reuse("out_proj") is None:
        y = tp_exit(y, ctx)
        if self.bo is not None and ctx.tp_size > 1:
          y = y + self.bo.leaf().to(y.dtype)       # row-parallel: the bias is added once, after the reduction
      elif self.bo is not None and ctx.tp_size > 1:
        bl = self.bo.leaf().to(y.dtype)
        y = y + (bl - bl.detach())                 # the saved output already holds the bias; keep its gradient path
    ctx.keep("out_proj", y)
    return y


# ------------------------------------------------------------------------------------------ MLA
class MLA:
  """DeepSeek multi-head latent attention (src/maxtext/layers/attention_mla.py:785-1115).

  q = query(x) (or wq_b(q_norm(wq_a(x)))), split [nope | rope]; wkv_a(x) -> [kv_lora | k_rope];
  kv_norm on the latent; wkv_b -> per head [k_nope | v]; the single RoPE'd k_rope head is broadcast to
  all heads. Softmax scale (incl. YaRN mscale) multiplies the query at runtime."""

  def __init__(self, b: Builder, config, rope_inv_ts, interleaved, name="self_attention"):
    c = config
    self.c = c
    self.h = c.num_query_heads // b.tp_size
    self.nope, self.rope_d, self.vd = c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim
    self.qk = self.nope + self.rope_d
    self.inv_ts, self.interleaved = rope_inv_ts, interleaved
    ab = b.sub(name)
    d = c.emb_dim
    if c.q_lora_rank > 0:
      self.wq_a = ab.sub("wq_a").linear("kernel", (d,), (c.q_lora_rank,), ("embed", "q_lora"))
      self.q_norm = Norm(ab, "q_norm", c.q_lora_rank, c.normalization_layer_epsilon)
      self.wq_b = ab.sub("wq_b").linear("kernel", (c.q_lora_rank,), (c.num_query_heads, self.qk),
                                        ("q_lora", "q_heads", "kv"), tp="col")
      self.query = None
    else:
      self.query = ab.sub("query").linear("kernel", (d,), (c.num_query_heads, self.qk), ("embed", "q_heads", "kv"), tp="col")
    self.wkv_a = ab.sub("wkv_a").linear("kernel", (d,), (c.kv_lora_rank + self.rope_d,), ("embed", "kv_lora"))
    self.kv_norm = Norm(ab, "kv_norm", c.kv_lora_rank, c.normalization_layer_epsilon)
    self.wkv_b = ab.sub("wkv_b").linear("kernel", (c.kv_lora_rank,), (c.num_query_heads, self.nope + self.vd),
                                        ("kv_lora", "kv_heads", "kv_head_dim"), tp="col")
    self.o = ab.sub("out").linear("kernel", (c.num_query_heads, self.vd), (d,), ("heads", "kv", "embed"), tp="row")
    self.indexer = None
    if bool(getattr(c, "use_indexer", False)):
      # src/maxtext/layers/attention_mla.py:735-750: DeepSeek-V3.2 sparse attention; shares the rotary table, not the layout
      from .indexer import Indexer
      assert b.tp_size == 1, "use_indexer is not split over the tensor axis"
      self.indexer = Indexer(ab, c, rope_inv_ts)
    scale = self.qk ** -0.5
    if c.max_position_embeddings > c.original_max_position_embeddings and c.rope_type == "yarn":
      m = 0.1 * c.mscale * math.log(c.rope_factor) + 1.0
      scale = scale * m * m
    self.softmax_scale = scale

  def __call__(self, x, ctx):
    c = self.c
    x = tp_enter(x, ctx)
    B, S, _ = x.shape
    low_rank_q = None
    if self.query is not None:
      q = F.linear(x, self.query)
    else:
      low_rank_q = self.q_norm(F.linear(x, self.wq_a))
      q = F.linear(low_rank_q, self.wq_b)
    q = q.view(B, S, self.h, self.qk)
    q_nope, q_rope = q[..., :self.nope], q[..., self.nope:]
    q_rope = F.rope(q_rope, ctx.positions, self.inv_ts, self.interleaved)
    q = torch.cat([q_nope, q_rope], dim=-1) * self.softmax_scale
    kva = F.linear(x, self.wkv_a)
    latent, k_rope = kva[..., :c.kv_lora_rank], kva[..., c.kv_lora_rank:]
    k_rope = F.rope(k_rope.reshape(B, S, 1, self.rope_d), ctx.positions, self.inv_ts, self.interleaved)
    latent = self.kv_norm(latent.contiguous())
    if ctx.cache is not None:
      out = ctx.cache.attend_mla(q, latent, k_rope, self, ctx)
    else:
      kv = F.linear(latent, self.wkv_b).view(B, S, self.h, self.nope + self.vd)
      k = torch.cat([kv[..., :self.nope], k_rope.expand(B, S, self.h, self.rope_d)], dim=-1)
      v = kv[..., self.nope:]
      if c.use_qk_clip and ctx.mode == "train" and not ctx.recompute and ctx.max_logits is not None:
        ctx.max_logits[(ctx.layer_index, self)] = _max_logit_per_head(q, k, ctx.positions, ctx.segment_ids)
      sparse = None
      if self.indexer is not None:
        sparse, score, allowed = self.indexer(x, low_rank_q, ctx.positions, ctx.segment_ids)
        if sparse is not None and ctx.mode == "train" and float(c.indexer_loss_scaling_factor) > 0:
          ctx.aux_losses.append(("indexer_loss", self.indexer.loss(score, q, k, allowed, sparse)))
      if sparse is not None:
        # a per-query key set is not a mask form of the flash kernels: this path is the fp32 definition with an explicit mask
        out = ref.attention(q, k, v, sparse, 1.0)
      else:
        out = F.attention(q, k.contiguous(), v.contiguous(), ctx.positions, ctx.segment_ids, 1.0, 0.0, 0)
    y = F.linear(out.reshape(B, S, -1), self.o)
    return tp_exit(y, ctx)


@torch.no_grad()
def _max_logit_per_head(q, k, positions, segment_ids, chunk: int = 512) -> torch.Tensor:
  """Largest causal attention logit of every head over the batch ([H] fp32): what QK-clip compares with its threshold
  (src/maxtext/layers/attention_mla.py:1330-1341 `record_max_logits`)."""
  B, S, H, _ = q.shape
  best = torch.full((H,), -1e30, dtype=torch.float32, device=q.device)
  kf = k.float()
  for s0 in range(0, S, chunk):
    e = min(S, s0 + chunk)
    logits = torch.einsum("bqhd,bkhd->bhqk", q[:, s0:e].float(), kf[:, :e])
    m = ref.attention_mask(positions[:, s0:e], positions[:, :e], segment_ids[:, s0:e] if segment_ids is not None else None,
                           segment_ids[:, :e] if segment_ids is not None else None, True, 0)
    best = torch.maximum(best, logits.masked_fill(~m, -1e30).amax(dim=(0, 2, 3)))
  return best


# ------------------------------------------------------------------------------------------ dense MLP
class MLP:
  """wo( act(wi_0 x) * (wi_1 x) ) (src/maxtext/layers/linears.py:422-625)."""

  def __init__(self, b: Builder, config, name="mlp", hidden: int | None = None, acts=None, bias=False):
    c = config
    self.acts = list(acts or c.mlp_activations)
    f = hidden or c.mlp_dim
    mb = b.sub(name)
    d = c.emb_dim
    self.gated = len(self.acts) == 2
    self.wi_0 = mb.sub("wi_0" if self.gated else "wi").linear("kernel", (d,), (f,), ("embed", "mlp"), tp="col")
    self.wi_1 = mb.sub("wi_1").linear("kernel", (d,), (f,), ("embed", "mlp"), tp="col") if self.gated else None
    self.wo = mb.sub("wo").linear("kernel", (f,), (d,), ("mlp", "embed"), tp="row")
    self.wi = FusedParam([self.wi_0, self.wi_1]) if self.gated and FusedParam.possible([self.wi_0, self.wi_1]) else None
    self.bi = mb.sub("wi_0" if self.gated else "wi").vector("bias", f, ("mlp",), init="zeros", tp=True) if bias else None
    self.bo = mb.sub("wo").vector("bias", d, ("embed",), init="zeros") if bias else None
    if self.bo is not None and b.tp_size > 1 and sp_enabled(c):
      self.bo.pdef.tp_partial = True

  def __call__(self, x, ctx):
    tp_rt = tp_fused.runtime_for(ctx, x, x.shape[-1]) if ctx.tp_size > 1 else None
    fuse_in = tp_rt is not None and self.gated and self.wi is not None and self.wi.fusable()
    if not fuse_in:
      x = tp_enter(x, ctx)
    if self.gated:
      if self.wi is not None and self.wi.fusable():
        gu = ctx.keep("mlpwi", F.linear(x, self.wi, ctx.reuse("mlpwi"), tp_reduce_dx=tp_rt if fuse_in else None))
      else:
        g = ctx.keep("mlpwi_0", F.linear(x, self.wi_0, ctx.reuse("mlpwi_0")))
        u = ctx.keep("mlpwi_1", F.linear(x, self.wi_1, ctx.reuse("mlpwi_1")))
        gu = torch.cat([g, u], dim=-1)
      h = F.gated_act(gu, self.acts[0])
    else:
      h = F.linear(x, self.wi_0, bias=self.bi)
      h = ref.act_fn(self.acts[0])(h.float()).to(x.dtype) if self.acts[0] != "linear" else h
    if tp_rt is not None and ctx.reuse("mlpwo") is None and self.bo is None and self.wo.lora is None:
      y = F.linear(h, self.wo, tp_reduce=tp_rt)
    else:
      y = F.linear(h, self.wo, ctx.reuse("mlpwo"), self.bo if ctx.tp_size == 1 else None)
      if ctx.reuse("mlpwo") is None:
        y = tp_exit(y, ctx)
        if self.bo is not None and ctx.tp_size > 1:
          y = y + self.bo.leaf().to(y.dtype)       # row-parallel: the bias is added once, after the reduction
      elif self.bo is not None and ctx.tp_size > 1:
        bl = self.bo.leaf().to(y.dtype)
        y = y + (bl - bl.detach())                 # the saved output already holds the bias; keep its gradient path
    ctx.keep("mlpwo", y)
    return y
