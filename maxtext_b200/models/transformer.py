"""Decoder-only transformer assembled from a per-family layer plan.

The role of src/maxtext/models/models.py:330-619 (`Transformer`) and
src/maxtext/layers/nnx_decoders.py:380-2025 (`NNXDecoder`): token embedding, a stack of decoder
layers chosen by `decoder_block`, final norm and output head. Instead of one traced function the
model is a list of *units* (embedding, each layer, head) that the training engine runs with an
explicit schedule (gather -> forward -> [recompute ->] backward -> reduce-scatter).

Family specifics (block structure, parameter names, norms, RoPE flavour, MoE style) are described by
`LayerPlan` entries built in `models/families.py`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from ..layers import blocks as L
from ..layers import moe as M
from ..layers.context import LayerCtx
from ..ops import functional as F
from ..ops import reference as ref
from ..parallel.param_store import ParamStore


@dataclass
class BlockPlan:
  """One attention + feed-forward residual pair."""
  suffix: str = ""                       # appended to every module name (gemma2: _local / _global)
  pre_attn_norm: str = "pre_self_attention_layer_norm"
  post_attn_norm: str | None = None      # norm applied to the attention output before the residual add
  pre_mlp_norm: str = "post_self_attention_layer_norm"
  post_mlp_norm: str | None = None
  attn_name: str = "self_attention"
  mlp_name: str = "mlp"
  attention: str = "gqa"                 # gqa | mla | gdn (gated delta network, qwen3-next)
  gated_attn: bool = False               # qwen3-next full attention: sigmoid output gate from a widened query projection
  window: int = 0
  rope: str = "default"                  # key into Transformer.rope_tables
  use_rope: bool = True
  qk_norm: bool = False
  attn_bias: bool = False
  query_scalar: float | None = None
  soft_cap: float = 0.0
  sinks: bool = False
  mlp: str = "dense"                     # dense | moe | moe_shared
  mlp_hidden: int | None = None
  mlp_bias: bool = False
  norm_kind: str = "rms"
  norm_offset: float = 0.0
  parallel_residual: bool = False
  prefix: str = ""                       # extra level in the parameter tree (olmo3: layers_0 .. layers_3 inside one cycle)
  attn_out_bias: bool | None = None      # None: same as attn_bias (qwen2 has q/k/v biases only)
  global_qk_norm: bool = False           # olmo3: q/k RMS statistic over all heads instead of per head
  l2_qk_norm: bool = False               # llama4: scale-free RMS normalisation of q and k after RoPE
  temperature_tuning: bool = False       # llama4 NoPE layers: position-dependent query scale
  chunk: int = 0                         # llama4 RoPE layers: attention restricted to chunks of this many tokens
  moe_style: str = ""                    # "" | "llama4" | "gpt_oss"
  head_dim: int | None = None            # gemma4 global layers: own head width ...
  kv_heads: int | None = None            # ... and key / value head count
  share_kv: bool = False                 # value = key projection
  v_norm: str = ""                       # "" | "noscale" | "scale": RMS normalisation of the value heads
  layer_scalar: bool = False             # learned scalar on the layer output
  compress_ratio: int = 0                # DeepSeek-V4 compressed attention: 0 (window only), 4 (sparse) or 128 (heavy)


@dataclass
class LayerPlan:
  stack: str = "layers"                  # name of the stacked collection in the checkpoint tree
  blocks: list = field(default_factory=lambda: [BlockPlan()])


class DecoderBlock:
  def __init__(self, b: L.Builder, config, plan: BlockPlan, rope_tables: dict, layer_index: int | None = None, hash_mapping=None):
    c, s = config, plan.suffix
    self.plan = plan
    self.engram = None
    if hash_mapping is not None and layer_index in hash_mapping.layer_ids:
      # src/maxtext/models/deepseek.py:105-137, 365-367: n-gram memory added to the layer input, before attention
      from ..layers.engram import Engram
      self.engram_norm = L.Norm(b, "engram_layer_norm", c.emb_dim, c.normalization_layer_epsilon)
      self.engram = Engram(b, c, hash_mapping.vocab_sizes(layer_index))
      self.engram_layer, self.hash_mapping = layer_index, hash_mapping
    if plan.prefix:
      b = b.sub(plan.prefix)
    eps = c.normalization_layer_epsilon
    mk = lambda n: L.Norm(b, n + s, c.emb_dim, eps, plan.norm_offset, kind=plan.norm_kind)  # noqa: E731
    self.n1 = mk(plan.pre_attn_norm) if plan.pre_attn_norm else None
    inv_ts, interleaved = rope_tables[plan.rope]
    rot = int(c.head_dim * c.partial_rotary_factor) if 0 < c.partial_rotary_factor < 1.0 else None
    if plan.attention == "mla":
      self.attn = L.MLA(b, c, inv_ts, interleaved, plan.attn_name + s)
    elif plan.attention == "gdn":
      from ..layers.gdn import GatedDeltaNet
      self.attn = GatedDeltaNet(b, c, plan.attn_name + s)
    elif plan.attention == "compressed":
      from ..layers.attention_compressed import CompressedAttention
      self.attn = CompressedAttention(b, c, plan.attn_name + s, plan.compress_ratio, int(c.sliding_window_size))
    else:
      self.attn = L.Attention(b, c, plan.attn_name + s, plan.window, inv_ts, interleaved, plan.use_rope, plan.qk_norm,
                              plan.query_scalar, plan.soft_cap, plan.attn_bias,
                              rotary_dim=rot, sinks=plan.sinks, l2_qk_norm=plan.l2_qk_norm,
                              temperature_tuning=plan.temperature_tuning, chunk=plan.chunk, out_bias=plan.attn_out_bias,
                              global_qk_norm=plan.global_qk_norm, gated=plan.gated_attn, qk_norm_offset=plan.norm_offset,
                              head_dim=plan.head_dim, num_kv_heads=plan.kv_heads, share_kv=plan.share_kv, v_norm=plan.v_norm)
    self.n1b = mk(plan.post_attn_norm) if plan.post_attn_norm else None
    self.n2 = mk(plan.pre_mlp_norm) if plan.pre_mlp_norm else None
    if plan.mlp == "moe":
      self.mlp = M.RoutedMoE(b, c, plan.mlp_name + s, style=plan.moe_style)
    elif plan.mlp == "moe_shared":
      hashed = layer_index is not None and layer_index < int(getattr(c, "first_num_hash_layers", 0) or 0) and plan.moe_style == ""
      self.mlp = M.RoutedAndSharedMoE(b, c, plan.mlp_name + s, style=plan.moe_style, hash_routing=hashed)
    elif plan.mlp == "gemma4_moe":
      self.mlp = M.Gemma4MoE(b, c, plan.mlp_name + s)
    else:
      self.mlp = L.MLP(b, c, plan.mlp_name + s, plan.mlp_hidden, bias=plan.mlp_bias)
    self.n2b = mk(plan.post_mlp_norm) if plan.post_mlp_norm else None
    self.layer_scalar = b._add("layer_scalar" + s, shape=(1,), ref_shape=(1,), logical_axes=(None,), kind="same", init="ones") \
        if plan.layer_scalar else None
    self.mhc_attn = self.mhc_mlp = None
    if int(getattr(c, "mhc_expansion_rate", 1)) > 1:
      # src/maxtext/models/deepseek.py:177-179: each branch of the block is wrapped by its own hyper-connection
      from ..layers.mhc import HyperConnection
      self.mhc_attn = HyperConnection(b, c, "mhc_attention", c.emb_dim)
      self.mhc_mlp = HyperConnection(b, c, "mhc_mlp", c.emb_dim)
    if b.tp_size > 1 and L.sp_enabled(c):
      # sequence-parallel residual stream: these norms see this rank's tokens only, their scale gradients are partial sums
      for n_ in (self.n1, self.n1b, self.n2, self.n2b):
        for v_ in ((n_.scale, n_.bias) if n_ is not None else ()):
          if v_ is not None:
            v_.pdef.tp_partial = True

  def __call__(self, x, ctx: LayerCtx):
    if self.engram is not None and ctx.tokens is not None:
      ids = self.hash_mapping.hashes(self.hash_mapping.ct(ctx.tokens), self.engram_layer)
      x = x + self.engram(self.engram_norm(x), ids)
    if self.mhc_attn is not None:               # x [B, S, k, D]: the residual adds live inside the hyper-connections
      x = self.mhc_attn(self.n1, lambda h: self.attn(h, ctx), x)
      return self.mhc_mlp(self.n2, lambda h: self.mlp(h, ctx), x)
    a = self.attn(self.n1(x) if self.n1 is not None else x, ctx)
    if self.n1b is not None:
      a = self.n1b(a)
    x = x + ctx.dropout(a, 0)                 # src/maxtext/models/llama2.py: dropout on each residual branch
    h = self.n2(x) if self.n2 is not None else x
    m = self.mlp(h, ctx, original=x) if self.plan.mlp == "gemma4_moe" else self.mlp(h, ctx)
    if self.n2b is not None:
      m = self.n2b(m)
    x = x + ctx.dropout(m, 1)
    if self.layer_scalar is not None:
      x = x * self.layer_scalar.leaf().to(x.dtype)
    return x


class DecoderLayer:
  """One schedulable unit: all parameters gathered / reduced together."""

  def __init__(self, config, index: int, stack_index: int, plan: LayerPlan, rope_tables, par, hash_mapping=None):
    self.index, self.plan = index, plan
    self.unit = f"layer_{index}"
    b = L.Builder(config, self.unit, stack_index, plan.stack, **par)
    self.blocks = [DecoderBlock(b, config, bp, rope_tables, layer_index=index, hash_mapping=hash_mapping) for bp in plan.blocks]
    self.params = b.params

  def __call__(self, x, ctx: LayerCtx):
    n = int(ctx.batch_split)
    if n > 1 and ctx.cache is None and x.shape[0] % n == 0:
      return self._call_split(x, ctx, n)
    return self._call_one(x, ctx)

  def _call_split(self, x, ctx: LayerCtx, n: int):
    """Batch-split schedule (the role of src/maxtext/models/deepseek_batchsplit.py:1939-2015 and its staggered layer body):
    the batch runs through this layer as n micro-batches on alternating CUDA streams, so the expert-parallel exchange
    (and any other collective) of one micro-batch overlaps the attention and GEMMs of the other. The backward pass of every
    operation runs on the stream of its forward, so the overlap carries over. Results are the concatenation of the
    micro-batch results; auxiliary losses are averaged, per-head logit maxima are merged by maximum."""
    parts = x.chunk(n, 0)
    lanes = _split_lanes(x.device, min(n, 2)) if x.is_cuda else None
    main = torch.cuda.current_stream(x.device) if lanes else None
    outs, subs = [], []
    for j in range(n):
      sub = ctx.micro(j, n)
      subs.append(sub)
      if lanes:
        lane = lanes[j % len(lanes)]
        lane.wait_stream(main)
        with torch.cuda.stream(lane):
          outs.append(self._call_one(parts[j], sub))
      else:
        outs.append(self._call_one(parts[j], sub))
    if lanes:
      for lane in lanes:
        main.wait_stream(lane)
      for o in outs:
        o.record_stream(main)
    names = [nm for nm, _ in subs[0].aux_losses]
    for i, nm in enumerate(names):
      ctx.aux_losses.append((nm, sum(s_.aux_losses[i][1] for s_ in subs) / n))
    if ctx.max_logits is not None:
      for s_ in subs:
        for k_, v_ in s_.max_logits.items():
          ctx.max_logits[k_] = torch.maximum(ctx.max_logits[k_], v_) if k_ in ctx.max_logits and s_ is not subs[0] else v_
    return torch.cat(outs, 0)

  def _call_one(self, x, ctx: LayerCtx):
    caches = ctx.cache                      # inference: one cache per block of this layer
    for i, blk in enumerate(self.blocks):
      ctx.name_prefix = f"b{i}/" if len(self.blocks) > 1 else ""
      if caches is not None:
        ctx.cache = caches[i] if isinstance(caches, (list, tuple)) else caches
      x = blk(x, ctx)
    ctx.name_prefix = ""
    ctx.cache = caches
    ds = ctx.deepstack
    if ds is not None and self.index < len(ds[1]) and x.shape[1] == ds[0].shape[1]:
      # Qwen3-VL deepstack: intermediate vision features join the hidden states of the image positions after the first layers
      from ..multimodal.utils import merge_mm_embeddings
      x = x + merge_mm_embeddings(torch.zeros_like(x), ds[1][self.index], ds[0])
    return x


_LANES: dict = {}


def _split_lanes(device, n: int):
  """Side streams of the batch-split schedule, one set per device."""
  key = (device.index if device.index is not None else torch.cuda.current_device(), n)
  if key not in _LANES:
    _LANES[key] = [torch.cuda.Stream(device=device) for _ in range(n)]
  return _LANES[key]


class _CollapsingNorm:
  """Final norm of a model with hyper-connections: the k residual streams are summed before the norm, or, for DeepSeek-V4,
  mixed by the learned gates of its hyper-head (src/maxtext/layers/decoders.py:1279-1288)."""

  def __init__(self, norm, hyper_head=None):
    self.norm, self.hyper_head = norm, hyper_head
    self.scale, self.bias = norm.scale, norm.bias

  def __call__(self, x):
    if x.dim() == 4:
      from ..layers.mhc import reduce_streams
      x = self.hyper_head(x) if self.hyper_head is not None else reduce_streams(x)
    return self.norm(x)


class MTPLayer:
  """One multi-token-prediction module (src/maxtext/layers/multi_token_prediction.py:160-310): the previous hidden state and
  the embedding of the token one step further ahead are normalised separately, concatenated [embedding | hidden], projected
  back to the model width and passed through one decoder layer of the model's own kind."""

  def __init__(self, b: L.Builder, config, k: int, plan: LayerPlan, rope_tables, norm_offset, norm_kind):
    c = config
    mb = b.sub("mtp_block", f"mtp_layer_{k}")
    eps = c.normalization_layer_epsilon
    self.k = k
    self.embedding_norm = L.Norm(mb, f"mtp_{k}_embedding_norm", c.emb_dim, eps, norm_offset, kind=norm_kind)
    self.hidden_state_norm = L.Norm(mb, f"mtp_{k}_hidden_state_norm", c.emb_dim, eps, norm_offset, kind=norm_kind)
    self.projection = mb.sub(f"mtp_{k}_projection").linear("kernel", (2 * c.emb_dim,), (c.emb_dim,), ("concat_embed", "embed"))
    tb = mb.sub(f"mtp_{k}_transformer_layer")
    self.blocks = [DecoderBlock(tb, c, bp, rope_tables) for bp in plan.blocks]

  def __call__(self, prev_hidden, target_embedding, ctx: LayerCtx):
    feats = torch.cat([self.embedding_norm(target_embedding), self.hidden_state_norm(prev_hidden)], dim=-1)
    x = F.linear(feats, self.projection)
    for blk in self.blocks:
      x = blk(x, ctx)
    return x


def roll_left(x: torch.Tensor, segment_ids: torch.Tensor | None = None) -> torch.Tensor:
  """Shift one position to the left along the sequence; the last position, and positions whose right neighbour belongs to
  another document, become zero (multi_token_prediction.py:91-158)."""
  out = torch.zeros_like(x)
  out[:, :-1] = x[:, 1:]
  if segment_ids is not None:
    nxt = torch.zeros_like(segment_ids)
    nxt[:, :-1] = segment_ids[:, 1:]
    keep = (nxt == segment_ids) & (segment_ids != 0)
    out = out * keep.to(out.dtype) if out.dtype != torch.bool else out & keep
  return out


class Transformer:
  def __init__(self, config, mesh=None, device="cpu", build_store: bool = True, stage: tuple | None = None):
    """`stage` = (index, count) builds only what pipeline stage `index` owns: layer l belongs to stage
    (l // num_layers_per_pipeline_stage) % count (circular repeats wrap around), the embedding to stage 0, the
    final norm and output head to the last stage (src/maxtext/layers/pipeline.py)."""
    from . import families
    c = self.config = config
    self.mesh = mesh
    self.device = torch.device(device)
    tp_axes = ("tensor", "tensor_sequence")
    tp_size = mesh.axis_size(tp_axes) if mesh is not None else 1
    tp_rank = mesh.axis_index(tp_axes) if mesh is not None else 0
    ep_size = mesh.axis_size("expert") if (mesh is not None and c.num_experts > 1) else 1
    ep_rank = mesh.axis_index("expert") if (mesh is not None and c.num_experts > 1) else 0
    self.par = dict(tp_size=tp_size, tp_rank=tp_rank, ep_size=ep_size, ep_rank=ep_rank)
    self.rope_tables = families.rope_tables(c, self.device)
    self.family = families.describe(c)
    self.stage = stage
    self.has_embed = stage is None or stage[0] == 0
    self.has_head = stage is None or stage[0] == stage[1] - 1
    # ---- embedding unit
    eb = L.Builder(c, "embed", None, None, **self.par)
    self.embedding = eb.sub("token_embedder").table("embedding", (c.vocab_size, c.emb_dim), ("vocab", "embed_vocab"))
    self.pos_embedding = None
    if c.trainable_position_size > 0:
      self.pos_embedding = eb.sub("decoder", "position_embedder").table(
          "embedding", (c.trainable_position_size, c.emb_dim), (None, "embed"))
    self.embed_params = eb.params if self.has_embed else []
    # ---- layers
    self.mhc_k = int(getattr(c, "mhc_expansion_rate", 1) or 1)
    self.hash_mapping = None
    if list(getattr(c, "engram_layers", []) or []):
      from ..input_pipeline.tokenizer import build_tokenizer
      from ..layers.engram import NgramHashMapping
      tok = build_tokenizer(c)
      self.hash_mapping = NgramHashMapping(c.engram_vocab_bases, c.engram_max_ngram_size, c.engram_num_heads, c.engram_layers, tok,
                                           int(getattr(tok, "pad_id", 0) or 0), int(c.engram_seed))
    self.layers: list[DecoderLayer] = []
    counters: dict[str, int] = {}
    for i, plan in enumerate(families.layer_plans(c)):
      si = counters.get(plan.stack, 0)
      counters[plan.stack] = si + 1
      if stage is not None and (i // max(1, int(c.num_layers_per_pipeline_stage))) % stage[1] != stage[0]:
        continue
      self.layers.append(DecoderLayer(c, i, si, plan, self.rope_tables, self.par, hash_mapping=self.hash_mapping))
    self.stack_sizes = counters
    # ---- multi-token prediction unit (training only; the last stage owns it)
    self.mtp_layers: list[MTPLayer] = []
    self.mtp_params = []
    if int(c.mtp_num_layers) > 0 and self.has_head:
      mb = L.Builder(c, "mtp", None, None, **self.par)
      last_plan = families.layer_plans(c)[-1]
      self.mtp_layers = [MTPLayer(mb, c, k, last_plan, self.rope_tables, self.family.norm_offset, self.family.norm_kind)
                         for k in range(1, int(c.mtp_num_layers) + 1)]
      self.mtp_params = mb.params
    # ---- head unit
    hb = L.Builder(c, "head", None, None, **self.par)
    norm = L.Norm(hb.sub("decoder"), "decoder_norm", c.emb_dim, c.normalization_layer_epsilon,
                  self.family.norm_offset, kind=self.family.norm_kind)
    hyper_head = None
    if self.mhc_k > 1 and c.decoder_block == "deepseek4":
      from ..layers.mhc import HyperHead
      hyper_head = HyperHead(hb.sub("decoder"), c, "hc_head")
    self.final_norm = _CollapsingNorm(norm, hyper_head) if self.mhc_k > 1 else norm
    self.logits_dense = None
    if not c.logits_via_embedding:
      self.logits_dense = hb.sub("decoder", "logits_dense").linear("kernel", (c.emb_dim,), (c.vocab_size,),
                                                                   ("embed_vocab", "vocab"))
    self.head_params = hb.params if self.has_head else []
    # multimodal: the vision tower is a unit of its own; it is frozen unless freeze_vision_encoder_params is off
    self.vision, self.vision_params, self._deepstack = None, [], None
    if bool(getattr(c, "use_multimodal", False)) and self.has_embed:
      kind = getattr(c, "vision_encoder_block", "") or c.decoder_block
      qwen_vl = kind in ("qwen3", "qwen3_moe", "qwen3_5", "qwen3_next", "qwen3_vl", "qwen3_omni")
      if kind not in ("gemma3", "gemma4", "llama4") and not qwen_vl:
        raise NotImplementedError("use_multimodal is implemented for the Gemma-3, Gemma-4, Llama-4 and Qwen3-VL / Omni vision towers")
      from .vision import Gemma3Vision, Gemma4Vision, Llama4Vision, Qwen3VLVision
      self.vision = {"gemma3": Gemma3Vision, "gemma4": Gemma4Vision, "llama4": Llama4Vision}.get(kind, Qwen3VLVision)(c, self.par)
      self.vision_params = self.vision.params
      if bool(getattr(c, "freeze_vision_encoder_params", True)):
        for p in self.vision_params:
          p.pdef.frozen = True
    # Qwen3-Omni audio tower (frozen with the vision tower)
    self.audio, self.audio_params = None, []
    if bool(getattr(c, "use_multimodal", False)) and bool(getattr(c, "use_audio", False)) and self.has_embed:
      from .audio import Qwen3OmniAudio
      self.audio = Qwen3OmniAudio(c, self.par)
      self.audio_params = self.audio.params
      if bool(getattr(c, "freeze_vision_encoder_params", True)):
        for p in self.audio_params:
          p.pdef.frozen = True
    if L.lora_spec(c) is not None:
      # LoRA fine-tuning: everything but the adapters keeps its value (no gradient, no weight decay)
      for p in self.all_params():
        if not p.pdef.name.endswith(("_lora_a", "_lora_b")):
          p.pdef.frozen = True
    import re
    pats = [re.compile(x) for x in (getattr(c, "trainable_parameters_mask", None) or [])]
    if pats:
      # whitelist (src/maxtext/optimizers/optimizers.py:236-250): everything no pattern matches keeps its value
      for p in self.all_params():
        if not any(r.search(p.pdef.name) or r.search("/".join(p.pdef.ref_path)) for r in pats):
          p.pdef.frozen = True
    nodecay = [re.compile(x) for x in (getattr(c, "adamw_mask", None) or [])]
    for p in self.all_params() if nodecay else ():
      if any(r.search(p.pdef.name) or r.search("/".join(p.pdef.ref_path)) for r in nodecay):
        p.pdef.weight_decay = False             # src/maxtext/optimizers/optimizers.py:47-49: matched parameters are not decayed
    self.store: ParamStore | None = None
    if build_store:
      self.store = ParamStore(self.all_params(), mesh or _SingleMesh(), c, self.device)

  # ------------------------------------------------------------------ params
  def all_params(self):
    out = list(self.embed_params)
    for l in self.layers:
      out.extend(l.params)
    out.extend(self.mtp_params)
    out.extend(self.head_params)
    out.extend(self.vision_params)
    out.extend(self.audio_params)
    return out

  def units_in_order(self) -> list[str]:
    return (["embed"] if self.has_embed else []) + [l.unit for l in self.layers] + (["mtp"] if self.mtp_layers else []) + \
        (["head"] if self.has_head else [])

  # ------------------------------------------------------------------ contexts
  def make_ctx(self, positions, segment_ids, mode="train", tokens=None) -> LayerCtx:
    from ..layers.context import saved_names
    m = self.mesh
    dev, off = saved_names(self.config) if mode == "train" else ((), ())
    ctx = LayerCtx(self.config, positions, segment_ids, mode, m, save_names=dev, offload_names=off, tokens=tokens)
    if m is not None:
      ctx.tp_size = m.axis_size(("tensor", "tensor_sequence"))
      ctx.tp_group = m.group(("tensor", "tensor_sequence")) if ctx.tp_size > 1 else None
      if self.config.num_experts > 1:
        ctx.ep_size = m.axis_size("expert")
        ctx.ep_group = m.group("expert") if ctx.ep_size > 1 else None
      ctx.cp_size = m.axis_size(("context", "context_usp_ulysses"))
      ctx.cp_group = m.group("context") if m.axis_size("context") > 1 else None
      ctx.usp_group = m.group("context_usp_ulysses") if m.axis_size("context_usp_ulysses") > 1 else None
    return ctx

  # ------------------------------------------------------------------ pieces run by the engine
  def encode_images(self, images, image_mask):
    """images [B, N, 3, H, W] -> (soft tokens [B, N*K, D], mask [B, S]) as `embed(..., mm=...)` takes them."""
    soft = self.vision(images.to(self.embedding.data.device))
    mask = image_mask.to(soft.device).bool()
    deep = getattr(self.vision, "deepstack", None)
    self._deepstack = (mask, [d.reshape(d.shape[0], -1, d.shape[-1]) for d in deep]) if deep else None
    return soft.reshape(soft.shape[0], -1, soft.shape[-1]), mask

  def encode_audio(self, audio, audio_mask):
    """audio: [B, mel, frames] or a list of [mel, frames_i] clips (one per sequence) -> (soft tokens [B, K, D], mask [B, S]);
    shorter clips are padded with zero rows that no mask position reaches."""
    dev = self.embedding.data.device
    clips = [self.audio(a.to(dev)) for a in audio]
    K = max(x.shape[0] for x in clips)
    soft = torch.stack([torch.nn.functional.pad(x, (0, 0, 0, K - x.shape[0])) for x in clips])
    return soft, audio_mask.to(dev).bool()

  def embed(self, tokens, positions, mm=None):
    """mm: (soft tokens, mask) of one modality, or a list of such pairs (images, audio) merged one after the other."""
    c = self.config
    x = F.embedding(tokens, self.embedding)
    if mm is not None:
      from ..multimodal.utils import merge_mm_embeddings
      for soft, mask in ([mm] if isinstance(mm, tuple) else mm):
        x = merge_mm_embeddings(x, soft, mask)
    if self.family.scale_embedding:
      x = (x.float() * math.sqrt(c.emb_dim)).to(x.dtype)
    if bool(getattr(c, "use_untrainable_positional_embedding", False)):
      # fixed sinusoids [sin | cos] with geometric wavelengths up to 10 000 (src/maxtext/layers/embeddings.py:1055-1120)
      half = c.emb_dim // 2
      inv = torch.exp(torch.arange(half, device=x.device, dtype=torch.float32) * -(math.log(10000.0) / max(half - 1, 1)))
      ang = positions.float()[..., None] * inv
      x = x + torch.cat([torch.sin(ang), torch.cos(ang)], dim=-1).to(x.dtype)
    if self.pos_embedding is not None:
      x = x + self.pos_embedding.leaf()[positions.long()].to(x.dtype)
    if self.mhc_k > 1:
      from ..layers.mhc import expand_streams
      x = expand_streams(x, self.mhc_k)        # src/maxtext/layers/decoders.py:880-883
    return x

  def head_param(self):
    return self.logits_dense if self.logits_dense is not None else self.embedding

  def head_logit_scale(self) -> float:
    c = self.config
    if c.logits_via_embedding and c.normalize_embedding_logits:
      return 1.0 / math.sqrt(c.emb_dim)
    return 1.0

  def logits(self, x):
    h = self.final_norm(x)
    return F.head_logits(h, self.head_param(), self.config.final_logits_soft_cap, self.head_logit_scale())

  # ------------------------------------------------------------------ plain forward (eval / inference / tests)
  @torch.no_grad()
  def forward(self, tokens, positions=None, segment_ids=None, mode="train", caches=None, images=None, image_mask=None, positions3=None,
              audio=None, audio_mask=None):
    """Full logits [B,S,V] in fp32; every unit must be resident (single rank or gathered by the caller).
    `images` [B, N, 3, H, W] with `image_mask` [B, S] (True at the soft-token positions) makes the prompt multimodal;
    `audio` (mel spectrograms, one clip per sequence) with `audio_mask` [B, S] does the same for the audio tower."""
    B, S = tokens.shape
    if positions is None:
      positions = torch.arange(S, device=tokens.device)[None].expand(B, S)
    ctx = self.make_ctx(positions, segment_ids, mode, tokens)
    ctx.positions3 = positions3.to(tokens.device) if positions3 is not None else None
    if str(getattr(self.config, "attention_type", "global")) == "block_diffusion" and caches is None:
      from ..diffusion.block_diffusion import same_block_mask
      ctx.bidir = same_block_mask(positions, int(self.config.causal_block_size), segment_ids)
    mm = None
    if images is not None:
      from ..multimodal.utils import bidirectional_block_mask
      mm = self.encode_images(images, image_mask)
      ctx.deepstack = self._deepstack
      if self.vision.__class__.__name__ in ("Gemma3Vision", "Gemma4Vision"):      # Llama-4 keeps plain causal attention over image tokens
        ctx.bidir = bidirectional_block_mask(mm[1])
    if audio is not None:
      am = self.encode_audio(audio, audio_mask)
      mm = am if mm is None else [mm, am]
    x = self.embed(tokens, positions, mm)
    for i, layer in enumerate(self.layers):
      ctx.layer_index = i
      ctx.cache = caches[i] if caches is not None else None
      x = layer(x, ctx)
    return self.logits(x)


class _SingleMesh:
  """Stand-in mesh for single-process use."""
  axis_names = ("fsdp",)
  shape = {"fsdp": 1}
  rank, world = 0, 1

  def axis_size(self, axes):
    return 1

  def axis_index(self, axes):
    return 0

  def group(self, axes):
    return None
