"""Per-family layer plans: which blocks make a layer, how they are named, which RoPE they use.

One entry per `decoder_block` value (src/maxtext/common/common_types.py:92-118), reproducing the
structure of the reference model files: llama2.py (Llama 2/3/3.x), mistral.py, mixtral.py,
deepseek.py, gemma.py / gemma2.py / gemma3.py, qwen2.py / qwen3.py, gpt3.py, gpt_oss.py, olmo3.py,
simple_layer.py.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..ops import reference as ref
from .transformer import BlockPlan, LayerPlan


@dataclass
class Family:
  norm_kind: str = "rms"
  norm_offset: float = 0.0
  scale_embedding: bool = False


def describe(c) -> Family:
  blk = c.decoder_block
  # Gemma checkpoints store the embedding table already multiplied by sqrt(emb_dim) and divide the tied logits by the
  # same factor (normalize_embedding_logits), so nothing is scaled at lookup (src/maxtext/layers/decoders.py:823-825,
  # src/maxtext/checkpoint_conversion/utils/param_mapping.py:498-508)
  if blk == "gpt3":
    return Family(norm_kind="layernorm")
  if blk in ("qwen3_next", "qwen3_5"):
    return Family(norm_offset=1.0)           # every RMS scale is stored zero-centred and applied as (1 + scale)
  return Family()


def rope_tables(c, device) -> dict:
  """name -> (inverse timescales [rot_dim/2] fp32 on `device`, interleaved-lane flag)."""
  yarn = dict(rope_factor=c.rope_factor, original_max_position_embeddings=c.original_max_position_embeddings,
              beta_fast=c.beta_fast, beta_slow=c.beta_slow, rope_truncate=c.rope_truncate)
  rt = c.rope_type
  if c.model_name.startswith("llama3.1") or c.model_name.startswith("llama3.3"):
    rt = "llama3.1"
  dim = c.qk_rope_head_dim if c.attention_type == "mla" else c.head_dim
  rot = int(dim * c.partial_rotary_factor) if c.partial_rotary_factor < 1.0 else dim
  interleaved = rt.startswith("llama3.1") or (rt == "yarn" and c.rope_interleave)
  scaling = c.rope_linear_scaling_factor
  tables = {
      "default": (ref.rope_inv_timescale(rot, c.rope_min_timescale, c.rope_max_timescale, scaling, rt, c.rope_use_scale,
                                         yarn).to(device), interleaved),
  }
  local_max = c.local_rope_max_timescale if c.local_rope_max_timescale > 0 else c.rope_max_timescale
  # local (sliding-window) layers never use the long-context linear scaling (gemma3)
  tables["local"] = (ref.rope_inv_timescale(rot, c.rope_min_timescale, local_max, 1.0, "default").to(device), False)
  if c.decoder_block == "gemma4":
    # proportional rotary embedding (src/maxtext/models/gemma4.py:198-213): frequencies are spaced over the WHOLE head width and
    # only the first `proportion` of the angle pairs rotate; the others keep frequency zero (identity)
    def prop(head_dim, proportion, max_ts):
      t = ref.rope_inv_timescale(head_dim, c.rope_min_timescale, max_ts, 1.0, "default")
      t[int(proportion * head_dim // 2):] = 0.0
      return t.to(device)
    g_dim = int(c.global_head_dim or c.head_dim)
    g_max = c.global_rope_max_timescale if c.global_rope_max_timescale > 0 else c.rope_max_timescale
    tables["gemma4_global"] = (prop(g_dim, float(c.global_rope_proportion), g_max), False)
    tables["gemma4_local"] = (prop(int(c.head_dim), float(c.local_rope_proportion), local_max), False)
  return tables


def _llama_like(c, **kw) -> BlockPlan:
  return BlockPlan(window=c.sliding_window_size if c.attention_type == "local_sliding" or c.decoder_block == "mistral" else 0,
                   qk_norm=c.use_qk_norm, attn_bias=c.attention_bias, soft_cap=c.attn_logits_soft_cap, **kw)


def layer_plans(c) -> list[LayerPlan]:
  n = c.num_decoder_layers
  blk = c.decoder_block
  mla = c.attention_type == "mla"
  attn = "mla" if mla else "gqa"
  if blk in ("default", "llama2", "mistral", "simple", "simple_mlp"):
    return [LayerPlan("layers", [_llama_like(c, attention=attn)]) for _ in range(n)]
  if blk == "qwen3":
    # src/maxtext/models/qwen3.py:1451: q and k are RMS-normalised per head, so 1/sqrt(head_dim) cannot live in the
    # query weights; it multiplies the normalised query at run time
    return [LayerPlan("layers", [_llama_like(c, attention=attn, query_scalar=c.head_dim ** -0.5)]) for _ in range(n)]
  if blk == "olmo3":
    # src/maxtext/models/olmo3.py: no pre-norms; the attention and MLP outputs are normalised before the residual add;
    # cycles of (local, local, local, global) attention form one scanned block with sub-trees layers_0 .. layers_3
    cyc = max(1, int(c.inhomogeneous_layer_cycle_interval))
    assert n % cyc == 0, "olmo3 layers must be a multiple of inhomogeneous_layer_cycle_interval"
    blocks = [BlockPlan(prefix=f"layers_{j}", pre_attn_norm=None, pre_mlp_norm=None, attn_name="attention",
                        post_attn_norm="post_self_attention_layer_norm", post_mlp_norm="post_mlp_layer_norm",
                        window=c.sliding_window_size if (j % 4) != 3 else 0, qk_norm=c.use_qk_norm, query_scalar=c.head_dim ** -0.5,
                        global_qk_norm=True, attn_bias=c.attention_bias) for j in range(cyc)]
    return [LayerPlan("layers", blocks) for _ in range(n // cyc)]
  if blk == "envy":
    # src/maxtext/models/envy.py: cycles of inhomogeneous_layer_cycle_interval layers (sub-trees layers_0 ..) form one scanned
    # block; every interleave_moe_layer_step-th layer of a cycle has a routed MoE (MoeBlock_0), the others a dense MLP; the
    # query is scaled by head_dim^-1/2 at run time; optional q/k norms and a norm on the feed-forward output
    cyc = max(1, int(c.inhomogeneous_layer_cycle_interval))
    assert n % cyc == 0, "envy layers must be a multiple of inhomogeneous_layer_cycle_interval"
    step = max(1, int(c.interleave_moe_layer_step))
    blocks = []
    for j in range(cyc):
      is_moe = c.num_experts > 1 and (j + 1) % step == 0
      blocks.append(BlockPlan(prefix=f"layers_{j}", query_scalar=c.head_dim ** -0.5, qk_norm=bool(c.use_qk_norm),
                              post_mlp_norm="post_ffw_norm" if c.use_post_ffw_norm else None,
                              mlp="moe" if is_moe else "dense", mlp_name="MoeBlock_0" if is_moe else "mlp"))
    return [LayerPlan("layers", blocks) for _ in range(n // cyc)]
  if blk == "llama4":
    # src/maxtext/models/llama4.py:267-420: every nope_layer_interval-th layer has no RoPE, global attention and the
    # temperature-tuned query; the others use RoPE, chunked attention and scale-free q/k normalisation; MoE layers
    # (routed top-1 + shared expert) every interleave_moe_layer_step layers
    plans = []
    for i in range(n):
      nope = c.nope_layer_interval > 0 and (i + 1) % c.nope_layer_interval == 0
      is_moe = c.num_experts > 1 and (i + 1) % max(1, c.interleave_moe_layer_step) == 0
      plans.append(LayerPlan("layers", [BlockPlan(
          use_rope=not nope, chunk=0 if nope else int(c.chunk_attn_window_size), query_scalar=c.head_dim ** -0.5, l2_qk_norm=bool(c.use_qk_norm) and not nope,
          temperature_tuning=bool(c.temperature_tuning) and nope, mlp="moe_shared" if is_moe else "dense",
          mlp_name="Llama4MoEBlock_0" if is_moe else "mlp", moe_style="llama4" if is_moe else "")]))
    return plans
  if blk == "qwen2":
    bp = _llama_like(c, attention=attn)
    bp.attn_bias = True
    bp.attn_out_bias = False
    return [LayerPlan("layers", [bp]) for _ in range(n)]
  if blk == "mixtral":
    return [LayerPlan("layers", [_llama_like(c, mlp="moe", mlp_name="MoeBlock_0")]) for _ in range(n)]
  if blk in ("qwen3_moe", "qwen3_custom_moe"):
    return [LayerPlan("layers", [_llama_like(c, mlp="moe", mlp_name="moe_block", query_scalar=c.head_dim ** -0.5)])
            for _ in range(n)]
  if blk in ("qwen3_next", "qwen3_5"):
    # qwen3_5 reuses the qwen3-next layers unchanged (src/maxtext/models/qwen3_5.py)
    # src/maxtext/models/qwen3.py:1196-1420: cycles of inhomogeneous_layer_cycle_interval layers form one scanned block with
    # sub-trees layer_0 .. layer_{n-1}; the last layer of a cycle is gated full attention (partial RoPE, zero-centred
    # per-head q/k norms), the others are gated delta networks; every layer has the routed + gated shared expert MLP
    cyc = max(1, int(c.inhomogeneous_layer_cycle_interval))
    assert n % cyc == 0, "qwen3_next layers must be a multiple of inhomogeneous_layer_cycle_interval"
    blocks = []
    for j in range(cyc):
      full = (j + 1) % cyc == 0
      blocks.append(BlockPlan(prefix=f"layer_{j}", pre_attn_norm="input_layernorm", pre_mlp_norm="post_attention_layernorm",
                              attention="gqa" if full else "gdn", attn_name="attention/attention" if full else "attention",
                              gated_attn=full, qk_norm=full, query_scalar=c.head_dim ** -0.5 if full else None, norm_offset=1.0,
                              mlp="moe_shared", mlp_name="mlp", moe_style="qwen3_next"))
    return [LayerPlan("layers", blocks) for _ in range(n // cyc)]
  if blk == "deepseek":
    nd = c.first_num_dense_layers
    dense = [LayerPlan("dense_layers", [_llama_like(c, attention=attn)]) for _ in range(nd)]
    moe = [LayerPlan("moe_layers", [_llama_like(c, attention=attn, mlp="moe_shared", mlp_name="DeepSeekMoeBlock_0")])
           for _ in range(n - nd)]
    return dense + moe
  if blk == "deepseek4":
    # src/maxtext/models/deepseek4.py + src/maxtext/layers/decoders.py:1554-1640: `first_num_hash_layers` prefix layers with
    # their own compression ratios and hash routing, then pairs of (heavy, sparse) compressed-attention layers that form
    # one scanned block (`scanned_blocks`, sub-trees layers_0 / layers_1). Every layer has a routed MoE with shared experts.
    ratios = [int(r) for r in c.compress_ratios]
    nh = int(c.first_num_hash_layers)
    assert len(ratios) >= n, "compress_ratios must name every decoder layer"
    assert (n - nh) % 2 == 0, "the layers after the hash-routed prefix come in (heavy, sparse) pairs"

    def v4(ratio, prefix=""):
      return _llama_like(c, attention="compressed", attn_name="self_attention", mlp="moe_shared", mlp_name="DeepSeekMoeBlock_0",
                         compress_ratio=ratio, prefix=prefix)
    plans = [LayerPlan("layers", [v4(ratios[i])]) for i in range(nh)]
    for i in range(nh, n, 2):
      plans.append(LayerPlan("scanned_blocks", [v4(ratios[i], "layers_0"), v4(ratios[i + 1], "layers_1")]))
    return plans
  if blk == "gemma":
    bp = BlockPlan(pre_attn_norm="pre_self_attention_norm", pre_mlp_norm="pre_ffw_norm", soft_cap=c.attn_logits_soft_cap)
    return [LayerPlan("layers", [bp]) for _ in range(n)]
  if blk == "gemma2":
    def sub(suffix, window):
      return BlockPlan(suffix=suffix, pre_attn_norm="pre_self_attention_norm", pre_mlp_norm="pre_ffw_norm",
                       post_attn_norm="post_self_attention_norm" if c.use_post_attn_norm else None,
                       post_mlp_norm="post_ffw_norm" if c.use_post_ffw_norm else None, window=window,
                       soft_cap=c.attn_logits_soft_cap)
    return [LayerPlan("layers", [sub("_local", c.sliding_window_size), sub("_global", 0)]) for _ in range(n)]
  if blk == "gemma3":
    plans = []
    if c.model_name in ("gemma3-27b",):
      qs = (c.base_emb_dim // c.base_num_query_heads) ** -0.5
    else:
      qs = c.head_dim ** -0.5
    for i in range(n):
      local = (i % 6) != 5
      plans.append(LayerPlan("layers", [BlockPlan(
          pre_attn_norm="pre_self_attention_norm", pre_mlp_norm="pre_ffw_norm",
          post_attn_norm="post_self_attention_norm" if c.use_post_attn_norm else None,
          post_mlp_norm="post_ffw_norm" if c.use_post_ffw_norm else None,
          window=c.sliding_window_size if local else 0, rope="local" if local else "default", qk_norm=True,
          query_scalar=qs, soft_cap=c.attn_logits_soft_cap)]))
    return plans
  if blk == "gemma4":
    # src/maxtext/models/gemma4.py:40-55,150-410: five sliding-window layers then one global layer; global layers may have their
    # own head width / key-value head count and reuse the key projection as the value; q, k (scaled) and v (scale-free) are
    # RMS-normalised, no 1/sqrt(d) factor; every layer output is multiplied by a learned scalar; MoE variants add routed
    # experts next to the dense MLP (the "shared expert")
    plans = []
    for i in range(n):
      glob = (i % 6) == 5
      plans.append(LayerPlan("layers", [BlockPlan(
          pre_attn_norm="pre_self_attention_norm", pre_mlp_norm="pre_ffw_norm",
          post_attn_norm="post_self_attention_norm" if c.use_post_attn_norm else None,
          post_mlp_norm="post_ffw_norm" if c.use_post_ffw_norm else None,
          window=0 if glob else c.sliding_window_size, rope="gemma4_global" if glob else "gemma4_local", qk_norm=True,
          query_scalar=1.0, soft_cap=c.attn_logits_soft_cap, v_norm="scale" if c.v_norm_with_scale else "noscale",
          head_dim=int(c.global_head_dim or c.head_dim) if glob else None,
          kv_heads=int(c.global_num_kv_heads or c.num_kv_heads) if glob else None,
          share_kv=bool(c.share_kv_projections) and glob, layer_scalar=True,
          mlp="gemma4_moe" if c.num_experts > 1 else "dense")]))
    return plans
  if blk == "gpt3":
    bp = BlockPlan(pre_attn_norm="pre_self_attention_norm", pre_mlp_norm="post_self_attention_norm", use_rope=False,
                   attn_bias=True, mlp_bias=True, norm_kind="layernorm")
    return [LayerPlan("layers", [bp]) for _ in range(n)]
  if blk == "gpt_oss":
    plans = []
    for i in range(n):
      local = (i % 2) == 0
      plans.append(LayerPlan("layers", [BlockPlan(window=c.sliding_window_size if local else 0, attn_bias=True, sinks=True,
                                                  query_scalar=c.head_dim ** -0.5, mlp="moe", mlp_name="GptOssMlp", moe_style="gpt_oss")]))
    return plans
  raise NotImplementedError(
      f"decoder_block={blk!r} parses but has no model implementation here yet (implemented: llama2, mistral, mixtral, "
      "deepseek, gemma, gemma2, gemma3, qwen2, qwen3, qwen3_moe, qwen3_next, qwen3_5, gpt3, gpt_oss, olmo3, llama4, envy, gemma4, deepseek4, simple)")
