"""HuggingFace <-> this framework's parameters (Llama / Mistral / Qwen2/3 / Gemma dense families, Mixtral MoE).

The stored conventions are MaxText's (src/maxtext/checkpoint_conversion/utils/param_mapping.py:2436-2570):
kernels `[in..., out...]`, query pre-multiplied by 1/sqrt(head_dim) (unless the model uses QK-norm or an explicit
query scalar) and, for rope_type=llama3.1 (interleaved lanes), query/key lanes permuted from HF's concatenated-halves
order to adjacent pairs. `to_maxtext` loads an HF state dict into a ParamStore, `to_hf` exports one;
`convert_*_checkpoint` wrap them around safetensors files and this repository's checkpoint directories.
"""
from __future__ import annotations

import json
import math
import os

import torch

from ..parallel import param_store as ps


def _interleave(w_out_in: torch.Tensor, heads: int, dh: int) -> torch.Tensor:
  """[heads*dh, in] with per-head lanes (first half | second half) -> adjacent pairs."""
  w = w_out_in.view(heads, 2, dh // 2, -1)
  return w.permute(0, 2, 1, 3).reshape(heads * dh, -1)


def _deinterleave(w_out_in: torch.Tensor, heads: int, dh: int) -> torch.Tensor:
  w = w_out_in.view(heads, dh // 2, 2, -1)
  return w.permute(0, 2, 1, 3).reshape(heads * dh, -1)


def _locate(pdef, cfg) -> tuple[str, int | None]:
  """(path relative to one HF decoder layer, HF layer index) of one of our parameters.

  Stacks that hold several HF layers per scanned unit are unrolled here: gemma2 keeps a (local, global) pair per
  unit with suffixed module names, olmo3 a cycle of `layers_<j>` sub-trees, deepseek numbers its MoE stack after
  the dense one."""
  parts = list(pdef.ref_path)
  L = pdef.layer
  if L is None:
    return "/".join(parts), None
  blk = cfg.decoder_block
  if blk == "olmo3" and parts[0].startswith("layers_"):
    cyc = max(1, int(cfg.inhomogeneous_layer_cycle_interval))
    L = L * cyc + int(parts[0].split("_")[1])
    parts = parts[1:]
    if parts[0] == "attention":
      parts[0] = "self_attention"
  elif blk in ("qwen3_next", "qwen3_5") and parts[0].startswith("layer_"):
    cyc = max(1, int(cfg.inhomogeneous_layer_cycle_interval))
    L = L * cyc + int(parts[0].split("_")[1])
    parts = parts[1:]
    if parts[:2] == ["attention", "attention"]:
      parts = ["self_attention"] + parts[2:]
  elif blk == "gemma2":
    for sfx, j in (("_local", 0), ("_global", 1)):
      if parts[0].endswith(sfx):
        parts[0] = parts[0][:-len(sfx)]
        L = 2 * L + j
        break
  elif blk == "deepseek" and getattr(pdef, "stack", "") == "moe_layers":
    L = L + int(cfg.first_num_dense_layers)
  return "/".join(parts), L


# which expert matrix a stacked MoE parameter is, by the last path component
_EXPERT_PART = {"wi_0": "gate", "wi_1": "up", "wo": "down", "wi_0_bias": "gate_bias", "wi_1_bias": "up_bias", "wo_bias": "down_bias"}


def _llama4_vision_name(path: str) -> tuple[str, str] | None:
  """Llama-4 vision tower (HF: `vision_model.*`, `multi_modal_projector.linear_1`)."""
  import re
  vm = "vision_model."
  rest = path.split("/", 2)[2] if path.count("/") >= 2 else ""
  if path.startswith("vision_encoder/Llama4MultiModalProjector_0/"):
    return "multi_modal_projector.linear_1.weight", "linear"
  top = {"Llama4UnfoldConvolution_0/vit_unfold_linear/kernel": (vm + "patch_embedding.linear.weight", "linear"),
         "class_embedding": (vm + "class_embedding", "vec"), "positional_embedding_vlm": (vm + "positional_embedding_vlm", "vec"),
         "layernorm_pre/scale": (vm + "layernorm_pre.weight", "vec"), "layernorm_pre/bias": (vm + "layernorm_pre.bias", "vec"),
         "layernorm_post/scale": (vm + "layernorm_post.weight", "vec"), "layernorm_post/bias": (vm + "layernorm_post.bias", "vec"),
         "Llama4VisionPixelShuffleMLP_0/pixel_shuffle_mlp/vit_pixel_shuffle_mlp_fc1/kernel": (vm + "vision_adapter.mlp.fc1.weight", "linear"),
         "Llama4VisionPixelShuffleMLP_0/pixel_shuffle_mlp/vit_pixel_shuffle_mlp_fc2/kernel": (vm + "vision_adapter.mlp.fc2.weight", "linear")}
  if rest in top:
    return top[rest]
  m = re.match(r"Llama4VisionEncoder_0/layers_(\d+)/(.+)", rest)
  if not m:
    return None
  pre = f"{vm}model.layers.{m.group(1)}."
  sub = {"input_layer_norm": "input_layernorm", "post_attention_layer_norm": "post_attention_layernorm",
         "self_attention_vision/query": "self_attn.q_proj", "self_attention_vision/key": "self_attn.k_proj",
         "self_attention_vision/value": "self_attn.v_proj", "self_attention_vision/out": "self_attn.o_proj",
         "Llama4VisionMLP_0/vit_encoder_layer_mlp_fc1": "mlp.fc1", "Llama4VisionMLP_0/vit_encoder_layer_mlp_fc2": "mlp.fc2"}
  mod, leaf = m.group(2).rsplit("/", 1)
  if mod not in sub:
    return None
  return pre + sub[mod] + (".bias" if leaf == "bias" else ".weight"), ("linear" if leaf == "kernel" else "vec")


def _qwen_audio_name(path: str) -> tuple[str, str] | None:
  """Qwen3-Omni audio tower (HF: thinker.audio_tower.*): convolutions, encoder layers with biased projections, output head."""
  import re
  a = "thinker.audio_tower."
  m = re.match(r"audio_encoder/(conv2d[123]|conv_out)/(kernel|bias)$", path)
  if m:
    return a + m.group(1) + (".weight" if m.group(2) == "kernel" else ".bias"), ("linear" if m.group(1) == "conv_out" else "vec")
  m = re.match(r"audio_encoder/ln_post/(scale|bias)$", path)
  if m:
    return a + "ln_post." + ("weight" if m.group(1) == "scale" else "bias"), "vec"
  m = re.match(r"audio_projector/(proj[12])/(kernel|bias)$", path)
  if m:
    return a + m.group(1) + (".weight" if m.group(2) == "kernel" else ".bias"), ("linear" if m.group(2) == "kernel" else "vec")
  m = re.match(r"audio_encoder/layers_(\d+)/(.+)/(scale|bias|kernel)$", path)
  if not m:
    return None
  pre, mod, leaf = a + f"layers.{m.group(1)}.", m.group(2), m.group(3)
  sub = {"self_attn_layer_norm": "self_attn_layer_norm", "final_layer_norm": "final_layer_norm", "self_attn/query": "self_attn.q_proj",
         "self_attn/key": "self_attn.k_proj", "self_attn/value": "self_attn.v_proj", "self_attn/out": "self_attn.out_proj", "fc1": "fc1", "fc2": "fc2"}.get(mod)
  if sub is None:
    return None
  return pre + sub + (".bias" if leaf == "bias" else ".weight"), ("linear" if leaf == "kernel" else "vec")


def _qwen_vision_name(path: str) -> tuple[str, str] | None:
  """Qwen3-VL vision tower (HF: model.visual.*). The fused qkv of the HF blocks is cut into our query / key / value (kinds
  qkv0..2 name the third), the 3-D patch convolution becomes a matrix over (t, py, px, c) features (kind patch3d)."""
  import re
  v = "model.visual."
  top = {"vision_encoder/patch_embed/proj/kernel": (v + "patch_embed.proj.weight", "patch3d"),
         "vision_encoder/patch_embed/proj/bias": (v + "patch_embed.proj.bias", "vec"),
         "vision_encoder/pos_embed_interpolate/pos_embed": (v + "pos_embed.weight", "vec")}
  if path in top:
    return top[path]
  m = re.match(r"(vision_projector/merger|vision_encoder/merger_(\d+))/(ln_q|mlp_0|mlp_2)/(scale|bias|kernel)$", path)
  if m:
    mod = "merger" if m.group(2) is None else f"deepstack_merger_list.{m.group(2)}"
    sub = {"ln_q": "norm", "mlp_0": "linear_fc1", "mlp_2": "linear_fc2"}[m.group(3)]
    return v + f"{mod}.{sub}." + ("bias" if m.group(4) == "bias" else "weight"), ("linear" if m.group(4) == "kernel" else "vec")
  m = re.match(r"vision_encoder/blocks_(\d+)/(.+)/(scale|bias|kernel)$", path)
  if not m:
    return None
  pre, mod, leaf = v + f"blocks.{m.group(1)}.", m.group(2), m.group(3)
  suffix = "bias" if leaf == "bias" else "weight"
  if mod in ("ln1", "ln2"):
    return pre + {"ln1": "norm1", "ln2": "norm2"}[mod] + "." + suffix, "vec"
  if mod in ("attn/attn/query", "attn/attn/key", "attn/attn/value"):
    j = ("query", "key", "value").index(mod.rsplit("/", 1)[1])
    return pre + "attn.qkv." + suffix, f"qkv{j}"
  sub = {"attn/attn/out": "attn.proj", "mlp": "mlp.linear_fc1", "mlp_out": "mlp.linear_fc2"}.get(mod)
  if sub is None:
    return None
  return pre + sub + "." + suffix, ("linear" if leaf == "kernel" else "vec")


def _vision_name(path: str) -> tuple[str, str] | None:
  """Gemma-3 vision tower and projector (HF: SigLIP under model.vision_tower, model.multi_modal_projector)."""
  import re
  if path.startswith(("vision_encoder/patch_embed/", "vision_encoder/pos_embed_interpolate/", "vision_encoder/blocks_", "vision_encoder/merger_",
                      "vision_projector/merger/")):
    return _qwen_vision_name(path)
  if path.startswith(("vision_encoder/Llama4VisionModel_0/", "vision_encoder/Llama4MultiModalProjector_0/")):
    return _llama4_vision_name(path)
  vt = "model.vision_tower.vision_model."
  if path.startswith("vision_encoder/VisionEmbedder_0/"):
    return {"mm_soft_embedding_norm/scale": ("model.multi_modal_projector.mm_soft_emb_norm.weight", "norm"),
            "mm_input_projection/w": ("model.multi_modal_projector.mm_input_projection_weight", "linear_io")}.get(path.split("/", 2)[2])
  rest = path.split("/", 2)[2]
  top = {"embedding/kernel": (vt + "embeddings.patch_embedding.weight", "patch"),
         "embedding/bias": (vt + "embeddings.patch_embedding.bias", "vec"),
         "pos_embedding": (vt + "embeddings.position_embedding.weight", "vec"),
         "Transformer/encoder_norm/scale": (vt + "post_layernorm.weight", "vec"),
         "Transformer/encoder_norm/bias": (vt + "post_layernorm.bias", "vec")}
  if rest in top:
    return top[rest]
  m = re.match(r"Transformer/encoderblock_(\d+)/(.+)", rest)
  if not m:
    return None
  pre = f"{vt}encoder.layers.{m.group(1)}."
  sub = {"LayerNorm_0": "layer_norm1", "LayerNorm_1": "layer_norm2", "MultiHeadDotProductAttention_0/query": "self_attn.q_proj",
         "MultiHeadDotProductAttention_0/key": "self_attn.k_proj", "MultiHeadDotProductAttention_0/value": "self_attn.v_proj",
         "MultiHeadDotProductAttention_0/out": "self_attn.out_proj", "MlpBlockViT_0/Dense_0": "mlp.fc1", "MlpBlockViT_0/Dense_1": "mlp.fc2"}
  mod, leaf = m.group(2).rsplit("/", 1)
  if mod not in sub:
    return None
  return pre + sub[mod] + (".bias" if leaf == "bias" else ".weight"), ("linear" if leaf == "kernel" else "vec")


def _hf_name(pdef, cfg) -> tuple[str, str] | None:
  """(hf key, kind) for one of our parameters. Kinds: linear, vec, norm, embed, q, k, qbias, kbias, and
  experts:<part> for stacked expert tensors (the key is then the HF layer prefix)."""
  path, L = _locate(pdef, cfg)
  if path.startswith(("vision_encoder/", "vision_projector/")):
    return _vision_name(path)
  if path.startswith(("audio_encoder/", "audio_projector/")):
    return _qwen_audio_name(path)
  pre = f"model.layers.{L}." if L is not None else ""
  blk = cfg.decoder_block
  sandwich = blk in ("gemma2", "gemma3", "gemma4")
  table = {
      "token_embedder/embedding": ("model.embed_tokens.weight", "embed"),
      "decoder/decoder_norm/scale": ("model.norm.weight", "norm"),
      "decoder/logits_dense/kernel": ("lm_head.weight", "linear"),
      "self_attention/query/kernel": (pre + "self_attn.q_proj.weight", "q"),
      "self_attention/key/kernel": (pre + "self_attn.k_proj.weight", "k"),
      "self_attention/value/kernel": (pre + "self_attn.v_proj.weight", "linear"),
      "self_attention/out/kernel": (pre + "self_attn.o_proj.weight", "linear"),
      "self_attention/query/bias": (pre + "self_attn.q_proj.bias", "qbias"),
      "self_attention/key/bias": (pre + "self_attn.k_proj.bias", "kbias"),
      "self_attention/value/bias": (pre + "self_attn.v_proj.bias", "vec"),
      "self_attention/out/bias": (pre + "self_attn.o_proj.bias", "vec"),
      "self_attention/sinks": (pre + "self_attn.sinks", "vec"),
      "self_attention/query_norm/scale": (pre + "self_attn.q_norm.weight", "norm"),
      "self_attention/key_norm/scale": (pre + "self_attn.k_norm.weight", "norm"),
      # multi-head latent attention (DeepSeek)
      "self_attention/query/kernel#mla": (pre + "self_attn.q_proj.weight", "linear"),
      "self_attention/wq_a/kernel": (pre + "self_attn.q_a_proj.weight", "linear"),
      "self_attention/q_norm/scale": (pre + "self_attn.q_a_layernorm.weight", "norm"),
      "self_attention/wq_b/kernel": (pre + "self_attn.q_b_proj.weight", "linear"),
      "self_attention/wkv_a/kernel": (pre + "self_attn.kv_a_proj_with_mqa.weight", "linear"),
      "self_attention/kv_norm/scale": (pre + "self_attn.kv_a_layernorm.weight", "norm"),
      "self_attention/wkv_b/kernel": (pre + "self_attn.kv_b_proj.weight", "linear"),
      "pre_self_attention_layer_norm/scale": (pre + "input_layernorm.weight", "norm"),
      "post_self_attention_layer_norm/scale": (pre + "post_attention_layernorm.weight", "norm"),
      "post_mlp_layer_norm/scale": (pre + "post_feedforward_layernorm.weight", "norm"),
      "pre_self_attention_norm/scale": (pre + "input_layernorm.weight", "norm"),
      "pre_ffw_norm/scale": (pre + ("pre_feedforward_layernorm.weight" if sandwich else "post_attention_layernorm.weight"), "norm"),
      "post_self_attention_norm/scale": (pre + "post_attention_layernorm.weight", "norm"),
      "post_ffw_norm/scale": (pre + "post_feedforward_layernorm.weight", "norm"),
      "mlp/wi_0/kernel": (pre + "mlp.gate_proj.weight", "linear"),
      "mlp/wi_1/kernel": (pre + "mlp.up_proj.weight", "linear"),
      "mlp/wo/kernel": (pre + "mlp.down_proj.weight", "linear"),
      "MoeBlock_0/gate/kernel": (pre + "block_sparse_moe.gate.weight", "linear"),
      "moe_block/gate/kernel": (pre + "mlp.gate.weight", "linear"),
      "DeepSeekMoeBlock_0/MoeBlock_0/gate/kernel": (pre + "mlp.gate.weight", "linear"),
      "DeepSeekMoeBlock_0/MoeBlock_0/gate/bias": (pre + "mlp.gate.e_score_correction_bias", "vec"),
      "DeepSeekMoeBlock_0/shared_experts/wi_0/kernel": (pre + "mlp.shared_experts.gate_proj.weight", "linear"),
      "DeepSeekMoeBlock_0/shared_experts/wi_1/kernel": (pre + "mlp.shared_experts.up_proj.weight", "linear"),
      "DeepSeekMoeBlock_0/shared_experts/wo/kernel": (pre + "mlp.shared_experts.down_proj.weight", "linear"),
      # qwen3-next: gated delta network layers and the gated shared expert
      "input_layernorm/scale": (pre + "input_layernorm.weight", "norm"),
      "post_attention_layernorm/scale": (pre + "post_attention_layernorm.weight", "norm"),
      "attention/in_proj_qkvz/kernel": (pre + "linear_attn.in_proj_qkvz.weight", "linear"),
      "attention/in_proj_ba/kernel": (pre + "linear_attn.in_proj_ba.weight", "linear"),
      "attention/conv1d/kernel": (pre + "linear_attn.conv1d.weight", "conv"),
      "attention/A_log": (pre + "linear_attn.A_log", "vec"),
      "attention/dt_bias": (pre + "linear_attn.dt_bias", "vec"),
      "attention/norm/rms_norm/scale": (pre + "linear_attn.norm.weight", "vec"),
      "attention/out_proj/kernel": (pre + "linear_attn.out_proj.weight", "linear"),
      "mlp/routed_experts/gate/kernel": (pre + "mlp.gate.weight", "linear"),
      "mlp/shared_expert/wi_0/kernel": (pre + "mlp.shared_expert.gate_proj.weight", "linear"),
      "mlp/shared_expert/wi_1/kernel": (pre + "mlp.shared_expert.up_proj.weight", "linear"),
      "mlp/shared_expert/wo/kernel": (pre + "mlp.shared_expert.down_proj.weight", "linear"),
      "mlp/shared_expert_gate/kernel": (pre + "mlp.shared_expert_gate.weight", "linear"),
      "GptOssMlp/gate/kernel": (pre + "mlp.router.weight", "linear"),
      "GptOssMlp/gate/bias": (pre + "mlp.router.bias", "vec"),
      # gemma4: learned layer scalar; MoE layers keep a dense MLP (stored as the block's shared experts) next to the routed experts
      "layer_scalar": (pre + "layer_scalar", "vec"),
      "mlp/moe_block/shared_experts/wi_0/kernel": (pre + "mlp.gate_proj.weight", "linear"),
      "mlp/moe_block/shared_experts/wi_1/kernel": (pre + "mlp.up_proj.weight", "linear"),
      "mlp/moe_block/shared_experts/wo/kernel": (pre + "mlp.down_proj.weight", "linear"),
      "mlp/moe_block/MoeBlock_0/gate/kernel": (pre + "router.proj.weight", "linear"),
      "mlp/moe_block/MoeBlock_0/per_expert_scale": (pre + "router.per_expert_scale", "vec"),
      "mlp/pre_forward_scale_2": (pre + "router.scale", "vec"),
      "mlp/pre_feedforward_layernorm_2/scale": (pre + "pre_feedforward_layernorm_2.weight", "norm"),
      "mlp/post_feedforward_layernorm_1/scale": (pre + "post_feedforward_layernorm_1.weight", "norm"),
      "mlp/post_feedforward_layernorm_2/scale": (pre + "post_feedforward_layernorm_2.weight", "norm"),
      "Llama4MoEBlock_0/MoeBlock_0/gate/kernel": (pre + "feed_forward.router.weight", "linear"),
      "Llama4MoEBlock_0/shared_experts/wi_0/kernel": (pre + "feed_forward.shared_expert.gate_proj.weight", "linear"),
      "Llama4MoEBlock_0/shared_experts/wi_1/kernel": (pre + "feed_forward.shared_expert.up_proj.weight", "linear"),
      "Llama4MoEBlock_0/shared_experts/wo/kernel": (pre + "feed_forward.shared_expert.down_proj.weight", "linear"),
  }
  if cfg.attention_type == "mla" and path == "self_attention/query/kernel":
    path += "#mla"
  if blk == "llama4" and path.startswith("mlp/"):
    return pre + "feed_forward." + {"wi_0": "gate_proj", "wi_1": "up_proj", "wo": "down_proj"}[path.split("/")[1]] + ".weight", "linear"
  hit = table.get(path)
  if hit is not None:
    return hit
  last = path.split("/")[-1]
  if pdef.kind == "experts" or (last in _EXPERT_PART and path.split("/")[0] in
                                ("MoeBlock_0", "moe_block", "DeepSeekMoeBlock_0", "GptOssMlp", "Llama4MoEBlock_0", "mlp")):
    return pre, "experts:" + _EXPERT_PART[last]
  return None


def _expert_style(cfg) -> str:
  return {"mixtral": "mixtral", "gpt_oss": "gpt_oss", "llama4": "llama4", "gemma4": "gemma4"}.get(cfg.decoder_block, "split")


def _load_experts(hf_state: dict, pre: str, part: str, cfg) -> torch.Tensor | None:
  """Stacked `[E, out, in]` (or `[E, out]` bias) tensor of one expert matrix from whichever layout the HF dict uses:
  one module per expert (hub checkpoints) or one stacked tensor with gate and up fused (in-memory models)."""
  E = cfg.num_experts
  style = _expert_style(cfg)
  if style == "gpt_oss":
    # gate_up_proj [E, in, 2*out] with gate and up in alternating columns; down_proj [E, in, out]
    base = pre + "mlp.experts."
    if part in ("gate", "up"):
      gu = hf_state.get(base + "gate_up_proj")
      return None if gu is None else gu.float()[:, :, (0 if part == "gate" else 1)::2].transpose(1, 2).contiguous()
    if part in ("gate_bias", "up_bias"):
      gb = hf_state.get(base + "gate_up_proj_bias")
      return None if gb is None else gb.float()[:, (0 if part == "gate_bias" else 1)::2].contiguous()
    if part == "down":
      d = hf_state.get(base + "down_proj")
      return None if d is None else d.float().transpose(1, 2).contiguous()
    d = hf_state.get(base + "down_proj_bias")
    return None if d is None else d.float()
  if style == "llama4":
    # gate_up_proj [E, in, 2*out] (gate | up halves); down_proj [E, in, out]
    base = pre + "feed_forward.experts."
    if part == "down":
      d = hf_state.get(base + "down_proj")
      return None if d is None else d.float().transpose(1, 2).contiguous()
    gu = hf_state.get(base + "gate_up_proj")
    if gu is None:
      return None
    half = gu.shape[2] // 2
    return (gu.float()[:, :, :half] if part == "gate" else gu.float()[:, :, half:]).transpose(1, 2).contiguous()
  if style == "gemma4":
    # experts sit directly under the layer: gate_up_proj [E, 2*out, in] (gate | up halves), down_proj [E, out, in]
    if part == "down":
      d = hf_state.get(pre + "experts.down_proj")
      return None if d is None else d.float()
    gu = hf_state.get(pre + "experts.gate_up_proj")
    if gu is None:
      return None
    half = gu.shape[1] // 2
    return gu.float()[:, :half] if part == "gate" else gu.float()[:, half:]
  if style == "mixtral":
    per = pre + "block_sparse_moe.experts.{e}." + {"gate": "w1", "up": "w3", "down": "w2"}[part] + ".weight"
  else:
    per = pre + "mlp.experts.{e}." + part + "_proj.weight"
  if per.format(e=0) in hf_state:
    return torch.stack([hf_state[per.format(e=e)].float() for e in range(E)])
  base = pre + "mlp.experts."
  if part == "down":
    d = hf_state.get(base + "down_proj")
    return None if d is None else d.float()
  gu = hf_state.get(base + "gate_up_proj")
  if gu is None:
    return None
  half = gu.shape[1] // 2
  return gu.float()[:, :half] if part == "gate" else gu.float()[:, half:]


def _store_experts(out: dict, pre: str, part: str, w: torch.Tensor, cfg):
  """Inverse of `_load_experts`, writing the layout hub checkpoints of the family use."""
  style = _expert_style(cfg)
  if style == "gemma4":
    if part == "down":
      out[pre + "experts.down_proj"] = w.contiguous()
    else:
      E_, half, d_in = w.shape
      gu = out.setdefault(pre + "experts.gate_up_proj", torch.zeros(E_, 2 * half, d_in))
      (gu[:, :half] if part == "gate" else gu[:, half:]).copy_(w)
    return
  if style in ("gpt_oss", "llama4"):
    base = pre + ("mlp.experts." if style == "gpt_oss" else "feed_forward.experts.")
    if part == "down":
      out[base + "down_proj"] = w.transpose(1, 2).contiguous()
    elif part == "down_bias":
      out[base + "down_proj_bias"] = w.contiguous()
    else:
      bias = part.endswith("_bias")
      key = base + ("gate_up_proj_bias" if bias else "gate_up_proj")
      piece = w if bias else w.transpose(1, 2)                       # [E, out] or [E, in, out]
      if key not in out:
        out[key] = torch.zeros(*piece.shape[:-1], 2 * piece.shape[-1])
      o = piece.shape[-1]
      first = part.startswith("gate")
      if style == "gpt_oss":
        out[key][..., (0 if first else 1)::2] = piece
      else:
        out[key][..., (slice(0, o) if first else slice(o, 2 * o))] = piece
    return
  per = (pre + "block_sparse_moe.experts.{e}." + {"gate": "w1", "up": "w3", "down": "w2"}[part] + ".weight") if style == "mixtral" \
      else (pre + "mlp.experts.{e}." + part + "_proj.weight")
  for e in range(w.shape[0]):
    out[per.format(e=e)] = w[e].contiguous()


def _norm_offset(cfg) -> float:
  # HF Gemma stores (scale - 1); MaxText stores the effective scale
  return 1.0 if cfg.decoder_block in ("gemma", "gemma2", "gemma3") else 0.0


def _embed_scale(cfg) -> float:
  # Gemma: HF multiplies the looked-up embedding by sqrt(hidden) at run time; here the factor lives in the table
  return math.sqrt(cfg.emb_dim) if cfg.decoder_block in ("gemma", "gemma2", "gemma3", "gemma4") else 1.0


def _q_scale(cfg) -> float:
  """Factor folded into the stored query projection: 1/sqrt(head_dim) unless the family scales at run time."""
  if cfg.use_qk_norm or cfg.attention_type == "mla" or cfg.decoder_block in ("gemma3", "gemma4", "qwen3", "qwen3_moe", "qwen3_custom_moe", "olmo3",
                                                                              "llama4", "gpt_oss", "qwen3_next", "qwen3_5"):
    return 1.0
  return 1.0 / math.sqrt(cfg.head_dim)


def _interleaved(cfg) -> bool:
  """Whether q/k lanes must be permuted from HF's concatenated halves to adjacent pairs. HF Llama-4 rotates adjacent
  pairs itself, so its tensors are already in that order."""
  if cfg.decoder_block == "llama4":
    return False
  return cfg.rope_type.startswith("llama3.1") or cfg.model_name.startswith("llama3.1") or cfg.model_name.startswith("llama3.3")


_ALIASES = (("block_sparse_moe.gate", "mlp.gate"),)


def _gdn_dims(cfg):
  hk, hv, dk, dv = int(cfg.gdn_num_key_heads), int(cfg.gdn_num_value_heads), int(cfg.gdn_key_head_dim), int(cfg.gdn_value_head_dim)
  return hk, hv, dk, dv, hv // hk


def _qwen35_pack(hf_state: dict, key: str, cfg) -> torch.Tensor | None:
  """Qwen3.5 stores the gated-delta input projections flat and separate (in_proj_qkv = [q | k | v], in_proj_z, in_proj_b,
  in_proj_a); the layer here (like Qwen3-Next) wants them grouped per key head: [q_h | k_h | v of its value heads | z of
  them] and [b | a]."""
  hk, hv, dk, dv, r = _gdn_dims(cfg)
  base = key.rsplit(".", 2)[0] + "."
  if key.endswith("in_proj_qkvz.weight"):
    qkv, z = hf_state.get(base + "in_proj_qkv.weight"), hf_state.get(base + "in_proj_z.weight")
    if qkv is None or z is None:
      return None
    qkv, z = qkv.float(), z.float()
    d = qkv.shape[1]
    q, k, v = qkv[:hk * dk].view(hk, dk, d), qkv[hk * dk:2 * hk * dk].view(hk, dk, d), qkv[2 * hk * dk:].view(hk, r * dv, d)
    return torch.cat([q, k, v, z.view(hk, r * dv, d)], dim=1).reshape(-1, d)
  b, a = hf_state.get(base + "in_proj_b.weight"), hf_state.get(base + "in_proj_a.weight")
  if b is None or a is None:
    return None
  d = b.shape[1]
  return torch.cat([b.float().view(hk, r, d), a.float().view(hk, r, d)], dim=1).reshape(-1, d)


def _qwen35_unpack(out: dict, key: str, w: torch.Tensor, cfg):
  hk, hv, dk, dv, r = _gdn_dims(cfg)
  base = key.rsplit(".", 2)[0] + "."
  d = w.shape[1]
  if key.endswith("in_proj_qkvz.weight"):
    g = w.view(hk, 2 * dk + 2 * r * dv, d)
    q, k, v, z = g[:, :dk], g[:, dk:2 * dk], g[:, 2 * dk:2 * dk + r * dv], g[:, 2 * dk + r * dv:]
    out[base + "in_proj_qkv.weight"] = torch.cat([q.reshape(-1, d), k.reshape(-1, d), v.reshape(-1, d)]).contiguous()
    out[base + "in_proj_z.weight"] = z.reshape(-1, d).contiguous()
  else:
    g = w.view(hk, 2 * r, d)
    out[base + "in_proj_b.weight"], out[base + "in_proj_a.weight"] = g[:, :r].reshape(-1, d).contiguous(), g[:, r:].reshape(-1, d).contiguous()


def to_maxtext(hf_state: dict, store, cfg) -> list[str]:
  """Fill `store` from an HF state dict. Returns the list of our parameters that had no HF source."""
  missing = []
  inter = _interleaved(cfg)
  for name, p in store.params.items():
    m = _hf_name(p.pdef, cfg)
    if m is None:
      missing.append(name)
      continue
    key, kind = m
    if kind.startswith("experts:"):
      w = None
      for pre_ in (key, "language_model." + key, "model.language_model." + key[6:]):      # multimodal checkpoints nest the text model
        w = _load_experts(hf_state, pre_, kind.split(":")[1], cfg)
        if w is not None:
          break
      if w is None:
        missing.append(name)
        continue
      store.load_full(name, p.pdef.local_slice(w.contiguous().reshape(p.pdef.global_shape())))
      continue
    if cfg.decoder_block == "qwen3_5" and key.endswith(("in_proj_qkvz.weight", "in_proj_ba.weight")) and key not in hf_state:
      w = _qwen35_pack(hf_state, key, cfg)
      if w is None:
        missing.append(name)
        continue
      store.load_full(name, p.pdef.local_slice(w.reshape(p.pdef.global_shape())))
      continue
    if key not in hf_state and key.startswith("model.") and "model.language_model." + key[6:] in hf_state:
      key = "model.language_model." + key[6:]          # multimodal checkpoints nest the text model one level deeper
    if key not in hf_state and "language_model." + key in hf_state:
      key = "language_model." + key                    # Llama-4 multimodal checkpoints
    if key not in hf_state:
      for a, b_ in _ALIASES:
        if a in key and key.replace(a, b_) in hf_state:
          key = key.replace(a, b_)
    if key not in hf_state:
      if key == "lm_head.weight" and "model.embed_tokens.weight" in hf_state:
        key = "model.embed_tokens.weight"
      else:
        missing.append(name)
        continue
    w = hf_state[key].float()
    if kind.startswith("qkv"):
      third = w.shape[0] // 3                # HF fuses query | key | value along the output dimension
      w = w[int(kind[3]) * third:(int(kind[3]) + 1) * third]
    elif kind == "patch3d":
      w = w.permute(0, 2, 3, 4, 1).reshape(w.shape[0], -1)          # conv [out, C, T, P, P] -> features (t, py, px, c)
    if kind == "q":
      if inter:
        w = _interleave(w, cfg.num_query_heads, cfg.head_dim)
      w = w * _q_scale(cfg)
    elif kind == "k" and inter:
      w = _interleave(w, cfg.num_kv_heads, cfg.head_dim)
    elif kind == "qbias":
      w = (_interleave(w[:, None], cfg.num_query_heads, cfg.head_dim)[:, 0] if inter else w) * _q_scale(cfg)
    elif kind == "kbias" and inter:
      w = _interleave(w[:, None], cfg.num_kv_heads, cfg.head_dim)[:, 0]
    elif kind == "norm":
      w = w + _norm_offset(cfg)
    elif kind == "embed":
      w = w * _embed_scale(cfg)
    elif kind == "conv":
      w = w.permute(2, 1, 0)               # HF depthwise filter [channels, 1, kernel] -> [kernel, 1, channels]
    elif kind == "patch":
      w = w.permute(0, 2, 3, 1)            # HF conv [out, C, P, P] -> rows ordered (py, px, C) like the patch cutter
    elif kind == "linear_io":
      w = w.t()                            # stored [in, out] on the HF side
    store.load_full(name, p.pdef.local_slice(w.reshape(p.pdef.global_shape())))
  store.sync_compute_from_master()
  return missing


def to_hf(store, cfg) -> dict:
  """Export the (fp32 master) parameters as an HF state dict."""
  out = {}
  inter = _interleaved(cfg)
  for name, p in store.params.items():
    m = _hf_name(p.pdef, cfg)
    if m is None:
      continue
    key, kind = m
    w = store.full_master(p).float().clone()
    if kind.startswith("qkv"):
      j, third = int(kind[3]), w.shape[0]
      full = out.setdefault(key, torch.zeros((3 * third,) + tuple(w.shape[1:])))
      full[j * third:(j + 1) * third] = w
      continue
    if kind == "patch3d":
      P, T = int(cfg.patch_size_for_vit), int(cfg.temporal_patch_size_for_vit)
      out[key] = w.view(w.shape[0], T, P, P, -1).permute(0, 4, 1, 2, 3).contiguous()
      continue
    if kind.startswith("experts:"):
      _store_experts(out, key, kind.split(":")[1], w, cfg)
      continue
    if cfg.decoder_block == "qwen3_5" and key.endswith(("in_proj_qkvz.weight", "in_proj_ba.weight")):
      _qwen35_unpack(out, key, w, cfg)
      continue
    if kind == "q":
      w = w / _q_scale(cfg)
      if inter:
        w = _deinterleave(w, cfg.num_query_heads, cfg.head_dim)
    elif kind == "k" and inter:
      w = _deinterleave(w, cfg.num_kv_heads, cfg.head_dim)
    elif kind == "qbias":
      w = w / _q_scale(cfg)
      if inter:
        w = _deinterleave(w[:, None], cfg.num_query_heads, cfg.head_dim)[:, 0]
    elif kind == "kbias" and inter:
      w = _deinterleave(w[:, None], cfg.num_kv_heads, cfg.head_dim)[:, 0]
    elif kind == "norm":
      w = w - _norm_offset(cfg)
    elif kind == "embed":
      w = w / _embed_scale(cfg)
    elif kind == "conv":
      w = w.permute(2, 1, 0)
    elif kind == "patch":
      P = cfg.patch_size_for_vit
      w = w.view(w.shape[0], P, P, -1).permute(0, 3, 1, 2)
    elif kind == "linear_io":
      w = w.t()
    elif key.endswith("position_embedding.weight"):
      w = w.reshape(-1, w.shape[-1])
    out[key] = w.contiguous()
  return out


def hf_config_dict(cfg) -> dict:
  arch = {"llama2": "LlamaForCausalLM", "mistral": "MistralForCausalLM", "mixtral": "MixtralForCausalLM", "qwen2": "Qwen2ForCausalLM",
          "qwen3": "Qwen3ForCausalLM", "gemma": "GemmaForCausalLM", "gemma2": "Gemma2ForCausalLM"}.get(cfg.decoder_block, "LlamaForCausalLM")
  return {"architectures": [arch], "hidden_size": cfg.emb_dim, "intermediate_size": cfg.mlp_dim, "num_hidden_layers": cfg.num_decoder_layers,
          "num_attention_heads": cfg.num_query_heads, "num_key_value_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
          "vocab_size": cfg.vocab_size, "rms_norm_eps": cfg.normalization_layer_epsilon, "rope_theta": float(cfg.rope_max_timescale),
          "max_position_embeddings": cfg.max_target_length, "tie_word_embeddings": bool(cfg.logits_via_embedding), "torch_dtype": "float32",
          "num_local_experts": cfg.num_experts, "num_experts_per_tok": cfg.num_experts_per_tok}


def convert_hf_to_checkpoint(hf_dir: str, config, out_dir: str):
  """`to_maxtext` CLI core: safetensors directory -> params-only checkpoint directory (step 0)."""
  from safetensors.torch import load_file
  from ..checkpoint import manager as ckpt
  from ..train.engine import TrainEngine
  state = {}
  for f in sorted(os.listdir(hf_dir)):
    if f.endswith(".safetensors"):
      state.update(load_file(os.path.join(hf_dir, f)))
  eng = TrainEngine(config, None, torch.device("cpu"), init=False)
  missing = to_maxtext(state, eng.store, config)
  if missing:
    raise KeyError(f"no HF tensor for {missing[:5]} ...")
  mgr = ckpt.CheckpointManager(config, eng, None, directory=out_dir)
  mgr.save(0, force=True)
  return os.path.join(out_dir, "0")


def convert_checkpoint_to_hf(ckpt_step_dir: str, config, out_dir: str):
  """`to_huggingface` CLI core."""
  from safetensors.torch import save_file
  from ..checkpoint import manager as ckpt
  from ..train.engine import TrainEngine
  eng = TrainEngine(config, None, torch.device("cpu"), init=False)
  ckpt.load_params_only(ckpt_step_dir, eng)
  os.makedirs(out_dir, exist_ok=True)
  save_file(to_hf(eng.store, config), os.path.join(out_dir, "model.safetensors"))
  with open(os.path.join(out_dir, "config.json"), "w") as fh:
    json.dump(hf_config_dict(config), fh, indent=1)
  return out_dir
