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


def _hf_name(pdef, cfg) -> tuple[str, str] | None:
  """(hf key, kind) for one of our parameters; kind in {linear, norm, embed, q, k, expert:<j>...}."""
  path = "/".join(pdef.ref_path)
  L = pdef.layer
  pre = f"model.layers.{L}." if L is not None else ""
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
      "self_attention/query_norm/scale": (pre + "self_attn.q_norm.weight", "norm"),
      "self_attention/key_norm/scale": (pre + "self_attn.k_norm.weight", "norm"),
      "pre_self_attention_layer_norm/scale": (pre + "input_layernorm.weight", "norm"),
      "post_self_attention_layer_norm/scale": (pre + "post_attention_layernorm.weight", "norm"),
      "pre_self_attention_norm/scale": (pre + "input_layernorm.weight", "norm"),
      "pre_ffw_norm/scale": (pre + ("pre_feedforward_layernorm.weight" if cfg.decoder_block in ("gemma2", "gemma3") else "post_attention_layernorm.weight"), "norm"),
      "post_self_attention_norm/scale": (pre + "post_attention_layernorm.weight", "norm"),
      "post_ffw_norm/scale": (pre + "post_feedforward_layernorm.weight", "norm"),
      "mlp/wi_0/kernel": (pre + "mlp.gate_proj.weight", "linear"),
      "mlp/wi_1/kernel": (pre + "mlp.up_proj.weight", "linear"),
      "mlp/wo/kernel": (pre + "mlp.down_proj.weight", "linear"),
      "MoeBlock_0/gate/kernel": (pre + "block_sparse_moe.gate.weight", "linear"),
      "MoeBlock_0/wi_0": (pre + "block_sparse_moe.experts.{e}.w1.weight", "experts"),
      "MoeBlock_0/wi_1": (pre + "block_sparse_moe.experts.{e}.w3.weight", "experts"),
      "MoeBlock_0/wo": (pre + "block_sparse_moe.experts.{e}.w2.weight", "experts"),
  }
  return table.get(path)


def _norm_offset(cfg) -> float:
  # HF Gemma stores (scale - 1); MaxText stores the effective scale
  return 1.0 if cfg.decoder_block in ("gemma", "gemma2", "gemma3") else 0.0


def _q_scale(cfg) -> float:
  if cfg.use_qk_norm or cfg.decoder_block in ("gemma3",):
    return 1.0
  return 1.0 / math.sqrt(cfg.head_dim)


def _interleaved(cfg) -> bool:
  return cfg.rope_type.startswith("llama3.1") or cfg.model_name.startswith("llama3.1") or cfg.model_name.startswith("llama3.3")


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
    if kind == "experts":
      fused = key.split("block_sparse_moe")[0] + "mlp.experts."
      if key.format(e=0) in hf_state:
        w = torch.stack([hf_state[key.format(e=e)].float() for e in range(cfg.num_experts)])
      elif key.endswith("w2.weight"):                      # newer HF layout: experts stacked, gate|up fused
        w = hf_state[fused + "down_proj"].float()
      else:
        gu = hf_state[fused + "gate_up_proj"].float()
        half = gu.shape[1] // 2
        w = gu[:, :half] if key.endswith("w1.weight") else gu[:, half:]
      store.load_full(name, p.pdef.local_slice(w.contiguous()))
      continue
    if key not in hf_state and "block_sparse_moe.gate" in key:
      key = key.replace("block_sparse_moe.gate", "mlp.gate")
    if key not in hf_state:
      if key == "lm_head.weight" and "model.embed_tokens.weight" in hf_state:
        key = "model.embed_tokens.weight"
      else:
        missing.append(name)
        continue
    w = hf_state[key].float()
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
    if kind == "experts":
      for e in range(w.shape[0]):
        out[key.format(e=e)] = w[e].contiguous()
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
