"""Logit parity with the HuggingFace implementations of every decoder family both sides have.

A randomly initialised tiny HF model is converted with `checkpoint_conversion.hf.to_maxtext` and both models score
the same tokens in fp32; the logits must agree to rounding. This is the CPU analogue of MaxText's golden-logit
check (tests/utils/forward_pass_logit_checker.py) and covers, per family, the attention variant (GQA / MLA / sinks /
sliding and chunked windows / per-head, all-head and scale-free q-k norms / gated delta network with gated full attention), the rotary variant (plain, llama-3.1
and linear scaling, YaRN with attention scaling, adjacent-pair lanes), the router (softmax top-k, sigmoid with
groups and bias, top-1 sigmoid, biased logits) and the expert tensor layouts of the converter.
"""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from helpers import BASE_YML  # noqa: E402
from maxtext_b200.checkpoint_conversion import hf as conv  # noqa: E402
from maxtext_b200.config import pyconfig  # noqa: E402
from maxtext_b200.models.transformer import Transformer  # noqa: E402

V, S = 128, 24


def _tiny(model, extra=()):
  base = {"base_emb_dim": 64, "base_num_query_heads": 4, "base_num_kv_heads": 2, "head_dim": 16, "base_mlp_dim": 128,
          "base_num_decoder_layers": 2, "vocab_size": V, "max_target_length": S, "dtype": "float32", "hardware": "cpu",
          "log_config": "false", "rope_max_timescale": 10000}
  for e in extra:
    k, v = e.split("=", 1)
    base[k] = v
  return pyconfig.initialize(["t", BASE_YML, f"model_name={model}", "override_model_config=true"] + [f"{k}={v}" for k, v in base.items()],
                             num_devices=1)


def _yarn(cfg):
  return {"rope_type": "yarn", "factor": float(cfg.rope_factor), "beta_fast": float(cfg.beta_fast), "beta_slow": float(cfg.beta_slow),
          "truncate": bool(cfg.rope_truncate), "original_max_position_embeddings": int(cfg.original_max_position_embeddings),
          "rope_theta": float(cfg.rope_max_timescale)}


def _common(cfg, **kw):
  d = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
           vocab_size=V, rms_norm_eps=cfg.normalization_layer_epsilon, tie_word_embeddings=False, max_position_embeddings=64)
  d.update(kw)
  return d


def _gemma(_):
  cfg = _tiny("gemma-2b", ["base_num_kv_heads=1"])
  hc = transformers.GemmaConfig(**_common(cfg, num_key_value_heads=1, rope_theta=10000.0, tie_word_embeddings=True,
                                          hidden_activation="gelu_pytorch_tanh"))
  return cfg, transformers.GemmaForCausalLM, hc


def _gemma2(_):
  cfg = _tiny("gemma2-2b", ["sliding_window_size=8"])
  hc = transformers.Gemma2Config(**_common(cfg, num_hidden_layers=4, rope_theta=10000.0, sliding_window=8, query_pre_attn_scalar=16,
                                           attn_logit_softcapping=50.0, final_logit_softcapping=30.0, tie_word_embeddings=True))
  return cfg, transformers.Gemma2ForCausalLM, hc


def _gemma3(_):
  cfg = _tiny("gemma3-4b", ["sliding_window_size=8", "base_num_decoder_layers=6", "local_rope_max_timescale=10000", "rope_max_timescale=1000000"])
  rp = {"sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
        "full_attention": {"rope_type": "linear", "factor": float(cfg.rope_linear_scaling_factor), "rope_theta": 1000000.0}}
  hc = transformers.Gemma3TextConfig(**_common(cfg, num_hidden_layers=6, sliding_window=8, query_pre_attn_scalar=16, tie_word_embeddings=True,
                                               rope_parameters=rp))
  return cfg, transformers.Gemma3ForCausalLM, hc


def _qwen2(_):
  cfg = _tiny("qwen2.5-7b")
  hc = transformers.Qwen2Config(**{k: v for k, v in _common(cfg, rope_theta=10000.0).items() if k != "head_dim"})
  return cfg, transformers.Qwen2ForCausalLM, hc


def _qwen3(_):
  cfg = _tiny("qwen3-8b")
  hc = transformers.Qwen3Config(**_common(cfg, rope_theta=10000.0, attention_bias=False, use_sliding_window=False))
  return cfg, transformers.Qwen3ForCausalLM, hc


def _qwen3_moe(_):
  cfg = _tiny("qwen3-30b-a3b", ["num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=32"])
  hc = transformers.Qwen3MoeConfig(**_common(cfg, moe_intermediate_size=32, num_experts=4, num_experts_per_tok=2, rope_theta=10000.0,
                                             norm_topk_prob=True))
  return cfg, transformers.Qwen3MoeForCausalLM, hc


def _mistral(_):
  cfg = _tiny("mistral-7b", ["sliding_window_size=8"])
  hc = transformers.MistralConfig(**_common(cfg, rope_theta=10000.0, sliding_window=8))
  return cfg, transformers.MistralForCausalLM, hc


def _deepseek3(_):
  cfg = _tiny("deepseek3-tiny", ["num_experts=8", "num_experts_per_tok=2", "base_moe_mlp_dim=32", "base_num_decoder_layers=3", "kv_lora_rank=32",
                                 "q_lora_rank=24", "qk_nope_head_dim=16", "qk_rope_head_dim=8", "v_head_dim=16", "n_routing_groups=4",
                                 "topk_routing_group=2", "first_num_dense_layers=1", "base_num_kv_heads=4", "shared_experts=1"])
  rp = dict(_yarn(cfg), mscale=float(cfg.mscale), mscale_all_dim=float(cfg.mscale))
  rp.pop("truncate")
  hc = transformers.DeepseekV3Config(**{k: v for k, v in _common(
      cfg, moe_intermediate_size=32, n_routed_experts=8, num_experts_per_tok=2, num_hidden_layers=3, num_key_value_heads=4, kv_lora_rank=32,
      q_lora_rank=24, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, n_group=4, topk_group=2, first_k_dense_replace=1,
      n_shared_experts=1, routed_scaling_factor=cfg.routed_scaling_factor, rope_parameters=rp, max_position_embeddings=S).items()
      if k != "head_dim"})
  return cfg, transformers.DeepseekV3ForCausalLM, hc


def _deepseek2(_):
  # HF's DeepSeek-V2 port leaves the YaRN mscale^2 factor out of the softmax scale (its V3 port and MaxText's MLA,
  # src/maxtext/layers/attention_mla.py:890-893, apply it), so the comparison runs with mscale = 0, where the factor is one
  cfg = _tiny("deepseek2-16b", ["num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=32", "base_num_decoder_layers=3", "kv_lora_rank=32",
                                "qk_nope_head_dim=16", "qk_rope_head_dim=8", "v_head_dim=16", "shared_experts=1", "base_num_kv_heads=4",
                                "first_num_dense_layers=1", "mscale=0.0"])
  rp = dict(_yarn(cfg), mscale=0.707, mscale_all_dim=0.707)
  rp.pop("truncate")
  hc = transformers.DeepseekV2Config(**{k: v for k, v in _common(
      cfg, moe_intermediate_size=32, n_routed_experts=4, num_experts_per_tok=2, num_hidden_layers=3, num_key_value_heads=4, kv_lora_rank=32,
      q_lora_rank=None, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, n_group=1, topk_group=1, first_k_dense_replace=1,
      n_shared_experts=1, routed_scaling_factor=cfg.routed_scaling_factor, topk_method="greedy", norm_topk_prob=False, rope_parameters=rp,
      max_position_embeddings=S).items() if k != "head_dim"})
  return cfg, transformers.DeepseekV2ForCausalLM, hc


def _gpt_oss(_):
  cfg = _tiny("gpt-oss-20b", ["num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=32", "sliding_window_size=8"])
  hc = transformers.GptOssConfig(**_common(cfg, intermediate_size=32, num_local_experts=4, num_experts_per_tok=2, sliding_window=8,
                                           rope_parameters=_yarn(cfg), max_position_embeddings=S))
  return cfg, transformers.GptOssForCausalLM, hc


def _olmo3(_):
  cfg = _tiny("olmo3-7b", ["base_num_decoder_layers=4", "sliding_window_size=8"])
  hc = transformers.Olmo3Config(**{k: v for k, v in _common(cfg, num_hidden_layers=4, sliding_window=8, rope_parameters=_yarn(cfg),
                                                            max_position_embeddings=S).items() if k != "head_dim"})
  return cfg, transformers.Olmo3ForCausalLM, hc


def _llama4(_):
  cfg = _tiny("llama4-17b-16e", ["base_num_decoder_layers=4", "num_experts=4", "base_moe_mlp_dim=32", "chunk_attn_window_size=16",
                                 "nope_layer_interval=2", "interleave_moe_layer_step=2"])
  rp = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192,
        "rope_theta": float(cfg.rope_max_timescale)}
  hc = transformers.Llama4TextConfig(**_common(
      cfg, intermediate_size=32, intermediate_size_mlp=128, num_hidden_layers=4, num_local_experts=4, num_experts_per_tok=1,
      interleave_moe_layer_step=2, no_rope_layers=[1, 0, 1, 0], attention_chunk_size=16, use_qk_norm=True, attn_temperature_tuning=True,
      floor_scale=8192, attn_scale=0.1, rope_parameters=rp))
  return cfg, transformers.Llama4ForCausalLM, hc


def _qwen3_next(_):
  cfg = _tiny("qwen3-next-80b-a3b", ["base_num_decoder_layers=4", "num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=32",
                                     "gdn_key_head_dim=8", "gdn_value_head_dim=8", "gdn_num_key_heads=2", "gdn_num_value_heads=4",
                                     "gdn_chunk_size=8"])
  hc = transformers.Qwen3NextConfig(**_common(
      cfg, num_hidden_layers=4, moe_intermediate_size=32, shared_expert_intermediate_size=32, num_experts=4, num_experts_per_tok=2,
      linear_conv_kernel_dim=4, linear_key_head_dim=8, linear_value_head_dim=8, linear_num_key_heads=2, linear_num_value_heads=4,
      rope_parameters={"rope_theta": float(cfg.rope_max_timescale), "partial_rotary_factor": 0.25, "rope_type": "default"}))
  return cfg, transformers.Qwen3NextForCausalLM, hc


def _qwen3_5(_):
  cfg = _tiny("qwen3.5-35b-a3b", ["base_num_decoder_layers=4", "num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=32",
                                  "gdn_key_head_dim=8", "gdn_value_head_dim=8", "gdn_num_key_heads=2", "gdn_num_value_heads=4",
                                  "gdn_chunk_size=8"])
  hc = transformers.Qwen3_5MoeTextConfig(**_common(
      cfg, num_hidden_layers=4, moe_intermediate_size=32, shared_expert_intermediate_size=32, num_experts=4, num_experts_per_tok=2,
      linear_conv_kernel_dim=4, linear_key_head_dim=8, linear_value_head_dim=8, linear_num_key_heads=2, linear_num_value_heads=4,
      rope_parameters={"rope_theta": float(cfg.rope_max_timescale), "partial_rotary_factor": 0.25, "rope_type": "default",
                       "mrope_section": [1, 1, 0], "mrope_interleaved": True}))
  return cfg, transformers.Qwen3_5MoeForCausalLM, hc


CASES = {"qwen3_next": _qwen3_next, "qwen3_5": _qwen3_5, "gemma": _gemma, "gemma2": _gemma2, "gemma3": _gemma3, "qwen2": _qwen2, "qwen3": _qwen3, "qwen3_moe": _qwen3_moe,
         "mistral": _mistral, "deepseek2": _deepseek2, "deepseek3": _deepseek3, "gpt_oss": _gpt_oss, "olmo3": _olmo3, "llama4": _llama4}


def _randomise(hf):
  """HF initialises norms to one, biases and sinks to zero and some stacked expert tensors to nothing in particular:
  give all of them values that a wrong mapping cannot reproduce by accident."""
  g = torch.Generator().manual_seed(1)
  for n, p in hf.named_parameters():
    if "conv1d" in n or "dt_bias" in n:
      p.data = 0.5 + 0.2 * torch.randn(p.shape, generator=g)
    elif "norm" in n:
      p.data = 1.0 + 0.1 * torch.randn(p.shape, generator=g)
    elif "bias" in n or "sinks" in n:
      p.data = 0.1 * torch.randn(p.shape, generator=g)
    elif "experts" in n:
      p.data = 0.06 * torch.randn(p.shape, generator=g)


@pytest.mark.parametrize("family", sorted(CASES))
def test_logits_match_hf(family):
  try:
    cfg, cls, hc = CASES[family](None)
  except (AttributeError, TypeError) as e:       # an older transformers without the family or with other config keys
    pytest.skip(f"transformers cannot build {family}: {e}")
  hc._attn_implementation = "eager"
  torch.manual_seed(0)
  hf = cls(hc).float().eval()
  _randomise(hf)
  model = Transformer(cfg, None, "cpu")
  missing = conv.to_maxtext(hf.state_dict(), model.store, cfg)
  assert not missing, missing
  toks = torch.randint(0, V, (2, S))
  with torch.no_grad():
    want = hf(toks).logits
  got = model.forward(toks)
  err = (got - want).abs().max().item()
  assert err < 2e-5 * max(1.0, want.abs().max().item()), (family, err)
  # and back: the exported state dict reproduces the HF tensors it came from
  back = conv.to_hf(model.store, cfg)
  src = hf.state_dict()
  for k, v in back.items():
    if k in src:
      assert torch.allclose(v, src[k].float(), atol=1e-5), k
