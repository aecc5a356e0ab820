"""Gemma-4 text stack (dense and MoE) against the HuggingFace model with the same weights, fp32."""
import math

import pytest
import torch

from helpers import tiny_config

D, H, HKV, DH, GDH, GKV, F, L, V = 48, 4, 2, 16, 32, 1, 64, 6, 128


def _hf(moe: bool):
  from transformers.models.gemma4.configuration_gemma4 import Gemma4TextConfig
  from transformers.models.gemma4.modeling_gemma4 import Gemma4ForCausalLM
  cfg = Gemma4TextConfig(
      vocab_size=V, hidden_size=D, intermediate_size=F, num_hidden_layers=L, num_attention_heads=H, num_key_value_heads=HKV, head_dim=DH,
      global_head_dim=GDH, num_global_key_value_heads=GKV, attention_k_eq_v=True, sliding_window=8, max_position_embeddings=64,
      layer_types=["sliding_attention"] * 5 + ["full_attention"], hidden_size_per_layer_input=0, vocab_size_per_layer_input=V,
      final_logit_softcapping=30.0, rope_parameters={"sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                                                      "full_attention": {"rope_type": "proportional", "rope_theta": 1000000.0, "partial_rotary_factor": 0.25}},
      enable_moe_block=moe, num_experts=4 if moe else None, top_k_experts=2 if moe else None, moe_intermediate_size=24 if moe else None,
      tie_word_embeddings=True)
  cfg._attn_implementation = "eager"
  torch.manual_seed(0)
  m = Gemma4ForCausalLM(cfg).float().eval()
  with torch.no_grad():
    for n, p in m.named_parameters():
      p.copy_(torch.randn_like(p) * (0.3 if p.dim() > 1 else 0.5) + (1.0 if "norm" in n or "scale" in n else 0.0))
    for n, b in m.named_buffers():
      if n.endswith("layer_scalar"):
        b.copy_(torch.rand(1) + 0.5)
  return m


def _ours(moe: bool):
  extra = ["num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=24", "shared_experts=1", "norm_topk_prob=true", "load_balance_loss_weight=0.0"] if moe \
      else ["num_experts=1"]
  cfg = tiny_config("gemma4-26b", [f"base_emb_dim={D}", f"base_num_query_heads={H}", f"base_num_kv_heads={HKV}", f"head_dim={DH}", f"global_head_dim={GDH}",
                                   f"global_num_kv_heads={GKV}", f"base_mlp_dim={F}", f"base_num_decoder_layers={L}", f"vocab_size={V}", "sliding_window_size=8",
                                   "max_target_length=16", "tokenizer_type=byte", "normalize_embedding_logits=true", "float32_gate_logits=true"] + extra)
  from maxtext_b200.models.transformer import Transformer
  model = Transformer(cfg, None, torch.device("cpu"))
  model.store.initialize(seed=0)
  return cfg, model


def _load(model, hf, moe):
  sd = {k: v.detach().float() for k, v in hf.state_dict().items()}
  st = model.store

  def put(name, t):
    p = st.params[name]
    assert tuple(p.pdef.shape) == tuple(t.shape), (name, tuple(p.pdef.shape), tuple(t.shape))
    st.load_full(name, t.contiguous())
  put("token_embedder/embedding", sd["model.embed_tokens.weight"] * math.sqrt(D))
  put("decoder/decoder_norm/scale", sd["model.norm.weight"])
  for i in range(L):
    a, b = f"layers_{i}/", f"model.layers.{i}."
    put(a + "pre_self_attention_norm/scale", sd[b + "input_layernorm.weight"])
    put(a + "post_self_attention_norm/scale", sd[b + "post_attention_layernorm.weight"])
    put(a + "pre_ffw_norm/scale", sd[b + "pre_feedforward_layernorm.weight"])
    put(a + "post_ffw_norm/scale", sd[b + "post_feedforward_layernorm.weight"])
    put(a + "layer_scalar", sd[b + "layer_scalar"])
    put(a + "self_attention/query/kernel", sd[b + "self_attn.q_proj.weight"])
    put(a + "self_attention/key/kernel", sd[b + "self_attn.k_proj.weight"])
    if i % 6 != 5:
      put(a + "self_attention/value/kernel", sd[b + "self_attn.v_proj.weight"])
    put(a + "self_attention/out/kernel", sd[b + "self_attn.o_proj.weight"])
    put(a + "self_attention/query_norm/scale", sd[b + "self_attn.q_norm.weight"])
    put(a + "self_attention/key_norm/scale", sd[b + "self_attn.k_norm.weight"])
    mlp = a + ("mlp/moe_block/shared_experts/" if moe else "mlp/")
    put(mlp + "wi_0/kernel", sd[b + "mlp.gate_proj.weight"])
    put(mlp + "wi_1/kernel", sd[b + "mlp.up_proj.weight"])
    put(mlp + "wo/kernel", sd[b + "mlp.down_proj.weight"])
    if moe:
      r = a + "mlp/moe_block/MoeBlock_0/"
      put(r + "gate/kernel", sd[b + "router.proj.weight"])
      put(r + "per_expert_scale", sd[b + "router.per_expert_scale"])
      gu = sd[b + "experts.gate_up_proj"]                                   # [E, 2F, D]
      put(r + "wi_0", gu[:, :24])
      put(r + "wi_1", gu[:, 24:])
      put(r + "wo", sd[b + "experts.down_proj"])
      put(a + "mlp/pre_forward_scale_2", sd[b + "router.scale"])
      put(a + "mlp/pre_feedforward_layernorm_2/scale", sd[b + "pre_feedforward_layernorm_2.weight"])
      put(a + "mlp/post_feedforward_layernorm_1/scale", sd[b + "post_feedforward_layernorm_1.weight"])
      put(a + "mlp/post_feedforward_layernorm_2/scale", sd[b + "post_feedforward_layernorm_2.weight"])
  st.sync_compute_from_master()


@pytest.mark.parametrize("moe", [False, True])
def test_logits_match_huggingface(moe):
  pytest.importorskip("transformers")
  hf = _hf(moe)
  cfg, model = _ours(moe)
  _load(model, hf, moe)
  torch.manual_seed(1)
  ids = torch.randint(0, V, (2, 14))                              # longer than the sliding window of 8
  with torch.no_grad():
    want = hf(input_ids=ids).logits.float()
    got = model.forward(ids)
  err = float((got - want).abs().max())
  assert err < 2e-3 * max(1.0, float(want.abs().max())), err


def test_vision_tower_matches_huggingface():
  pytest.importorskip("transformers")
  from transformers.models.gemma4.configuration_gemma4 import Gemma4VisionConfig
  from transformers.models.gemma4.modeling_gemma4 import Gemma4VisionModel
  from maxtext_b200.models.vision import Gemma4Vision
  d, h, f, P, depth = 32, 2, 48, 4, 2
  hf_cfg = Gemma4VisionConfig(hidden_size=d, intermediate_size=f, num_hidden_layers=depth, num_attention_heads=h, num_key_value_heads=h, head_dim=d // h,
                              patch_size=P, position_embedding_size=16, pooling_kernel_size=2, standardize=False, use_clipped_linears=False,
                              rope_parameters={"rope_type": "default", "rope_theta": 100.0}, hidden_activation="gelu_pytorch_tanh", rms_norm_eps=1e-6)
  hf_cfg._attn_implementation = "eager"
  torch.manual_seed(0)
  hf = Gemma4VisionModel(hf_cfg).float().eval()
  with torch.no_grad():
    for n, p in hf.named_parameters():
      p.copy_(torch.randn_like(p) * 0.3 + (1.0 if "norm" in n else 0.0))
  cfg = tiny_config("gemma4-26b", ["use_multimodal=true", f"hidden_size_for_vit={d}", f"num_attention_heads_for_vit={h}", f"intermediate_size_for_vit={f}",
                                   f"num_hidden_layers_for_vit={depth}", f"patch_size_for_vit={P}", "num_position_embeddings_for_vit=16", "rope_theta_for_vit=100",
                                   "vision_output_length=6", "image_size_for_vit=[16,24]", "num_experts=1", "tokenizer_type=byte"])
  tower = Gemma4Vision(cfg, {})
  sd = {k: v.detach().float() for k, v in hf.state_dict().items()}
  Pm = {p.name: p for p in tower.params}

  def put(name, t):
    assert tuple(Pm[name].shape) == tuple(t.shape), (name, tuple(Pm[name].shape), tuple(t.shape))
    Pm[name].data = t.clone()
  put("vision_encoder/entry/input_projection/kernel", sd["patch_embedder.input_proj.weight"])
  put("vision_encoder/entry/pos_emb", sd["patch_embedder.position_embedding_table"])
  for i in range(depth):
    a, b = f"vision_encoder/layers_{i}/", f"encoder.layers.{i}."
    for ours, theirs in (("pre_attention_norm", "input_layernorm"), ("post_attention_norm", "post_attention_layernorm"),
                         ("pre_ffw_norm", "pre_feedforward_layernorm"), ("post_ffw_norm", "post_feedforward_layernorm")):
      put(a + ours + "/scale", sd[b + theirs + ".weight"])
    for ours, theirs in (("query", "q_proj"), ("key", "k_proj"), ("value", "v_proj"), ("out", "o_proj")):
      put(a + f"attention/{ours}/kernel", sd[b + f"self_attn.{theirs}.linear.weight"])
    put(a + "attention/query_norm/scale", sd[b + "self_attn.q_norm.weight"])
    put(a + "attention/key_norm/scale", sd[b + "self_attn.k_norm.weight"])
    for ours, theirs in (("wi_0", "gate_proj"), ("wi_1", "up_proj"), ("wo", "down_proj")):
      put(a + f"mlp/{ours}/kernel", sd[b + f"mlp.{theirs}.linear.weight"])
  Pm["vision_projector/projection/kernel"].data = torch.randn(Pm["vision_projector/projection/kernel"].shape) * 0.1
  H, W = 16, 24                                   # 4 x 6 patches, pooled 2 x 2 -> 6 soft tokens
  images = torch.rand(2, 3, H, W) * 2 - 1         # already in [-1, 1]
  with torch.no_grad():
    gh, gw, xy = tower._grid(H, W, images.device)
    patches = tower.patches(images)
    got = tower.encode(patches, xy, 6)
    # HuggingFace takes pixels in [0, 1] (it applies 2 (x - 0.5) itself) and one (x, y) pair per patch
    want = hf(pixel_values=(patches + 1) / 2, pixel_position_ids=xy[None].expand(2, -1, -1)).last_hidden_state.view(2, 6, d)
    out = tower(images[None])
  assert torch.allclose(got, want, atol=2e-3, rtol=2e-3), float((got - want).abs().max())
  assert out.shape == (1, 2, 6, cfg.emb_dim) and torch.isfinite(out).all()


@pytest.mark.parametrize("moe", [False, True])
def test_checkpoint_converter_covers_the_text_model(moe):
  """`to_maxtext` fills every decoder parameter from the HuggingFace state dict exactly as the hand-written loader of this file
  does, and `to_hf` gives the HuggingFace tensors back."""
  pytest.importorskip("transformers")
  from maxtext_b200.checkpoint_conversion import hf as conv
  hf = _hf(moe)
  _, model_a = _ours(moe)
  _, model_b = _ours(moe)
  _load(model_a, hf, moe)
  missing = conv.to_maxtext(hf.state_dict(), model_b.store, model_b.config)
  assert not missing, missing[:8]
  for name, p in model_a.store.params.items():
    a, b = model_a.store.full_master(p), model_b.store.full_master(model_b.store.params[name])
    assert torch.allclose(a, b, atol=1e-6), name
  back = conv.to_hf(model_b.store, model_b.config)
  sd = hf.state_dict()
  for k, v in sd.items():
    if k in back:
      assert torch.allclose(back[k].reshape(v.shape), v.float(), atol=1e-5), k
  assert {"model.embed_tokens.weight", "model.layers.0.layer_scalar", "model.layers.0.self_attn.q_proj.weight"} <= set(back)
  if moe:
    assert "model.layers.0.experts.gate_up_proj" in back and "model.layers.0.router.scale" in back
