"""Multimodal (Gemma-3): vision tower + projector + embedding merge + bidirectional image blocks against HuggingFace,
preprocessing, training through the engine, and prefill + decode with an image in the prompt."""
import numpy as np
import pytest
import torch

from helpers import tiny_config, make_engine, batch_of
from maxtext_b200 import multimodal as mm

MM = ["sliding_window_size=8", "base_num_decoder_layers=6", "use_multimodal=true", "hidden_size_for_vit=32", "intermediate_size_for_vit=64",
      "num_hidden_layers_for_vit=2", "num_attention_heads_for_vit=4", "patch_size_for_vit=4", "conv_stride_for_vit=4",
      "local_rope_max_timescale=10000", "rope_max_timescale=1000000", "vocab_size=128"]


def test_merge_and_masks_and_placeholders():
  text = torch.zeros(2, 6, 3)
  soft = torch.arange(2 * 4 * 3, dtype=torch.float32).view(2, 1, 4, 3)
  mask = torch.tensor([[0, 1, 1, 0, 1, 1], [1, 1, 0, 0, 0, 0]]).bool()
  out = mm.merge_mm_embeddings(text, soft, mask)
  assert torch.equal(out[0, [1, 2, 4, 5]], soft[0, 0]) and torch.equal(out[1, :2], soft[1, 0, :2]) and float(out[0, 0].abs().sum()) == 0
  with pytest.raises(ValueError):
    mm.merge_mm_embeddings(text, soft[:, :, :1], mask)
  b = mm.bidirectional_block_mask(mask)[:, 0]
  assert b[0, 1, 2] and b[0, 2, 1] and not b[0, 2, 4] and b[0, 4, 5] and not b[0, 0, 0] and not b[1, 2, 3]
  assert mm.expand_image_placeholders([1, 9, 2], 9, 7, 3, 5, 6) == [1, 5, 7, 7, 7, 6, 2]


def test_preprocess_images(tmp_path):
  from PIL import Image
  rng = np.random.default_rng(0)
  arr = rng.integers(0, 255, (40, 60, 3), dtype=np.uint8)
  p = str(tmp_path / "a.png")
  Image.fromarray(arr).save(p)
  out = mm.preprocess_images([p, arr], 32)
  assert out.shape == (2, 3, 32, 32) and torch.allclose(out[0], out[1]) and float(out.min()) >= -1.0 and float(out.max()) <= 1.0
  same = mm.preprocess_images([np.full((32, 32, 3), 255, dtype=np.uint8)], 32)
  assert torch.allclose(same, torch.ones_like(same))


def test_gemma3_multimodal_logits_match_hf():
  transformers = pytest.importorskip("transformers")
  from maxtext_b200.checkpoint_conversion import hf as conv
  cfg = tiny_config("gemma3-4b", MM + ["image_size_for_vit=128", "max_target_length=300", "weight_init=normal"])
  vc = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=128, patch_size=4, num_channels=3,
            layer_norm_eps=cfg.normalization_layer_epsilon)
  tc = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=6, num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=128,
            sliding_window=8, query_pre_attn_scalar=16, rms_norm_eps=cfg.normalization_layer_epsilon,
            rope_parameters={"sliding_attention": {"rope_type": "default", "rope_theta": 10000.0},
                             "full_attention": {"rope_type": "linear", "factor": 8.0, "rope_theta": 1000000.0}})
  try:
    hc = transformers.Gemma3Config(text_config=tc, vision_config=vc, mm_tokens_per_image=256, image_token_index=100, boi_token_index=101,
                                   eoi_token_index=102)
  except TypeError as e:
    pytest.skip(str(e))
  for c_ in (hc, hc.text_config, hc.vision_config):
    c_._attn_implementation = "eager"
  torch.manual_seed(0)
  hf = transformers.Gemma3ForConditionalGeneration(hc).float().eval()
  proj = hf.model.multi_modal_projector
  proj.mm_input_projection_weight.data.normal_(0, 0.1)          # HF starts the projector at zero, which would hide the tower
  proj.mm_soft_emb_norm.weight.data.normal_(0, 0.2)
  eng = make_engine(cfg)
  assert not conv.to_maxtext(hf.state_dict(), eng.store, cfg)
  toks = torch.randint(0, 100, (2, 280))
  toks[:, 5], toks[:, 6:262], toks[:, 262] = 101, 100, 102
  imgs = torch.randn(2, 1, 3, 128, 128)          # 32 x 32 patches, pooled 2 x 2 to the 256 soft tokens
  with torch.no_grad():
    want = hf(input_ids=toks, pixel_values=imgs[:, 0], token_type_ids=(toks == 100).long(), attention_mask=torch.ones_like(toks)).logits
  got = eng.model.forward(toks, images=imgs, image_mask=toks == 100)
  assert (got - want).abs().max() < 2e-5, (got - want).abs().max()
  # the image matters, and the text-only path of the same model is unchanged by the tower's presence
  assert (eng.model.forward(toks, images=imgs * 0, image_mask=toks == 100) - got).abs().max() > 1e-3


def test_multimodal_training_and_generation():
  cfg = tiny_config("gemma3-4b", MM + ["image_size_for_vit=64", "max_target_length=288", "per_device_batch_size=1"])
  eng = make_engine(cfg)
  vis_before = {p.name: eng.store.full_master(p).clone() for p in eng.model.vision_params}
  b = batch_of(cfg)
  B, S = b["inputs"].shape
  mask = torch.zeros(B, S, dtype=torch.bool)
  mask[:, 4:260] = True
  b["images"], b["image_mask"] = torch.randn(B, 1, 3, 64, 64), mask
  losses = [float(eng.train_step(b)["learning/loss"]) for _ in range(4)]
  assert losses[-1] < losses[0], losses
  assert all(torch.equal(vis_before[p.name], eng.store.full_master(p)) for p in eng.model.vision_params)     # frozen tower
  # prefill with the image, then decode: the cached path reproduces the full forward
  from maxtext_b200.inference.maxengine import MaxEngine
  me = MaxEngine(cfg, model=eng.model)
  prompt = b["inputs"][0, :270].long()
  prefix, _ = me.prefill(prompt, 270, images=b["images"][0], image_mask=mask[0])
  full = eng.model.forward(prompt[None], images=b["images"][:1], image_mask=mask[:1, :270])[:, -1]
  assert (prefix.logits - full).abs().max() < 1e-4


def test_llama4_multimodal_logits_match_hf():
  transformers = pytest.importorskip("transformers")
  from maxtext_b200.checkpoint_conversion import hf as conv
  cfg = tiny_config("llama4-17b-16e", [
      "base_num_decoder_layers=4", "num_experts=4", "base_moe_mlp_dim=32", "chunk_attn_window_size=16", "nope_layer_interval=2",
      "interleave_moe_layer_step=2", "use_multimodal=true", "hidden_size_for_vit=32", "intermediate_size_for_vit=128",
      "num_hidden_layers_for_vit=2", "num_attention_heads_for_vit=4", "image_size_for_vit=32", "tile_size_for_vit=32", "patch_size_for_vit=4",
      "projector_input_dim_for_vit=48", "projector_output_dim_for_vit=48", "vision_output_dim_for_vit=48", "pixel_shuffle_ratio_for_vit=0.5",
      "rope_theta_for_vit=10000", "vocab_size=128", "max_target_length=64", "rope_max_timescale=10000", "weight_init=normal"])
  vc = dict(hidden_size=32, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, image_size=32, patch_size=4, num_channels=3,
            projector_input_dim=48, projector_output_dim=48, vision_output_dim=48, pixel_shuffle_ratio=0.5, projector_dropout=0.0,
            rope_parameters={"rope_type": "default", "rope_theta": 10000.0})
  tc = dict(hidden_size=64, intermediate_size=32, intermediate_size_mlp=128, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
            head_dim=16, vocab_size=128, num_local_experts=4, num_experts_per_tok=1, interleave_moe_layer_step=2, no_rope_layers=[1, 0, 1, 0],
            attention_chunk_size=16, use_qk_norm=True, attn_temperature_tuning=True, floor_scale=8192, attn_scale=0.1,
            rms_norm_eps=cfg.normalization_layer_epsilon, tie_word_embeddings=False, max_position_embeddings=64,
            rope_parameters={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                             "original_max_position_embeddings": 8192, "rope_theta": 10000.0})
  try:
    hc = transformers.Llama4Config(text_config=tc, vision_config=vc, image_token_index=100, boi_token_index=101, eoi_token_index=102)
  except TypeError as e:
    pytest.skip(str(e))
  for c_ in (hc, hc.text_config, hc.vision_config):
    c_._attn_implementation = "eager"
  torch.manual_seed(0)
  hf = transformers.Llama4ForConditionalGeneration(hc).float().eval()
  g = torch.Generator().manual_seed(5)
  for n, p in hf.named_parameters():
    if n.startswith(("vision_model", "multi_modal_projector")) or "experts" in n:
      p.data = 0.15 * torch.randn(p.shape, generator=g) + (1.0 if ("norm" in n and n.endswith("weight")) else 0.0)
  eng = make_engine(cfg)
  assert not conv.to_maxtext(hf.state_dict(), eng.store, cfg)
  toks = torch.randint(0, 100, (1, 48))
  toks[0, 3], toks[0, 4:20], toks[0, 20], toks[0, 21:37], toks[0, 37] = 101, 100, 100, 100, 102      # two tiles of 16 soft tokens
  mask = torch.zeros(1, 48, dtype=torch.bool)
  mask[0, 4:20] = mask[0, 21:37] = True
  toks[0, 20] = 7
  tiles = torch.randn(2, 3, 32, 32)
  ids = toks.clone()
  ids[mask] = 100
  with torch.no_grad():
    want = hf(input_ids=ids, pixel_values=tiles, attention_mask=torch.ones_like(ids)).logits
  got = eng.model.forward(torch.where(mask, torch.zeros_like(toks), toks), images=tiles[None], image_mask=mask)
  assert (got - want).abs().max() < 5e-5 * max(1.0, float(want.abs().max())), (got - want).abs().max()
  assert (eng.model.forward(torch.where(mask, torch.zeros_like(toks), toks), images=tiles[None] * 0, image_mask=mask) - got).abs().max() > 1e-3


def test_llama4_processor_tiles_and_tokens():
  from maxtext_b200.multimodal import processor_llama4 as pl
  assert pl.best_grid(336, 336) == (1, 1) and pl.best_grid(336, 700) == (1, 2) and pl.best_grid(1000, 340) == (3, 1)
  assert pl.tokens_per_tile() == 144 and max(h * w for h, w in pl.supported_grids()) == 16
  rng = np.random.default_rng(0)
  tiles, grid = pl.preprocess_image(rng.integers(0, 255, (60, 130, 3), dtype=np.uint8), tile=32, max_tiles=4)
  assert grid == (2, 4) or grid[0] * grid[1] <= 4
  assert tiles.shape[1:] == (3, 32, 32) and tiles.shape[0] == grid[0] * grid[1] + (1 if grid[0] * grid[1] > 1 else 0)
  seq = pl.image_tokens((2, 2), 4)
  assert len(seq) == 27 and seq[0] == pl.BEGIN_IMAGE_TOKEN and seq[-1] == pl.END_IMAGE_TOKEN and seq.count(pl.PATCH_TOKEN) == 20
  assert seq.count(pl.TILE_X_SEPARATOR_TOKEN) == 2 and seq.count(pl.TILE_Y_SEPARATOR_TOKEN) == 2 and seq[-6] == pl.IMAGE_TOKEN
  ids, mask, pix = pl.prepare([5, pl.IMAGE_TOKEN, 6], [rng.integers(0, 255, (32, 64, 3), dtype=np.uint8)], tile=32, patch=4, max_tiles=4)
  assert pix.shape[0] == 3 and int(mask.sum()) == 3 * pl.tokens_per_tile(32, 4) and ids[0] == 5 and ids[-1] == 6


def test_unfrozen_tower_trains_and_its_gradient_matches_a_finite_difference():
  """freeze_vision_encoder_params=false: the vision parameters move, and the analytic directional derivative along a random
  direction in the tower's parameters equals the finite difference of the loss."""
  cfg = tiny_config("gemma3-4b", MM + ["image_size_for_vit=64", "max_target_length=288", "per_device_batch_size=1", "freeze_vision_encoder_params=false",
                                      "gradient_clipping_threshold=0"])
  eng = make_engine(cfg)
  store = eng.store
  assert not any(p.pdef.frozen for p in eng.model.vision_params)
  b = batch_of(cfg)
  B, S = b["inputs"].shape
  mask = torch.zeros(B, S, dtype=torch.bool)
  mask[:, 4:260] = True
  b["images"], b["image_mask"] = torch.randn(B, 1, 3, 64, 64, generator=torch.Generator().manual_seed(0)), mask
  eng.fwd_bwd(dict(b))
  store.finish_resident_grads()
  acc = eng._accum
  eng._accum = None
  g = store.grad_shard.clone() / float(acc["weights"])
  sel = torch.zeros_like(g, dtype=torch.bool)                  # the tower's part of the flat parameter vector
  for k, u in store.units.items():
    if k.split("#")[0] == "vision":
      sel[u.shard_offset: u.shard_offset + u.numel] = True
  assert float(g[sel].abs().sum()) > 0
  v = torch.randn(g.shape, generator=torch.Generator().manual_seed(1)) * sel
  v = v / v.norm()

  def loss():
    m = eng.eval_step(dict(b))
    return float(m["evaluation/total_loss"]) / float(m["evaluation/total_weights"])
  w0, eps = store.master.clone(), 1e-2
  vals = []
  for sign in (1.0, -1.0):
    store.master.copy_(w0 + sign * eps * v)
    store.sync_compute_from_master()
    vals.append(loss())
  store.master.copy_(w0)
  store.sync_compute_from_master()
  fd, an = (vals[0] - vals[1]) / (2 * eps), float((g * v).sum())
  assert abs(fd - an) <= 0.05 * max(abs(fd), abs(an)) + 1e-4, (fd, an)
  before = {p.name: store.full_master(p).clone() for p in eng.model.vision_params}
  losses = [float(eng.train_step(dict(b))["learning/loss"]) for _ in range(3)]
  assert losses[-1] < losses[0]
  assert any(not torch.equal(before[p.name], store.full_master(p)) for p in eng.model.vision_params)
