"""Qwen3-VL vision tower against the HuggingFace module (same weights, fp32), and the deepstack path into the decoder."""
import math

import pytest
import torch

from helpers import tiny_config

VIT = ["use_multimodal=true", "hidden_size_for_vit=32", "num_attention_heads_for_vit=4", "intermediate_size_for_vit=48", "num_hidden_layers_for_vit=3",
       "patch_size_for_vit=4", "temporal_patch_size_for_vit=2", "spatial_merge_size_for_vit=2", "num_position_embeddings_for_vit=36",
       "deepstack_visual_indexes_for_vit=[0,1]", "image_size_for_vit=16"]


def _load(vision, hf):
  """Copy the HuggingFace weights into the tower's parameters (internal layout [out, in])."""
  sd = {k: v.detach().float() for k, v in hf.state_dict().items()}
  P = {p.name: p for p in vision.params}
  d, h = 32, 4

  def put(name, t):
    assert tuple(P[name].shape) == tuple(t.shape), (name, tuple(P[name].shape), tuple(t.shape))
    P[name].data = t.clone()
  # conv weight [d, C, T, P, P] -> features ordered (t, py, px, c)
  put("vision_encoder/patch_embed/proj/kernel", sd["patch_embed.proj.weight"].permute(0, 2, 3, 4, 1).reshape(d, -1))
  put("vision_encoder/patch_embed/proj/bias", sd["patch_embed.proj.bias"])
  put("vision_encoder/pos_embed_interpolate/pos_embed", sd["pos_embed.weight"])
  for i in range(3):
    pre, hp = f"vision_encoder/blocks_{i}/", f"blocks.{i}."
    for ours, theirs in (("ln1", "norm1"), ("ln2", "norm2")):
      put(pre + ours + "/scale", sd[hp + theirs + ".weight"])
      put(pre + ours + "/bias", sd[hp + theirs + ".bias"])
    qkv_w, qkv_b = sd[hp + "attn.qkv.weight"], sd[hp + "attn.qkv.bias"]
    for j, n in enumerate(("query", "key", "value")):
      put(pre + f"attn/attn/{n}/kernel", qkv_w[j * d:(j + 1) * d])
      put(pre + f"attn/attn/{n}/bias", qkv_b[j * d:(j + 1) * d])
    put(pre + "attn/attn/out/kernel", sd[hp + "attn.proj.weight"])
    put(pre + "attn/attn/out/bias", sd[hp + "attn.proj.bias"])
    put(pre + "mlp/kernel", sd[hp + "mlp.linear_fc1.weight"])
    put(pre + "mlp/bias", sd[hp + "mlp.linear_fc1.bias"])
    put(pre + "mlp_out/kernel", sd[hp + "mlp.linear_fc2.weight"])
    put(pre + "mlp_out/bias", sd[hp + "mlp.linear_fc2.bias"])
  for ours, theirs in (("vision_projector/merger", "merger"), ("vision_encoder/merger_0", "deepstack_merger_list.0"), ("vision_encoder/merger_1", "deepstack_merger_list.1")):
    put(ours + "/ln_q/scale", sd[theirs + ".norm.weight"])
    put(ours + "/ln_q/bias", sd[theirs + ".norm.bias"])
    put(ours + "/mlp_0/kernel", sd[theirs + ".linear_fc1.weight"])
    put(ours + "/mlp_0/bias", sd[theirs + ".linear_fc1.bias"])
    put(ours + "/mlp_2/kernel", sd[theirs + ".linear_fc2.weight"])
    put(ours + "/mlp_2/bias", sd[theirs + ".linear_fc2.bias"])


def test_tower_matches_huggingface():
  tr = pytest.importorskip("transformers")
  from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLVisionConfig, Qwen3VLVisionModel
  from maxtext_b200.models.vision import Qwen3VLVision
  cfg = tiny_config("qwen3-vl-2b", VIT + ["out_hidden_size_for_vit=40"])
  hf_cfg = Qwen3VLVisionConfig(depth=3, hidden_size=32, hidden_act="gelu_pytorch_tanh", intermediate_size=48, num_heads=4, in_channels=3, patch_size=4,
                               spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=cfg.out_hidden_size_for_vit, num_position_embeddings=36,
                               deepstack_visual_indexes=[0, 1])
  hf_cfg._attn_implementation = "eager"
  torch.manual_seed(0)
  hf = Qwen3VLVisionModel(hf_cfg).float().eval()
  for p in hf.parameters():
    torch.nn.init.normal_(p, std=0.2)
  vision = Qwen3VLVision(cfg, {})
  _load(vision, hf)
  H, W = 16, 24                                              # a non-square grid of 4 x 6 patches, 2 x 3 merged tokens
  images = torch.randn(1, 2, 3, H, W)
  with torch.no_grad():
    got = vision(images)
    # HuggingFace input: patches in merge order, features (c, t, py, px), one row of grid_thw per image
    x, rc, gh, gw = vision.patches(images.reshape(2, 3, H, W))
    flat = x.reshape(2 * gh * gw, 2, 4, 4, 3).permute(0, 4, 1, 2, 3).reshape(2 * gh * gw, -1)
    out = hf(flat, grid_thw=torch.tensor([[1, gh, gw], [1, gh, gw]]))
  want = out.pooler_output.view(1, 2, (gh // 2) * (gw // 2), -1)
  assert got.shape == want.shape
  assert torch.allclose(got, want, atol=2e-3, rtol=2e-3), float((got - want).abs().max())
  for a, b in zip(vision.deepstack, out.deepstack_features):
    assert torch.allclose(a.reshape(b.shape), b, atol=2e-3, rtol=2e-3)


def test_deepstack_features_reach_the_decoder_at_image_positions():
  from maxtext_b200.models.transformer import Transformer
  cfg = tiny_config("qwen3-vl-2b", VIT + ["out_hidden_size_for_vit=64"])
  model = Transformer(cfg, None, torch.device("cpu"))
  model.store.initialize(seed=0)
  B, S = 1, 16
  tokens = torch.randint(1, 200, (B, S))
  mask = torch.zeros(B, S, dtype=torch.bool)
  mask[:, 3:7] = True                                          # one 16 x 16 image -> 2 x 2 soft tokens
  images = torch.randn(B, 1, 3, 16, 16)
  with torch.no_grad():
    a = model.forward(tokens, images=images, image_mask=mask)
    deep = [d.clone() for d in model.vision.deepstack]
    assert len(deep) == 2 and deep[0].shape == (1, 1, 4, 64)
    # without deepstack the logits differ: switch the injection off by clearing the list after encoding
    model.vision.deep_idx, model.vision.deep_mergers = [], []
    b = model.forward(tokens, images=images, image_mask=mask)
  assert a.shape == (B, S, cfg.vocab_size) and torch.isfinite(a).all()
  assert not torch.allclose(a, b)
  assert torch.allclose(a[:, :3], b[:, :3], atol=1e-5)         # causal: positions before the image are untouched


def test_processor_resizes_to_the_patch_grid_and_expands_placeholders():
  import numpy as np
  from maxtext_b200.multimodal import processor_qwen3 as pq
  cfg = tiny_config("qwen3-vl-2b", VIT + ["out_hidden_size_for_vit=64"])
  assert pq.smart_resize(100, 37, 8, 4 * 64, 10 ** 9) == (96, 40)
  assert pq.smart_resize(1000, 1000, 8, 256, 64 * 64) == (64, 64)          # capped by max_pixels, still a multiple of 8
  assert pq.smart_resize(3, 5, 8, 4 * 64, 10 ** 9)[0] % 8 == 0
  img = (np.random.default_rng(0).random((30, 45, 3)) * 255).astype(np.uint8)
  tk = pq.special_tokens("qwen3-vl-2b")
  ids, mask, pix = pq.prepare([5, tk["vision_start"], tk["image_pad"], tk["vision_end"], 9], [img], cfg)
  assert pix.shape == (1, 3, 32, 48) and float(pix.min()) >= -1.0 and float(pix.max()) <= 1.0
  K = (32 // 8) * (48 // 8)
  assert int(mask.sum()) == K and ids.tolist()[:2] == [5, tk["vision_start"]] and ids.tolist()[-2:] == [tk["vision_end"], 9]
  assert len(ids) == 2 + K + 2
  ids2, mask2, _ = pq.prepare([5, 9], [img, img], cfg)                      # no placeholder in the prompt: images are appended
  assert int(mask2.sum()) == 2 * K
  assert pq.special_tokens("qwen3.5-35b-a3b")["image_pad"] == 248056


def test_multi_axis_rotary_positions_and_angles_match_huggingface():
  pytest.importorskip("transformers")
  from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLTextConfig
  from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLTextRotaryEmbedding, apply_rotary_pos_emb
  from maxtext_b200.multimodal.processor_qwen3 import rope_index
  from maxtext_b200.ops import reference as ref
  # positions: 3 text tokens, a 2 x 3 image, 2 text tokens
  mask = [False] * 3 + [True] * 6 + [False] * 2
  p3 = rope_index(mask, [(2, 3)])
  assert p3.tolist() == [[0, 0, 0], [1, 1, 1], [2, 2, 2],
                         [3, 3, 3], [3, 3, 4], [3, 3, 5], [3, 4, 3], [3, 4, 4], [3, 4, 5],
                         [6, 6, 6], [7, 7, 7]]
  # angles: against the HuggingFace rotary module with the same sections
  D, sec = 32, [6, 5, 5]
  hf_cfg = Qwen3VLTextConfig(hidden_size=64, num_attention_heads=2, num_key_value_heads=2, head_dim=D, num_hidden_layers=1, intermediate_size=64, vocab_size=64,
                             rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": sec, "mrope_interleaved": True})
  rot = Qwen3VLTextRotaryEmbedding(hf_cfg)
  torch.manual_seed(0)
  x = torch.randn(1, len(mask), 2, D)
  pos_hf = p3.t()[:, None, :]                                              # [3, batch, seq]
  cos, sin = rot(x, pos_hf)
  want, _ = apply_rotary_pos_emb(x.transpose(1, 2), x.transpose(1, 2), cos, sin)
  inv = ref.rope_inv_timescale(D, 1, 10000.0)
  got = ref.apply_mrope(x, p3[None], inv, sec)
  assert torch.allclose(got, want.transpose(1, 2), atol=1e-5)
  # text-only positions reduce to the ordinary embedding
  p = torch.arange(11)[None]
  assert torch.allclose(ref.apply_mrope(x, p[..., None].expand(-1, -1, 3), inv, sec), ref.apply_rope(x, p, inv, False), atol=1e-6)
  # and the model takes them: logits change when the image positions are supplied
  from maxtext_b200.models.transformer import Transformer
  cfg = tiny_config("qwen3-vl-2b", VIT + ["out_hidden_size_for_vit=64", "mrope_section=[4,2,2]"])
  model = Transformer(cfg, None, torch.device("cpu"))
  model.store.initialize(seed=0)
  tokens = torch.randint(1, 200, (1, 11))
  with torch.no_grad():
    a = model.forward(tokens)
    b = model.forward(tokens, positions3=p3[None])
    c = model.forward(tokens, positions3=torch.arange(11)[None, :, None].expand(-1, -1, 3))
  assert torch.allclose(a, c, atol=1e-4) and not torch.allclose(a, b, atol=1e-4)


def test_unfrozen_qwen_tower_gradient_includes_the_deepstack_route():
  """The tower feeds the decoder twice (soft tokens at the embedding, deepstack features after the first layers); the analytic
  directional derivative over the tower's parameters matches the finite difference only if both routes are differentiated."""
  from helpers import batch_of, make_engine
  cfg = tiny_config("qwen3-vl-2b", VIT + ["out_hidden_size_for_vit=64", "freeze_vision_encoder_params=false", "gradient_clipping_threshold=0",
                                          "per_device_batch_size=1", "max_target_length=32"])
  eng = make_engine(cfg)
  store = eng.store
  b = batch_of(cfg)
  B, S = b["inputs"].shape
  mask = torch.zeros(B, S, dtype=torch.bool)
  mask[:, 3:7] = True
  b["images"], b["image_mask"] = torch.randn(B, 1, 3, 16, 16, generator=torch.Generator().manual_seed(0)), mask
  eng.fwd_bwd(dict(b))
  store.finish_resident_grads()
  acc = eng._accum
  eng._accum = None
  g = store.grad_shard.clone() / float(acc["weights"])
  sel = torch.zeros_like(g, dtype=torch.bool)
  for k, u in store.units.items():
    if k.split("#")[0] == "vision":
      sel[u.shard_offset: u.shard_offset + u.numel] = True
  # the deepstack mergers only act through the second route: they must have a gradient
  deep_names = [p.name for p in eng.model.vision_params if "vision_encoder/merger_" in p.name]
  assert deep_names and any(float(p.main_grad.abs().sum()) > 0 for p in eng.model.vision_params if p.name in deep_names)
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


def test_video_temporal_patches_match_huggingface_and_reach_the_decoder():
  pytest.importorskip("transformers")
  import numpy as np
  from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLVisionConfig, Qwen3VLVisionModel
  from maxtext_b200.models.transformer import Transformer
  from maxtext_b200.models.vision import Qwen3VLVision
  from maxtext_b200.multimodal import processor_qwen3 as pq
  cfg = tiny_config("qwen3-vl-2b", VIT + ["out_hidden_size_for_vit=40"])
  hf_cfg = Qwen3VLVisionConfig(depth=3, hidden_size=32, hidden_act="gelu_pytorch_tanh", intermediate_size=48, num_heads=4, in_channels=3, patch_size=4,
                               spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=40, num_position_embeddings=36, deepstack_visual_indexes=[0, 1])
  hf_cfg._attn_implementation = "eager"
  torch.manual_seed(0)
  hf = Qwen3VLVisionModel(hf_cfg).float().eval()
  for p in hf.parameters():
    torch.nn.init.normal_(p, std=0.2)
  vision = Qwen3VLVision(cfg, {})
  _load(vision, hf)
  T, H, W = 4, 16, 24                                           # four frames = two temporal patches
  video = torch.randn(1, T // 2, 2, 3, H, W)                    # [B, patches, frames per patch, 3, H, W]
  with torch.no_grad():
    got = vision(video)
    x, rc, gh, gw = vision.patches(video.reshape(T // 2, 2, 3, H, W))
    flat = x.reshape((T // 2) * gh * gw, 2, 4, 4, 3).permute(0, 4, 1, 2, 3).reshape((T // 2) * gh * gw, -1)     # HF features: (c, t, py, px)
    want = hf(flat, grid_thw=torch.tensor([[T // 2, gh, gw]])).pooler_output.view(1, T // 2, (gh // 2) * (gw // 2), -1)
  assert got.shape == want.shape and torch.allclose(got, want, atol=2e-3, rtol=2e-3), float((got - want).abs().max())
  # frames that differ inside a temporal patch give other tokens than a repeated frame
  with torch.no_grad():
    still = vision(video[:, :, :1].expand(-1, -1, 2, -1, -1, -1).contiguous())
  assert not torch.allclose(still, got)
  # processor: five frames -> three temporal patches (the last frame repeated), prompt expanded per patch
  cfg2 = tiny_config("qwen3-vl-2b", VIT + ["out_hidden_size_for_vit=64"])
  frames = (np.random.default_rng(0).random((5, 16, 16, 3)) * 255).astype(np.uint8)
  tk = pq.special_tokens("qwen3-vl-2b")
  ids, mask, pix = pq.prepare_video([5, tk["video_pad"], 9], frames, cfg2)
  assert pix.shape == (3, 2, 3, 16, 16) and torch.equal(pix[2, 0], pix[2, 1]) and int(mask.sum()) == 3 * 4
  assert ids.tolist()[0] == 5 and ids.tolist()[-1] == 9 and ids.tolist().count(tk["vision_start"]) == 3
  model = Transformer(cfg2, None, torch.device("cpu"))
  model.store.initialize(seed=0)
  with torch.no_grad():
    toks = ids[None] % cfg2.vocab_size
    a = model.forward(toks, images=pix[None], image_mask=mask[None])
    b = model.forward(toks, images=pix[None] * 0.5, image_mask=mask[None])
  assert torch.isfinite(a).all() and not torch.allclose(a, b)


def test_checkpoint_converter_maps_the_vision_tower_both_ways():
  """HuggingFace `model.visual.*` tensors -> the tower's parameters (fused qkv cut in three, 3-D patch convolution flattened) and
  back; the converted tower reproduces the HuggingFace tower's output."""
  pytest.importorskip("transformers")
  from transformers.models.qwen3_vl.modeling_qwen3_vl import Qwen3VLVisionConfig, Qwen3VLVisionModel
  from maxtext_b200.checkpoint_conversion import hf as conv
  from maxtext_b200.models.transformer import Transformer
  cfg = tiny_config("qwen3-vl-2b", VIT + ["out_hidden_size_for_vit=64"])
  hf_cfg = Qwen3VLVisionConfig(depth=3, hidden_size=32, hidden_act="gelu_pytorch_tanh", intermediate_size=48, num_heads=4, in_channels=3, patch_size=4,
                               spatial_merge_size=2, temporal_patch_size=2, out_hidden_size=64, num_position_embeddings=36, deepstack_visual_indexes=[0, 1])
  hf_cfg._attn_implementation = "eager"
  torch.manual_seed(0)
  hf = Qwen3VLVisionModel(hf_cfg).float().eval()
  for p in hf.parameters():
    torch.nn.init.normal_(p, std=0.2)
  state = {"model.visual." + k: v.detach() for k, v in hf.state_dict().items()}
  model = Transformer(cfg, None, torch.device("cpu"))
  model.store.initialize(seed=0)
  missing = conv.to_maxtext(state, model.store, cfg)
  vis = {p.name for p in model.vision_params}
  assert not (vis & set(missing)), sorted(vis & set(missing))[:5]            # every tower tensor found its source (the text side has none here)
  images = torch.randn(1, 1, 3, 16, 24)
  with torch.no_grad():
    got = model.vision(images)
    x, rc, gh, gw = model.vision.patches(images.reshape(1, 3, 16, 24))
    flat = x.reshape(gh * gw, 2, 4, 4, 3).permute(0, 4, 1, 2, 3).reshape(gh * gw, -1)
    want = hf(flat, grid_thw=torch.tensor([[1, gh, gw]])).pooler_output.view(got.shape)
  assert torch.allclose(got, want, atol=2e-3, rtol=2e-3), float((got - want).abs().max())
  back = conv.to_hf(model.store, cfg)
  for k, v in state.items():
    assert k in back and torch.allclose(back[k].reshape(v.shape), v.float(), atol=1e-6), k
