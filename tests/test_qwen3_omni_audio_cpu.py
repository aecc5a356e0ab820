"""Qwen3-Omni audio tower against the HuggingFace encoder with the same weights (fp32)."""
import pytest
import torch

from helpers import tiny_config


def test_audio_tower_matches_huggingface():
  pytest.importorskip("transformers")
  from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeAudioEncoderConfig
  from transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe import Qwen3OmniMoeAudioEncoder
  from maxtext_b200.models.audio import Qwen3OmniAudio, conv_output_length
  d, h, f, layers, mel, ch, out = 32, 2, 48, 2, 16, 8, 24
  hf_cfg = Qwen3OmniMoeAudioEncoderConfig(num_mel_bins=mel, encoder_layers=layers, encoder_attention_heads=h, encoder_ffn_dim=f, d_model=d,
                                          activation_function="gelu", scale_embedding=False, max_source_positions=64, n_window=50, output_dim=out,
                                          n_window_infer=200, conv_chunksize=4, downsample_hidden_size=ch)
  hf_cfg._attn_implementation = "eager"
  torch.manual_seed(0)
  hf = Qwen3OmniMoeAudioEncoder(hf_cfg).float().eval()
  with torch.no_grad():
    for n, p in hf.named_parameters():
      p.copy_(torch.randn_like(p) * 0.2 + (1.0 if ("norm" in n or "ln_post" in n) and n.endswith("weight") else 0.0))
  cfg = tiny_config("qwen3-omni-30b-a3b", [f"d_model_for_audio={d}", f"encoder_attention_heads_for_audio={h}", f"encoder_ffn_dim_for_audio={f}",
                                            f"encoder_layers_for_audio={layers}", f"num_mel_bins_for_audio={mel}", f"downsample_hidden_size_for_audio={ch}",
                                            f"output_dim_for_audio={out}", "n_window_for_audio=50", "n_window_infer_for_audio=200", "max_source_positions_for_audio=64",
                                            "num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=32", "tokenizer_type=byte"])
  tower = Qwen3OmniAudio(cfg, {})
  sd = {k: v.detach().float() for k, v in hf.state_dict().items()}
  P = {p.name: p for p in tower.params}

  def put(name, t):
    assert tuple(P[name].shape) == tuple(t.shape), (name, tuple(P[name].shape), tuple(t.shape))
    P[name].data = t.clone()
  for n in ("conv2d1", "conv2d2", "conv2d3"):
    put(f"audio_encoder/{n}/kernel", sd[f"{n}.weight"])
    put(f"audio_encoder/{n}/bias", sd[f"{n}.bias"])
  put("audio_encoder/conv_out/kernel", sd["conv_out.weight"])
  for i in range(layers):
    a, b = f"audio_encoder/layers_{i}/", f"layers.{i}."
    for ours, theirs in (("self_attn_layer_norm", "self_attn_layer_norm"), ("final_layer_norm", "final_layer_norm")):
      put(a + ours + "/scale", sd[b + theirs + ".weight"])
      put(a + ours + "/bias", sd[b + theirs + ".bias"])
    for ours, theirs in (("query", "q_proj"), ("key", "k_proj"), ("value", "v_proj"), ("out", "out_proj")):
      put(a + f"self_attn/{ours}/kernel", sd[b + f"self_attn.{theirs}.weight"])
      put(a + f"self_attn/{ours}/bias", sd[b + f"self_attn.{theirs}.bias"])
    for n in ("fc1", "fc2"):
      put(a + f"{n}/kernel", sd[b + f"{n}.weight"])
      put(a + f"{n}/bias", sd[b + f"{n}.bias"])
  put("audio_encoder/ln_post/scale", sd["ln_post.weight"])
  put("audio_encoder/ln_post/bias", sd["ln_post.bias"])
  for ours, theirs in (("proj1", "proj1"), ("proj2", "proj2")):
    put(f"audio_projector/{ours}/kernel", sd[f"{theirs}.weight"])
    put(f"audio_projector/{ours}/bias", sd[f"{theirs}.bias"])
  frames = 350                                     # three full chunks of 100 frames and one of 50: two attention windows
  feats = torch.randn(mel, frames)
  # the eager path of the HuggingFace encoder hands its layers the window boundaries only (its flash path applies them), so
  # give every layer the block-diagonal mask that the encoder's own helper builds from those boundaries
  def with_mask(module, args, kwargs):
    x, cu = (args + (kwargs.get("cu_seqlens"),))[:2] if len(args) < 2 else args[:2]
    kwargs["attention_mask"] = hf._prepare_attention_mask(x, cu)
    return args, kwargs
  for layer in hf.layers:
    layer.register_forward_pre_hook(with_mask, with_kwargs=True)
  with torch.no_grad():
    got = tower(feats)
    want = hf(feats, feature_lens=torch.tensor([frames])).last_hidden_state
  assert got.shape == want.shape == (sum(conv_output_length(v) for v in (100, 100, 100, 50)), out)
  assert torch.allclose(got, want, atol=2e-3, rtol=2e-3), float((got - want).abs().max())


AUDIO = ["d_model_for_audio=32", "encoder_attention_heads_for_audio=2", "encoder_ffn_dim_for_audio=48", "encoder_layers_for_audio=1",
         "num_mel_bins_for_audio=16", "downsample_hidden_size_for_audio=8", "max_source_positions_for_audio=64", "use_multimodal=true", "use_audio=true"]


def _omni(extra=()):
  base = tiny_config("qwen3-omni-30b-a3b", [])
  return tiny_config("qwen3-omni-30b-a3b", AUDIO + [f"output_dim_for_audio={base.emb_dim}", "hidden_size_for_vit=32", "intermediate_size_for_vit=48",
                                                    "num_attention_heads_for_vit=2", "num_hidden_layers_for_vit=2", "deepstack_visual_indexes_for_vit=[0]",
                                                    f"out_hidden_size_for_vit={base.emb_dim}", "num_position_embeddings_for_vit=16", "patch_size_for_vit=8",
                                                    "image_size_for_vit=16"] + list(extra))


def test_audio_soft_tokens_enter_the_decoder_at_their_positions():
  from maxtext_b200.models.audio import conv_output_length
  from maxtext_b200.models.transformer import Transformer
  cfg = _omni()
  model = Transformer(cfg, None, torch.device("cpu"))
  model.store.initialize(seed=0)
  assert model.audio is not None and all(p.pdef.frozen for p in model.audio_params)
  B, S, frames = 2, 24, 150
  K = conv_output_length(frames)                               # 13 + 7
  tokens = torch.randint(1, 200, (B, S))
  mask = torch.zeros(B, S, dtype=torch.bool)
  mask[:, 2:2 + K] = True
  audio = torch.randn(B, 16, frames)
  with torch.no_grad():
    soft, m = model.encode_audio(audio, mask)
    assert soft.shape == (B, K, cfg.emb_dim)
    x = model.embed(tokens, torch.arange(S)[None].expand(B, S), (soft, m))
    assert torch.allclose(x[:, 2:2 + K].float(), soft.float(), atol=1e-6)
    a = model.forward(tokens, audio=audio, audio_mask=mask)
    b = model.forward(tokens, audio=audio * 2.0, audio_mask=mask)
    t = model.forward(tokens)
  assert torch.isfinite(a).all() and not torch.allclose(a, t) and not torch.allclose(a, b)
  assert torch.allclose(a[:, :2], t[:, :2], atol=1e-5)         # causal: nothing before the clip changes


def test_engine_trains_on_a_batch_with_audio():
  from maxtext_b200.train.engine import TrainEngine
  cfg = _omni(["per_device_batch_size=2", "max_target_length=32", "steps=2", "learning_rate=1e-3"])
  eng = TrainEngine(cfg, None, torch.device("cpu"))
  S = 32
  g = torch.Generator().manual_seed(0)
  tokens = torch.randint(1, 200, (2, S + 1), generator=g)
  mask = torch.zeros(2, S, dtype=torch.bool)
  mask[:, 1:14] = True
  batch = {"inputs": tokens[:, :-1], "targets": tokens[:, 1:], "audio": torch.randn(2, 16, 100, generator=g), "audio_mask": mask}
  before = [p.data.clone() for p in eng.model.audio_params]
  l0 = float(eng.train_step(dict(batch))["learning/loss"])
  l1 = float(eng.train_step(dict(batch))["learning/loss"])
  assert l0 == l0 and l1 < l0
  assert all(torch.equal(a, p.data) for a, p in zip(before, eng.model.audio_params))          # the tower is frozen


def test_log_mel_features_match_the_whisper_front_end():
  pytest.importorskip("transformers")
  import numpy as np
  from transformers import WhisperFeatureExtractor
  from maxtext_b200.multimodal.audio_features import log_mel, mel_filters, prepare_audio
  rng = np.random.default_rng(0)
  t = np.arange(32000) / 16000.0
  wave = (0.3 * np.sin(2 * np.pi * 440 * t) + 0.1 * np.sin(2 * np.pi * 3000 * t) + 0.02 * rng.standard_normal(t.shape)).astype(np.float32)
  fe = WhisperFeatureExtractor(feature_size=128, sampling_rate=16000, hop_length=160, chunk_length=2, n_fft=400)
  want = fe(wave, sampling_rate=16000, return_tensors="np", padding="max_length").input_features[0]       # [128, 200]
  got = log_mel(wave).numpy()
  assert got.shape == want.shape == (128, 200)
  assert np.abs(got - want).max() < 2e-3, np.abs(got - want).max()
  f = mel_filters()
  assert f.shape == (201, 128) and float(f.min()) >= 0.0 and bool((f.sum(0) > 0).all())
  feats, tokens = prepare_audio(wave[:20000])                     # 1.25 s -> padded to 2 s
  assert feats.shape == (128, 200) and tokens == 26


def test_decode_cli_takes_an_audio_clip(tmp_path):
  """A 16 kHz .wav goes through the feature extractor, the prompt grows by the clip's soft tokens, the engine prefills with them."""
  import wave
  import numpy as np
  from maxtext_b200.inference.decode import decode
  from maxtext_b200.inference.maxengine import MaxEngine
  from maxtext_b200.multimodal import processor_qwen3 as pq
  path = str(tmp_path / "clip.wav")
  sig = (0.4 * np.sin(2 * np.pi * 330 * np.arange(16000) / 16000.0) * 32767).astype("<i2")
  with wave.open(path, "wb") as fh:
    fh.setnchannels(1)
    fh.setsampwidth(2)
    fh.setframerate(16000)
    fh.writeframes(sig.tobytes())
  w, sr = pq.read_wav(path)
  assert sr == 16000 and w.shape == (16000,) and abs(float(np.abs(w).max()) - 0.4) < 1e-3
  cfg = _omni(["num_mel_bins_for_audio=128", "max_prefill_predict_length=48", "max_target_length=56", "per_device_batch_size=1", f"audio_path={path}",
               "prompt=what is this"])
  ids, mask, feats = pq.prepare_audio_prompt([1, 2, 3], w, cfg)
  tk = pq.special_tokens(cfg.model_name)
  assert feats.shape == (128, 100) and int(mask.sum()) == 13 and ids.tolist()[3] == tk["audio_start"] and ids.tolist()[-1] == tk["audio_end"]
  ids2, mask2, _ = pq.prepare_audio_prompt([1, tk["audio_start"], tk["audio_pad"], tk["audio_end"], 9], w, cfg)
  assert ids2.tolist()[0] == 1 and ids2.tolist()[-1] == 9 and int(mask2.sum()) == 13 and len(ids2) == 2 + 15
  eng = MaxEngine(cfg, device="cpu")
  eng.load_params()
  with_audio = decode(cfg, engine=eng)
  silent = tmp_path / "silent.wav"
  with wave.open(str(silent), "wb") as fh:
    fh.setnchannels(1)
    fh.setsampwidth(2)
    fh.setframerate(16000)
    fh.writeframes((sig * 0).tobytes())
  other = decode(cfg.replace(audio_path=str(silent)), engine=eng)
  assert isinstance(with_audio, str) and isinstance(other, str)


def test_checkpoint_converter_maps_the_audio_tower_both_ways():
  pytest.importorskip("transformers")
  from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeAudioEncoderConfig
  from transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe import Qwen3OmniMoeAudioEncoder
  from maxtext_b200.checkpoint_conversion import hf as conv
  from maxtext_b200.models.transformer import Transformer
  cfg = _omni(["n_window_for_audio=50", "n_window_infer_for_audio=200"])
  hf_cfg = Qwen3OmniMoeAudioEncoderConfig(num_mel_bins=16, encoder_layers=1, encoder_attention_heads=2, encoder_ffn_dim=48, d_model=32,
                                          activation_function="gelu", scale_embedding=False, max_source_positions=64, n_window=50,
                                          output_dim=cfg.emb_dim, n_window_infer=200, conv_chunksize=4, downsample_hidden_size=8)
  hf_cfg._attn_implementation = "eager"
  torch.manual_seed(0)
  hf = Qwen3OmniMoeAudioEncoder(hf_cfg).float().eval()
  with torch.no_grad():
    for p in hf.parameters():
      p.copy_(torch.randn_like(p) * 0.2)
  state = {"thinker.audio_tower." + k: v.detach() for k, v in hf.state_dict().items() if "positional_embedding" not in k}
  model = Transformer(cfg, None, torch.device("cpu"))
  model.store.initialize(seed=0)
  missing = set(conv.to_maxtext(state, model.store, cfg))
  assert not ({p.name for p in model.audio_params} & missing), sorted({p.name for p in model.audio_params} & missing)[:5]
  feats = torch.randn(16, 100)
  with torch.no_grad():
    got = model.audio(feats)
    want = hf(feats, feature_lens=torch.tensor([100])).last_hidden_state          # one window: no mask needed on the HF side
  assert torch.allclose(got, want, atol=2e-3, rtol=2e-3), float((got - want).abs().max())
  back = conv.to_hf(model.store, cfg)
  for k, v in state.items():
    assert k in back and torch.allclose(back[k].reshape(v.shape), v.float(), atol=1e-6), k
