"""LoRA fine-tuning: adapters start as a no-op, only adapters train, merging reproduces the adapted model, and the
PEFT file format round-trips (src/maxtext/utils/lora_utils.py; `lora:` block of configs/post_train/sft.yml)."""
import torch

from helpers import tiny_config, make_engine, batch_of
from maxtext_b200.utils import lora_utils

LORA = ["lora={enable_lora: true, lora_rank: 4, lora_alpha: 8.0}", "weight_init=normal"]


def _copy_base(dst, src):
  for n, p in src.store.params.items():
    dst.store.load_full(n, src.store.full_master(p))
  dst.store.sync_compute_from_master()


def test_adapters_start_as_identity_and_only_adapters_train():
  base = make_engine(tiny_config("llama3-8b", ["weight_init=normal"]))
  eng = make_engine(tiny_config("llama3-8b", LORA))
  _copy_base(eng, base)
  batch = batch_of(base.config)
  toks = batch["inputs"].long()
  assert torch.equal(base.model.forward(toks), eng.model.forward(toks))          # B = 0
  before = {n: eng.store.full_master(p).clone() for n, p in eng.store.params.items()}
  losses = [float(eng.train_step(batch)["learning/loss"]) for _ in range(6)]
  assert losses[-1] < losses[0], losses
  changed = {n for n, p in eng.store.params.items() if not torch.equal(before[n], eng.store.full_master(p))}
  assert changed and all(n.endswith(("_lora_a", "_lora_b")) for n in changed), sorted(changed)[:5]
  assert any(n.endswith("_lora_a") for n in changed) and any(n.endswith("_lora_b") for n in changed)


def test_lora_gradient_matches_finite_difference():
  torch.manual_seed(0)
  eng = make_engine(tiny_config("llama3-8b", LORA + ["gradient_clipping_threshold=0"]))
  store = eng.store
  for _, a, b, _ in lora_utils.adapted(store):         # move off B = 0 so that A has a gradient too
    store.load_full(b.name, 0.05 * torch.randn(b.pdef.global_shape()))
  store.sync_compute_from_master()
  batch = batch_of(eng.config)
  eng.fwd_bwd(batch)
  store.finish_resident_grads()
  acc, eng._accum = eng._accum, None
  g = store.grad_shard.clone() / float(acc["weights"])
  mask = torch.zeros_like(g, dtype=torch.bool)
  for a, b in store.trainable_slices():
    mask[a:b] = True
  assert float(g[~mask].abs().max()) == 0.0               # frozen parameters get exactly zero
  v = torch.randn_like(g) * mask
  v = v / v.norm()
  from test_engine_cpu import _loss
  w0, eps = store.master.clone(), 1e-2
  store.master.copy_(w0 + eps * v); store.sync_compute_from_master(); lp = _loss(eng, batch)
  store.master.copy_(w0 - eps * v); store.sync_compute_from_master(); lm = _loss(eng, batch)
  fd, an = (lp - lm) / (2 * eps), float((g * v).sum())
  assert abs(fd - an) <= 0.05 * max(abs(fd), abs(an)) + 2e-4, (fd, an)


def test_merge_reproduces_adapted_model_and_peft_files_round_trip(tmp_path):
  torch.manual_seed(1)
  cfg = tiny_config("llama3-8b", LORA)
  eng = make_engine(cfg)
  for _, a, b, _ in lora_utils.adapted(eng.store):
    eng.store.load_full(b.name, 0.05 * torch.randn(b.pdef.global_shape()))
  eng.store.sync_compute_from_master()
  toks = batch_of(cfg)["inputs"].long()
  want = eng.model.forward(toks)
  # a plain model that loads the merged weights
  plain = make_engine(tiny_config("llama3-8b", ["weight_init=normal"]))
  merged = lora_utils.merged_base_state(eng.store)
  for n, p in plain.store.params.items():
    plain.store.load_full(n, merged.get(n, eng.store.full_master(eng.store.params[n])))
  plain.store.sync_compute_from_master()
  assert (plain.model.forward(toks) - want).abs().max() < 1e-4
  # in-place merge, then un-merge
  w_name = lora_utils.adapted(eng.store)[0][0].name
  w0 = eng.store.full_master(eng.store.params[w_name]).clone()
  lora_utils.merge(eng.store)
  assert not torch.equal(w0, eng.store.full_master(eng.store.params[w_name]))
  lora_utils.unmerge(eng.store)
  assert (w0 - eng.store.full_master(eng.store.params[w_name])).abs().max() < 1e-6
  # PEFT directory
  d = lora_utils.save_adapter(str(tmp_path / "adapter"), eng.store, cfg)
  other = make_engine(cfg)
  _copy_base(other, eng)
  for _, a, b, _ in lora_utils.adapted(other.store):
    other.store.load_full(a.name, torch.zeros(a.pdef.global_shape()))
    other.store.load_full(b.name, torch.zeros(b.pdef.global_shape()))
  acfg = lora_utils.load_adapter(d, other.store, cfg)
  assert acfg["r"] == 4 and abs(acfg["lora_alpha"] - 8.0) < 1e-6 and "q_proj" in acfg["target_modules"]
  assert (other.model.forward(toks) - want).abs().max() < 1e-5


def test_peft_adapter_matches_hf_model_with_the_same_delta():
  transformers = __import__("pytest").importorskip("transformers")
  from maxtext_b200.checkpoint_conversion import hf as conv
  cfg = tiny_config("llama3-8b", LORA + ["vocab_size=128", "rope_type=default"])
  hc = transformers.LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                head_dim=16, vocab_size=128, rms_norm_eps=cfg.normalization_layer_epsilon, rope_theta=float(cfg.rope_max_timescale),
                                tie_word_embeddings=False)
  torch.manual_seed(0)
  hf = transformers.LlamaForCausalLM(hc).float().eval()
  eng = make_engine(cfg)
  miss = conv.to_maxtext(hf.state_dict(), eng.store, cfg)
  assert all(n.endswith(("_lora_a", "_lora_b")) for n in miss), miss
  # a PEFT-style adapter on q_proj and down_proj of every layer, applied to the HF weights by hand
  peft, scale = {}, 8.0 / 4
  sd = hf.state_dict()
  for l in range(2):
    for mod in ("self_attn.q_proj", "self_attn.k_proj", "mlp.down_proj"):
      W = sd[f"model.layers.{l}.{mod}.weight"]
      A, B = 0.1 * torch.randn(4, W.shape[1]), 0.1 * torch.randn(W.shape[0], 4)
      peft[f"base_model.model.model.layers.{l}.{mod}.lora_A.weight"], peft[f"base_model.model.model.layers.{l}.{mod}.lora_B.weight"] = A, B
      W.add_(scale * B @ A)
  missing = lora_utils.from_peft(peft, eng.store, cfg)
  assert missing and all(("value" in n or "out" in n or "wi_" in n) for n in missing), missing
  toks = torch.randint(0, 128, (2, 16))
  with torch.no_grad():
    want = hf(toks).logits
  assert (eng.model.forward(toks) - want).abs().max() < 3e-4


def test_cli_lora_run_from_base_checkpoint_writes_peft_adapter(tmp_path):
  import os
  from helpers import TINY, BASE_YML
  from maxtext_b200.train import train as T
  out = str(tmp_path)
  base = [a for a in TINY if not a.startswith(("enable_checkpointing", "steps"))] + ["model_name=llama3-8b", f"base_output_directory={out}"]
  T.main(["train", BASE_YML] + base + ["steps=2", "enable_checkpointing=true", "checkpoint_period=1", "run_name=base", "async_checkpointing=false"])
  ck = os.path.join(out, "base", "checkpoints", "1")
  _, hist = T.main(["train", BASE_YML] + base + ["steps=3", "enable_checkpointing=false", "run_name=lora", f"load_parameters_path={ck}",
                                                 "lora={enable_lora: true, lora_rank: 4, lora_alpha: 8.0}"])
  assert hist[-1]["learning/loss"] < hist[0]["learning/loss"]
  d = os.path.join(out, "lora", "lora_adapter")
  assert sorted(os.listdir(d)) == ["adapter_config.json", "adapter_model.safetensors"]
  # a third run continues from the adapter
  _, hist2 = T.main(["train", BASE_YML] + base + ["steps=1", "enable_checkpointing=false", "run_name=lora2", f"load_parameters_path={ck}",
                                                  "lora={enable_lora: true, lora_rank: 4, lora_alpha: 8.0, lora_restore_path: " + d + "}"])
  assert hist2[0]["learning/loss"] < hist[0]["learning/loss"]


def test_trainable_parameters_mask_and_adamw_mask():
  """`trainable_parameters_mask`: only matching parameters change. `adamw_mask`: matching parameters get no weight decay
  (with a zero learning-rate-independent check: under pure decay, lr > 0 and zero gradients they must stay put)."""
  cfg = tiny_config("llama3-8b", ["trainable_parameters_mask=['.*mlp/wo.*','decoder_norm']"])
  eng = make_engine(cfg)
  before = {n: eng.store.full_master(p).clone() for n, p in eng.store.params.items()}
  b = batch_of(cfg)
  for _ in range(3):
    eng.train_step(b)
  changed = {n for n, p in eng.store.params.items() if not torch.equal(before[n], eng.store.full_master(p))}
  assert changed == {n for n in before if "mlp/wo" in n or "decoder_norm" in n}, sorted(changed)
  # decay mask: zero gradients (all-padding batch has zero loss weight), so the update is decay only
  cfg2 = tiny_config("llama3-8b", ["adamw_mask=['.*norm.*','.*embedding.*']", "adam_weight_decay=0.5", "learning_rate=0.1"])
  eng2 = make_engine(cfg2)
  before = {n: eng2.store.full_master(p).clone() for n, p in eng2.store.params.items()}
  b2 = dict(batch_of(cfg2))
  b2["targets_segmentation"] = torch.zeros_like(b2["targets"])
  eng2.train_step(b2)
  for n, p in eng2.store.params.items():
    same = torch.equal(before[n], eng2.store.full_master(p))
    assert same == ("norm" in n or "embedding" in n), n


def test_nf4_codes_round_trip_and_error_is_bounded():
  from maxtext_b200.utils import nf4
  torch.manual_seed(0)
  w = torch.randn(24, 128) * 0.05
  codes, absmax = nf4.quantize(w, 64)
  assert codes.dtype == torch.uint8 and int(codes.max()) <= 15 and absmax.shape == (48,)
  assert torch.equal(nf4.unpack(nf4.pack(codes)), codes) and nf4.pack(codes).numel() == w.numel() // 2
  back = nf4.dequantize(codes, absmax, w.shape, 64)
  # every value lands on its nearest level: the error is at most half the widest gap (0.16 of the tile's maximum)
  assert float(((back - w).abs() / absmax.repeat_interleave(64).view_as(w)).max()) <= 0.17
  assert torch.equal(nf4.snap(back, 64), back)                    # the grid is a fixed point
  # the extreme of every tile is kept exactly
  t = w.view(-1, 64)
  big = t.abs().argmax(1)
  assert torch.allclose(back.view(-1, 64).gather(1, big[:, None]), t.gather(1, big[:, None]))
  import pytest
  with pytest.raises(ValueError):
    nf4.quantize(torch.randn(4, 100), 64)


def test_qlora_rounds_only_the_adapted_base_weights_and_still_trains():
  from maxtext_b200.utils import nf4
  q = ["lora={enable_lora: true, lora_rank: 4, lora_alpha: 8.0, lora_weight_qtype: nf4, lora_tile_size: 32}", "weight_init=normal"]
  eng = make_engine(tiny_config("llama3-8b", q))
  before = {n: eng.store.full_master(p).clone() for n, p in eng.store.params.items()}
  n = nf4.snap_store(eng.store, eng.config)
  adapted = {p.name for p, _, _, _ in lora_utils.adapted(eng.store)}
  assert n == len(adapted) > 0
  for name, p in eng.store.params.items():
    now = eng.store.full_master(p)
    if name in adapted:
      assert not torch.equal(now, before[name]) and torch.equal(nf4.snap(now.float(), 32).view_as(now), now.float())
      assert len(torch.unique((now.float().view(-1, 32) / now.float().view(-1, 32).abs().amax(1, keepdim=True)).round(decimals=4))) <= 16
    else:
      assert torch.equal(now, before[name])
  batch = batch_of(eng.config)
  losses = [float(eng.train_step(batch)["learning/loss"]) for _ in range(5)]
  assert losses[-1] < losses[0]
  assert nf4.snap_store(eng.store, tiny_config("llama3-8b", LORA)) == 0          # plain LoRA leaves the base alone
