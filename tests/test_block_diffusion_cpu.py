"""Block-diffusion training: corruption, target alignment, attention pattern, the engine's loss and the data wrapper."""
import numpy as np
import pytest
import torch

from helpers import tiny_config
from maxtext_b200.diffusion.block_diffusion import align_to_targets, corrupt_tokens, same_block_mask, source_indices


def test_every_eligible_block_is_supervised_and_padding_is_untouched():
  rng = np.random.default_rng(0)
  tokens = rng.integers(5, 100, size=(6, 37))
  valid = np.ones_like(tokens, dtype=bool)
  valid[0, 20:] = False
  valid[1, :] = False
  r = corrupt_tokens(tokens, valid, np.random.default_rng(1), block_size=8, mask_id=3, min_noise=1e-3)
  assert r.inputs.shape == tokens.shape and (r.inputs[r.corruption_mask] == 3).all()
  assert (r.inputs[~r.corruption_mask] == tokens[~r.corruption_mask]).all()
  assert not r.corruption_mask[~valid].any() and (r.corruption_mask == r.targets_loss_mask).all()
  for row in range(6):
    for b0 in range(0, 37, 8):
      if valid[row, b0:b0 + 8].any():
        assert r.corruption_mask[row, b0:b0 + 8].any(), (row, b0)
  # noise level 1 masks everything that is eligible
  full = corrupt_tokens(tokens, valid, np.random.default_rng(2), block_size=8, mask_id=3, min_noise=1.0)
  assert (full.corruption_mask == valid).all()


def test_seed_and_mask_keeps_block_starts_clean_and_supervises_them():
  tokens = np.arange(1, 33).reshape(1, 32)
  valid = np.ones_like(tokens, dtype=bool)
  r = corrupt_tokens(tokens, valid, np.random.default_rng(0), block_size=8, mask_id=0, min_noise=1.0, logit_alignment="shifted",
                     canvas_policy="seed_and_mask")
  starts = np.arange(32) % 8 == 0
  assert not r.corruption_mask[0, starts].any() and r.corruption_mask[0, ~starts].all()
  assert not r.targets_loss_mask[0, 0] and r.targets_loss_mask[0, 8] and r.targets_loss_mask[0, 1:].all()
  with pytest.raises(ValueError):
    corrupt_tokens(tokens, valid, np.random.default_rng(0), block_size=8, mask_id=0, logit_alignment="shifted", canvas_policy="all_masked")
  with pytest.raises(ValueError):
    corrupt_tokens(tokens, valid, np.random.default_rng(0), block_size=8, mask_id=-1)
  # another sequence axis
  t3 = np.stack([tokens[0], tokens[0]], 1)                        # [32, 2]
  r3 = corrupt_tokens(t3, np.ones_like(t3, dtype=bool), np.random.default_rng(0), block_size=8, mask_id=0, min_noise=1.0, axis=0)
  assert r3.corruption_mask.all()


def test_shifted_alignment_follows_positions():
  x = torch.arange(2 * 6 * 3, dtype=torch.float32).view(2, 6, 3)
  assert align_to_targets(x, "same_position") is x
  y = align_to_targets(x, "shifted")
  assert torch.equal(y[:, 1:], x[:, :-1]) and torch.equal(y[:, 0], x[:, 0])
  # a row whose slots are out of position order: slot 0 holds position 2, slot 1 position 0, slot 2 position 1
  pos = torch.tensor([[2, 0, 1, 3, 4, 5], [0, 1, 2, 3, 4, 5]])
  idx = source_indices("shifted", 6, pos, torch.ones(2, 6, dtype=torch.bool))
  assert idx[0].tolist() == [2, 1, 1, 0, 3, 4] and idx[1].tolist() == [0, 0, 1, 2, 3, 4]
  with pytest.raises(ValueError):
    source_indices("diagonal", 6)


def test_attention_pattern_is_block_causal():
  pos = torch.arange(8)[None]
  m = same_block_mask(pos, 4) | (pos[:, None, :, None] >= pos[:, None, None, :])
  want = (pos[0][:, None] // 4) >= (pos[0][None, :] // 4)
  assert torch.equal(m[0, 0], want)
  seg = torch.tensor([[1, 1, 1, 2, 2, 2, 0, 0]])
  ms = same_block_mask(pos, 4, seg)
  assert not ms[0, 0, 2, 3] and ms[0, 0, 0, 2] and not ms[0, 0, 6, 7]


BD = ["attention_type=block_diffusion", "training_objective=block_diffusion", "causal_block_size=4", "block_diffusion_mask_id=3",
      "per_device_batch_size=2", "max_target_length=16", "learning_rate=3e-3", "packing=false"]


def _batch(cfg, shifted=False):
  from maxtext_b200.diffusion.block_diffusion.batches import BlockDiffusionIterator
  g = torch.Generator().manual_seed(0)
  clean = torch.randint(5, 200, (2, 16), generator=g, dtype=torch.int32)
  inner = iter([{"inputs": clean, "targets": clean.roll(-1, 1), "inputs_segmentation": torch.ones(2, 16, dtype=torch.int32),
                 "inputs_position": torch.arange(16, dtype=torch.int32)[None].expand(2, 16)}] * 4)
  return clean, BlockDiffusionIterator(cfg, inner)


@pytest.mark.parametrize("alignment", ["same_position", "shifted"])
def test_engine_trains_on_block_diffusion_batches(alignment):
  from maxtext_b200.train.engine import TrainEngine
  extra = ["block_diffusion_logit_alignment=shifted", "block_diffusion_canvas_policy=seed_and_mask"] if alignment == "shifted" else []
  cfg = tiny_config("llama2-7b", BD + extra)
  eng = TrainEngine(cfg, None, torch.device("cpu"))
  clean, it = _batch(cfg)
  b = next(it)
  assert torch.equal(b["targets"], clean) and (b["inputs"][b["corruption_mask"].bool()] == 3).all()
  losses = [float(eng.train_step(dict(b))["learning/loss"]) for _ in range(6)]
  assert losses[-1] < losses[0]
  # the loss counts the supervised slots only
  m = eng.eval_step(dict(b))
  assert float(m["evaluation/total_weights"]) == float(b["targets_loss_mask"].sum())
  # the model's own forward uses the same attention pattern: a later token of the active block changes an earlier one's logits
  with torch.no_grad():
    a = eng.model.forward(b["inputs"].long())
    t2 = b["inputs"].clone().long()
    t2[:, 3] = (t2[:, 3] + 1) % 200
    c2 = eng.model.forward(t2)
  assert not torch.allclose(a[:, 0], c2[:, 0]) and torch.allclose(a[:, 8:] * 0, c2[:, 8:] * 0)
  assert torch.allclose(a[:, :3] * 0 + 1, c2[:, :3] * 0 + 1)


def test_loss_matches_a_plain_reference():
  from maxtext_b200.train.engine import TrainEngine
  cfg = tiny_config("llama2-7b", BD + ["block_diffusion_logit_alignment=shifted", "block_diffusion_canvas_policy=seed_and_mask"])
  eng = TrainEngine(cfg, None, torch.device("cpu"))
  _, it = _batch(cfg)
  b = next(it)
  m = eng.eval_step(dict(b))
  with torch.no_grad():
    logits = eng.model.forward(b["inputs"].long(), positions=b["inputs_position"].long(), segment_ids=b["inputs_segmentation"])
  al = align_to_targets(logits, "shifted", b["inputs_position"], b["targets_segmentation"] != 0)
  w = (b["targets_loss_mask"] != 0).float()
  xent = torch.nn.functional.cross_entropy(al.reshape(-1, al.shape[-1]).float(), b["targets"].reshape(-1).long(), reduction="none")
  want = float((xent * w.reshape(-1)).sum())
  assert abs(float(m["evaluation/total_loss"]) - want) < 1e-2 * max(1.0, want), (float(m["evaluation/total_loss"]), want)


def test_rejected_combinations():
  from maxtext_b200.config.validators import ConfigValueError
  with pytest.raises((ConfigValueError, ValueError)):
    tiny_config("llama2-7b", ["training_objective=block_diffusion"])
  with pytest.raises((ConfigValueError, ValueError)):
    tiny_config("llama2-7b", BD + ["block_diffusion_logit_alignment=shifted"])


def test_iterator_wrapper_resumes_with_the_same_masks():
  cfg = tiny_config("llama2-7b", BD)
  _, a = _batch(cfg)
  first = [next(a) for _ in range(3)]
  _, b = _batch(cfg)
  next(b)
  st = b.state()
  _, c = _batch(cfg)
  c.load_state({"draws": st["draws"]})
  again = next(c)
  assert torch.equal(again["corruption_mask"], first[1]["corruption_mask"])
  assert not torch.equal(first[0]["corruption_mask"], first[1]["corruption_mask"])


def test_training_loop_runs_the_objective_on_synthetic_data(tmp_path):
  from maxtext_b200.train import train as train_mod
  cfg = tiny_config("llama2-7b", BD + ["steps=3", "dataset_type=synthetic", f"base_output_directory={tmp_path}", "run_name=bd", "enable_checkpointing=false",
                                      "hardware=cpu"])
  eng = train_mod.train_loop(cfg)
  assert eng is not None
