"""Checkpoint tree layout, exact round trip, resume continuity, params-only load, incomplete-save clean-up."""
import json
import os

import numpy as np
import torch

from helpers import batch_of, make_engine, tiny_config
from maxtext_b200.checkpoint import manager as ckpt
from maxtext_b200.checkpoint import zarr3


def _cfg(tmp, extra=()):
  return tiny_config("llama3-8b", ["enable_checkpointing=true", f"base_output_directory={tmp}", "run_name=r", "async_checkpointing=false",
                                   "checkpoint_period=2", *extra])


def test_zarr3_roundtrip_and_region_reads(tmp_path):
  a = np.arange(5 * 7 * 3, dtype=np.float32).reshape(5, 7, 3)
  zarr3.write_array(str(tmp_path / "a"), a, chunks=(2, 7, 2))
  assert np.array_equal(zarr3.read_array(str(tmp_path / "a")), a)
  assert np.array_equal(zarr3.read_array(str(tmp_path / "a"), (slice(1, 4), slice(0, 7), slice(2, 3))), a[1:4, :, 2:3])
  meta = json.load(open(tmp_path / "a" / "zarr.json"))
  assert meta["zarr_format"] == 3 and meta["shape"] == [5, 7, 3] and meta["data_type"] == "float32"
  zarr3.write_array(str(tmp_path / "s"), np.asarray(7, dtype=np.int32))
  assert int(zarr3.read_array(str(tmp_path / "s"))) == 7


def test_tree_layout_matches_reference_names_and_shapes(tmp_path):
  cfg = _cfg(tmp_path)
  eng = make_engine(cfg)
  eng.train_step(batch_of(cfg))
  mgr = ckpt.CheckpointManager(cfg, eng)
  mgr.save(0, force=True)
  items = os.path.join(cfg.checkpoint_dir, "0", "items")
  assert os.path.isfile(os.path.join(cfg.checkpoint_dir, "0", ckpt.COMMIT))
  def shape(name):
    return zarr3.read_meta(os.path.join(items, name))["shape"]
  L, D, H, KV, Dh, F, V = cfg.num_decoder_layers, cfg.emb_dim, cfg.num_query_heads, cfg.num_kv_heads, cfg.head_dim, cfg.mlp_dim, cfg.vocab_size
  # scanned layout: layer axis stacked at index 1, kernels stored [in..., out...]
  assert shape("params.params.decoder.layers.self_attention.query.kernel") == [D, L, H, Dh]
  assert shape("params.params.decoder.layers.self_attention.key.kernel") == [D, L, KV, Dh]
  assert shape("params.params.decoder.layers.self_attention.out.kernel") == [H, L, Dh, D]
  assert shape("params.params.decoder.layers.mlp.wi_0.kernel") == [D, L, F]
  assert shape("params.params.decoder.layers.mlp.wo.kernel") == [F, L, D]
  assert shape("params.params.decoder.layers.pre_self_attention_layer_norm.scale") == [D, L]
  assert shape("params.params.token_embedder.embedding") == [V, D]
  assert shape("params.params.decoder.logits_dense.kernel") == [D, V]
  assert shape("params.params.decoder.decoder_norm.scale") == [D]
  assert shape("opt_state.0.mu.params.decoder.layers.mlp.wi_0.kernel") == [D, L, F]
  assert int(zarr3.read_array(os.path.join(items, "step"))) == 1     # steps completed, like TrainState.step after step 0
  # the stored query kernel of layer 1 is the transpose of the internal [out, in] matrix
  q = zarr3.read_array(os.path.join(items, "params.params.decoder.layers.self_attention.query.kernel"))
  internal = eng.store.params["layers_1/self_attention/query/kernel"].data
  assert np.allclose(q[:, 1].reshape(D, H * Dh), internal.t().numpy())


def test_exact_roundtrip_and_unscanned_layout(tmp_path):
  for scan in ("true", "false"):
    cfg = _cfg(tmp_path / scan, [f"scan_layers={scan}"])
    eng = make_engine(cfg)
    b = batch_of(cfg)
    eng.train_step(b)
    mgr = ckpt.CheckpointManager(cfg, eng)
    mgr.save(0, force=True)
    if scan == "false":
      assert os.path.isdir(os.path.join(cfg.checkpoint_dir, "0", "items", "params.params.decoder.layers_1.mlp.wo.kernel"))
    eng2 = make_engine(cfg)
    assert not torch.equal(eng2.store.master, eng.store.master)
    mgr2 = ckpt.CheckpointManager(cfg, eng2)
    assert mgr2.restore_if_possible() == 1
    assert torch.equal(eng2.store.master, eng.store.master)
    assert torch.equal(eng2.store.exp_avg, eng.store.exp_avg) and torch.equal(eng2.store.exp_avg_sq, eng.store.exp_avg_sq)
    assert eng2.step_count == eng.step_count
    l1 = float(eng.train_step(b)["learning/loss"])
    l2 = float(eng2.train_step(b)["learning/loss"])
    assert l1 == l2


def test_train_loop_resume_continuity(tmp_path):
  from maxtext_b200.train import train as T
  cfg = _cfg(tmp_path, ["steps=5", f"metrics_file={tmp_path}/m1.jsonl"])
  _, hist = T.train_loop(cfg)
  assert sorted(os.listdir(cfg.checkpoint_dir)) == ["0", "2", "4"]
  # a second run with more steps resumes after the last committed step and continues the curve
  cfg2 = _cfg(tmp_path, ["steps=7", f"metrics_file={tmp_path}/m2.jsonl"])
  _, hist2 = T.train_loop(cfg2)
  assert [h["step"] for h in hist2] == [5, 6]
  assert hist2[0]["learning/loss"] < hist[-1]["learning/loss"] + 0.05
  lines = [json.loads(l) for l in open(f"{tmp_path}/m1.jsonl")]
  assert len(lines) == 5 and "perf/per_device_tokens_per_sec" in lines[0]


def test_params_only_load_and_incomplete_cleanup(tmp_path):
  cfg = _cfg(tmp_path)
  eng = make_engine(cfg)
  eng.train_step(batch_of(cfg))
  mgr = ckpt.CheckpointManager(cfg, eng)
  mgr.save(3, force=True)
  os.makedirs(os.path.join(cfg.checkpoint_dir, "9", "items"))          # a save that died before its commit marker
  mgr_new = ckpt.CheckpointManager(cfg, make_engine(cfg))
  assert mgr_new.all_steps() == [3] and not os.path.exists(os.path.join(cfg.checkpoint_dir, "9"))
  fresh = make_engine(tiny_config("llama3-8b"))
  ckpt.load_params_only(os.path.join(cfg.checkpoint_dir, "3"), fresh)
  assert torch.equal(fresh.store.master, eng.store.master)
  assert fresh.store.exp_avg.abs().sum() == 0


def test_retention(tmp_path):
  cfg = _cfg(tmp_path, ["max_num_checkpoints_to_keep=2", "checkpoint_period=1"])
  eng = make_engine(cfg)
  mgr = ckpt.CheckpointManager(cfg, eng)
  for s in range(4):
    mgr.save(s, force=True)
  assert mgr.all_steps() == [2, 3]


def test_local_tier_restores_newer_step_than_persistent(tmp_path):
  """Persistent saves every 4 steps, local every step: after 'losing' the job at step 5 the restart resumes from the
  local step 5 copy, and the curve continues exactly as an uninterrupted run."""
  import os
  from helpers import tiny_config
  from maxtext_b200.train import train as train_lib
  args = ["checkpoint_period=4", "enable_checkpointing=true", "async_checkpointing=false", f"base_output_directory={tmp_path}",
          "enable_emergency_checkpoint=true", f"local_checkpoint_directory={tmp_path}/local", "local_checkpoint_period=1",
          "save_checkpoint_on_completion=false", "learning_rate_schedule_steps=8"]
  _, ref = train_lib.train_loop(tiny_config(extra=args + ["steps=8", "run_name=ref", f"local_checkpoint_directory={tmp_path}/local_ref"]))
  train_lib.train_loop(tiny_config(extra=args + ["steps=6", "run_name=a"]))
  persistent = sorted(int(n) for n in os.listdir(os.path.join(tmp_path, "a", "checkpoints")) if n.isdigit())
  local = sorted(int(n) for n in os.listdir(os.path.join(tmp_path, "local")) if n.isdigit())
  assert persistent == [0, 4] and local[-1] == 5 and len(local) <= 2
  _, hist = train_lib.train_loop(tiny_config(extra=args + ["steps=8", "run_name=a"]))
  assert [h["step"] for h in hist] == [6, 7]
  assert abs(hist[-1]["learning/loss"] - ref[-1]["learning/loss"]) < 1e-5
