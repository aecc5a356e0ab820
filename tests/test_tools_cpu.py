"""Stand-alone drivers: checkpointer loop, data-loader loop, parameter-only checkpoint, FLOPs report."""
import os

import torch

from helpers import BASE_YML, TINY, make_engine, tiny_config
from maxtext_b200.utils import generate_param_only_checkpoint, get_flops, standalone_checkpointer, standalone_dataloader


def test_standalone_checkpointer_roundtrip(tmp_path):
  cfg = tiny_config(extra=["steps=5", "checkpoint_period=2", "enable_checkpointing=true", "async_checkpointing=false",
                           f"base_output_directory={tmp_path}", "run_name=sc"])
  out = standalone_checkpointer.checkpoint_loop(cfg)
  assert out["saves"] == 3 and out["restored_step"] == 5 and out["save_gb_per_s"] > 0 and out["roundtrip_exact"]
  assert sorted(int(n) for n in os.listdir(cfg.checkpoint_dir) if n.isdigit()) == [0, 2, 4]


def test_standalone_dataloader_counts_tokens():
  cfg = tiny_config(extra=["steps=4"])
  out = standalone_dataloader.data_load_loop(cfg)
  assert out["batches"] == 4 and out["seq_len"] == cfg.max_target_length and out["tokens_per_second"] > 0


def test_param_only_checkpoint_drops_optimizer_and_loads(tmp_path):
  from maxtext_b200.checkpoint import manager as ckpt_lib
  from maxtext_b200.train import train as train_lib
  cfg = tiny_config(extra=["steps=2", "checkpoint_period=1", "enable_checkpointing=true", "async_checkpointing=false",
                           f"base_output_directory={tmp_path}", "run_name=full"])
  eng, _ = train_lib.train_loop(cfg)
  full_step = os.path.join(cfg.checkpoint_dir, "1")
  cfg2 = tiny_config(extra=[f"load_full_state_path={full_step}", f"base_output_directory={tmp_path}", "run_name=po",
                            "enable_checkpointing=true"])
  items = generate_param_only_checkpoint.generate(cfg2)
  names = os.listdir(items)
  assert any(n.startswith("params") for n in names) and not any(n.startswith("opt_state.0.mu") or n.startswith("opt_state.0.nu") for n in names)
  fresh = make_engine(tiny_config())
  ckpt_lib.load_params_only(os.path.dirname(items), fresh)
  assert torch.equal(fresh.store.master, eng.store.master)


def test_get_flops_llama3_8b(capsys):
  out = get_flops.main(["t", BASE_YML, "model_name=llama3-8b", "per_device_batch_size=2", "max_target_length=8192"])
  # 6 * params(non-embedding) * tokens + attention: the number behind the bench's TFLOP/s/device figure
  assert 800 < out["total_tflops_per_device_per_step"] < 900
  assert out["tokens_per_device_per_step"] == 2 * 8192
