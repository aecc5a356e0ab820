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


def test_tokenizer_trainer_writes_a_loadable_sentencepiece_model(tmp_path):
  """The vocabulary trainer samples a jsonl corpus, trains a small unigram model and the data pipeline can load it."""
  import json
  import pytest
  pytest.importorskip("sentencepiece")
  from maxtext_b200.input_pipeline.tokenizer import build_tokenizer
  from maxtext_b200.trainers.tokenizer import train_tokenizer as tt
  words = ["alpha", "beta", "gamma", "delta", "epsilon", "zeta", "eta", "theta", "iota", "kappa", "lambda", "omega"]
  for j in range(2):
    with open(tmp_path / f"c{j}.jsonl", "w") as fh:
      for i in range(400):
        fh.write(json.dumps({"text": " ".join(words[(i * 7 + k * 3 + j) % len(words)] for k in range(12))}) + "\n")
  assert len(list(tt.example_texts(str(tmp_path / "*.jsonl")))) == 800
  tt.main([f"--train_files={tmp_path}/*.jsonl", "--file_type=jsonl", "--vocab_size=64", "--max_corpus_chars=20000",
           f"--assets_path={tmp_path}/assets", "--vocab_model_name=tok.model"])
  model = tmp_path / "assets" / "tok.model"
  assert model.is_file()
  cfg = tiny_config(extra=["tokenizer_type=sentencepiece", f"tokenizer_path={model}"])
  tok = build_tokenizer(cfg)
  ids = tok.encode("alpha beta omega", add_bos=False, add_eos=True)
  assert ids[-1] == 1 and "alpha" in tok.decode(ids)


def test_layerwise_quantization_matches_whole_model_quantization(tmp_path):
  """Quantising layer by layer from the checkpoint arrays gives the file the serving engine writes when it quantises the
  loaded model at once, and an engine that loads it generates with the de-quantised weights."""
  from safetensors.torch import load_file
  from maxtext_b200.checkpoint import manager as ckpt_lib
  from maxtext_b200.inference.maxengine import MaxEngine
  from maxtext_b200.utils import layerwise_quantization as LQ
  cfg = tiny_config(extra=["steps=1", "checkpoint_period=1", "enable_checkpointing=true", "async_checkpointing=false",
                           f"base_output_directory={tmp_path}", "run_name=lq"])
  eng = make_engine(cfg)
  eng.store.initialize(seed=3)
  ckpt_lib.CheckpointManager(cfg, eng).save_params_only(0)
  src = os.path.join(cfg.checkpoint_dir, "0")
  qcfg = cfg.replace(load_parameters_path=src, save_quantized_params_path=str(tmp_path / "q"), quantization="int8")
  info = LQ.layerwise_quantize(qcfg)
  assert info["layers"] == cfg.num_decoder_layers and info["quantized_bytes"] < info["fp32_bytes"] / 3
  assert info["peak_layer_bytes"] <= info["fp32_bytes"] // cfg.num_decoder_layers + 1
  got = load_file(info["file"])
  whole = MaxEngine(cfg.replace(load_parameters_path=src), device=torch.device("cpu"))
  whole.load_params()
  ref_file = whole.save_quantized_params(str(tmp_path / "ref"), 8)
  want = load_file(ref_file)
  assert set(got) == set(want) and all(torch.equal(got[k], want[k]) for k in want)
  served = MaxEngine(cfg.replace(load_parameters_path=src, checkpoint_is_quantized=True), device=torch.device("cpu"))
  os.replace(info["file"], os.path.join(src, "quantized_params.safetensors"))
  served.load_params()
  name = "layers_0/mlp/wo/kernel"
  assert torch.allclose(served.model.store.full_master(served.model.store.params[name]), whole.model.store.full_master(whole.model.store.params[name]))
