"""End-to-end train steps on a GPU: tiny Llama in bf16 tracks the fp32 CPU run of the same model."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(extra=()):
  from maxtext_b200.config import pyconfig
  return pyconfig.initialize(
      ["t", "maxtext_b200/configs/base.yml", "base_emb_dim=512", "base_num_query_heads=4", "base_num_kv_heads=2", "head_dim=128",
       "base_mlp_dim=1024", "base_num_decoder_layers=2", "vocab_size=4096", "max_target_length=256", "per_device_batch_size=2",
       "dataset_type=synthetic", "enable_checkpointing=false", "weight_init=normal", "log_config=false", "steps=4",
       "learning_rate=1e-3", "warmup_steps_fraction=0.0", *extra], num_devices=1)


def _losses(cfg, device, steps=4):
  from maxtext_b200.input_pipeline.synthetic import SyntheticDataIterator
  from maxtext_b200.train.engine import TrainEngine
  eng = TrainEngine(cfg, None, torch.device(device))
  it = SyntheticDataIterator(cfg, pin=False)
  return [float(eng.train_step(next(it))["learning/loss"]) for _ in range(steps)]


def test_tiny_llama_gpu_matches_cpu_fp32():
  from maxtext_b200.ops import backend
  E = backend.ext(required=True)
  gpu = _losses(_cfg(["hardware=gpu"]), "cuda")
  assert E.kernel_status(True) == 0
  cpu = _losses(_cfg(["hardware=cpu", "dtype=float32"]), "cpu")
  assert gpu[-1] < gpu[0]
  for a, b in zip(gpu, cpu):
    assert abs(a - b) < 0.08, (gpu, cpu)


def test_graft_smoke():
  import __graft_entry__ as g
  g.smoke()

