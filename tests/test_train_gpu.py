"""End-to-end train steps on a GPU: tiny Llama in bf16 tracks the fp32 CPU run of the same model."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cfg(extra=()):
  from maxtext_b200.config import pyconfig
  base = ["base_emb_dim=512", "base_num_query_heads=4", "base_num_kv_heads=2", "head_dim=128",
          "base_mlp_dim=1024", "base_num_decoder_layers=2", "vocab_size=4096", "max_target_length=256", "per_device_batch_size=2",
          "dataset_type=synthetic", "enable_checkpointing=false", "weight_init=normal", "log_config=false", "steps=4",
          "learning_rate=1e-3", "warmup_steps_fraction=0.0"]
  merged = {}
  for kv in list(base) + list(extra):
    merged[kv.split("=")[0]] = kv          # a later entry replaces an earlier one with the same key
  return pyconfig.initialize(["t", "maxtext_b200/configs/base.yml", *merged.values()], num_devices=1)


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


@pytest.mark.parametrize("model,extra", [
    ("qwen3-next-80b-a3b", ["base_num_decoder_layers=4", "num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=256", "gdn_key_head_dim=64",
                            "gdn_value_head_dim=64", "gdn_num_key_heads=2", "gdn_num_value_heads=4", "gdn_chunk_size=64"]),
    ("gpt-oss-20b", ["num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=256", "sliding_window_size=64"]),
    ("llama4-17b-16e", ["base_num_decoder_layers=4", "num_experts=4", "base_moe_mlp_dim=256", "chunk_attn_window_size=128", "nope_layer_interval=2",
                        "interleave_moe_layer_step=2"]),
    ("olmo3-7b", ["base_num_decoder_layers=4", "sliding_window_size=64"]),
    ("gemma3-4b", ["base_num_decoder_layers=6", "sliding_window_size=64"]),
    ("deepseek4-tiny", ["base_num_decoder_layers=5", "compress_ratios=[0,4,8,8,4]", "first_num_hash_layers=1", "sliding_window_size=64",
                        "qk_rope_head_dim=64", "q_lora_rank=64", "o_groups=2", "o_lora_rank=64", "indexer_head_dim=64", "indexer_n_heads=2",
                        "indexer_topk=8", "num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=256", "base_num_kv_heads=1",
                        "mhc_expansion_rate=2"]),
    ("gemma4-26b", ["base_num_decoder_layers=6", "sliding_window_size=64", "num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=256",
                    "global_head_dim=128", "global_num_kv_heads=1"]),
    ("envy-test", ["base_num_decoder_layers=4", "num_experts=4", "num_experts_per_tok=1", "base_moe_mlp_dim=256"]),
])
def test_newer_families_train_on_gpu_and_track_cpu(model, extra):
  """bf16 on the GPU (this repository's kernels wherever they apply) against fp32 on the CPU for families whose blocks take the
  general attention path: gated delta layers, sinks, chunked / windowed attention, all-head q/k norms, sandwich norms."""
  from maxtext_b200.ops import backend
  E = backend.ext(required=True)
  over = [f"model_name={model}", "override_model_config=true"] + extra
  gpu = _losses(_cfg(over + ["hardware=gpu"]), "cuda", 3)
  assert E.kernel_status(True) == 0
  cpu = _losses(_cfg(over + ["hardware=cpu", "dtype=float32"]), "cpu", 3)
  # top-1 routing (Llama-4) can flip an expert choice between bf16 and fp32, which moves the loss a little more
  # so can the sparse layers' top-k block choice and the routers of the small MoE variants below
  tol = 0.15 if model.startswith(("llama4", "deepseek4", "gemma4", "envy")) else 0.08
  assert all(abs(a - b) < tol for a, b in zip(gpu, cpu)), (gpu, cpu)
  assert gpu[-1] < gpu[0]


def test_batch_split_schedule_on_two_streams_matches_the_plain_step():
  """The micro-batches of a split layer run on two side streams; the losses must follow the unsplit run."""
  from maxtext_b200.ops import backend
  E = backend.ext(required=True)
  plain = _losses(_cfg(["hardware=gpu", "per_device_batch_size=4"]), "cuda")
  split = _losses(_cfg(["hardware=gpu", "per_device_batch_size=4", "use_batch_split_schedule=true"]), "cuda")
  assert E.kernel_status(True) == 0
  for a, b in zip(plain, split):
    assert abs(a - b) < 0.03, (plain, split)
