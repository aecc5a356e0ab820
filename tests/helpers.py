"""Shared helpers for CPU tests: tiny configurations of every model family."""
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE_YML = os.path.join(ROOT, "maxtext_b200", "configs", "base.yml")

TINY = ["override_model_config=true", "base_emb_dim=64", "base_num_query_heads=4", "base_num_kv_heads=2", "head_dim=16",
        "base_mlp_dim=128", "base_num_decoder_layers=2", "vocab_size=256", "max_target_length=32", "per_device_batch_size=2",
        "dataset_type=synthetic", "dtype=float32", "hardware=cpu", "enable_checkpointing=false", "log_config=false", "steps=3",
        "learning_rate=1e-3", "warmup_steps_fraction=0.0", "enable_data_shuffling=false"]

FAMILIES = {
    "llama3-8b": [],
    "mistral-7b": ["sliding_window_size=8"],
    "mixtral-8x7b": ["num_experts=4", "base_moe_mlp_dim=64", "load_balance_loss_weight=0.01"],
    "deepseek2-16b": ["num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=32", "base_num_decoder_layers=3", "kv_lora_rank=32",
                      "qk_nope_head_dim=16", "qk_rope_head_dim=8", "v_head_dim=16", "shared_experts=1"],
    "deepseek3-tiny": ["num_experts=8", "num_experts_per_tok=2", "base_moe_mlp_dim=32", "base_num_decoder_layers=3", "kv_lora_rank=32",
                       "q_lora_rank=24", "qk_nope_head_dim=16", "qk_rope_head_dim=8", "v_head_dim=16", "n_routing_groups=4",
                       "topk_routing_group=2", "first_num_dense_layers=1"],
    "gemma-2b": [],
    "gemma2-2b": ["sliding_window_size=8"],
    "gemma3-4b": ["sliding_window_size=8", "base_num_decoder_layers=6"],
    "qwen3-8b": [],
    "qwen2.5-7b": [],
    "qwen3-30b-a3b": ["num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=32"],
    "gpt3-6b": ["trainable_position_size=32"],
    "olmo3-7b": ["base_num_decoder_layers=4", "sliding_window_size=8"],
    "llama4-17b-16e": ["base_num_decoder_layers=4", "num_experts=4", "base_moe_mlp_dim=32", "chunk_attn_window_size=16", "nope_layer_interval=2"],
    "qwen3-next-80b-a3b": ["base_num_decoder_layers=4", "num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=32", "gdn_key_head_dim=8",
                           "gdn_value_head_dim=8", "gdn_num_key_heads=2", "gdn_num_value_heads=4", "gdn_chunk_size=8"],
    "qwen3.5-35b-a3b": ["base_num_decoder_layers=4", "num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=32", "gdn_key_head_dim=8",
                        "gdn_value_head_dim=8", "gdn_num_key_heads=2", "gdn_num_value_heads=4", "gdn_chunk_size=8"],
    "gemma4-26b": ["base_num_decoder_layers=6", "sliding_window_size=8", "global_head_dim=32", "global_num_kv_heads=1", "num_experts=4",
                   "num_experts_per_tok=2", "base_moe_mlp_dim=32", "shared_experts=1", "tokenizer_type=byte"],
    "deepseek4-tiny": ["base_num_decoder_layers=5", "compress_ratios=[0,4,8,8,4]", "first_num_hash_layers=1", "tokenizer_type=byte",
                       "sliding_window_size=8", "qk_rope_head_dim=8", "indexer_head_dim=16", "indexer_topk=2"],
    "envy-test": ["num_experts=4", "num_experts_per_tok=1", "base_moe_mlp_dim=32", "base_num_decoder_layers=4", "tokenizer_type=byte"],
    "gpt-oss-20b": ["base_num_decoder_layers=2", "num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=32", "sliding_window_size=8"],
}


def tiny_config(model="llama3-8b", extra=(), num_devices=1):
  from maxtext_b200.config import pyconfig
  merged = {}
  for e in list(FAMILIES.get(model, [])) + list(extra):
    merged[e.split("=")[0]] = e        # later entries win
  over = list(merged.values())
  keys = set(merged)
  args = [b for b in TINY if b.split("=")[0] not in keys] + ([f"model_name={model}"] if model else []) + over
  return pyconfig.initialize(["t", BASE_YML] + args, num_devices=num_devices)


def make_engine(cfg):
  from maxtext_b200.train.engine import TrainEngine
  return TrainEngine(cfg, None, torch.device("cpu"))


def batch_of(cfg):
  from maxtext_b200.input_pipeline.synthetic import SyntheticDataIterator
  return next(SyntheticDataIterator(cfg, pin=False))
