"""Configuration loader: defaults, YAML chain, model catalog, CLI / env overrides, derived values, validation."""
import glob
import os

import pytest

from helpers import BASE_YML, ROOT
from maxtext_b200.config import pyconfig
from maxtext_b200.config.pyconfig import ConfigError


def init(*args, n=1, **kw):
  return pyconfig.initialize(["t", BASE_YML, "log_config=false", *args], num_devices=n, **kw)


def test_every_model_catalog_entry_parses():
  files = sorted(glob.glob(os.path.join(ROOT, "maxtext_b200", "configs", "models", "*.yml")))
  assert len(files) >= 70
  for f in files:
    c = init(f"model_name={os.path.basename(f)[:-4]}")
    assert c.emb_dim > 0 and c.num_decoder_layers > 0


def test_every_shipped_recipe_parses():
  for sub, n in (("gpu", 8), ("post_train", 8), ("inference", 8)):
    for f in sorted(glob.glob(os.path.join(ROOT, "maxtext_b200", "configs", sub, "*.yml"))):
      if "lora_module_path" in f or f.endswith("vllm.yml") or "gpt_oss_20b" in f:
        continue   # not a run config / fixed 1-device mesh / 128-device recipe
      pyconfig.initialize(["t", f, "log_config=false"], num_devices=n)


def test_headline_configuration_derived_values():
  c = init("model_name=llama3-8b", "per_device_batch_size=2", "max_target_length=8192", "dataset_type=synthetic", n=8)
  assert (c.emb_dim, c.num_query_heads, c.num_kv_heads, c.mlp_dim, c.num_decoder_layers, c.vocab_size) == (4096, 32, 8, 14336, 32, 128256)
  assert c.global_batch_size_to_train_on == 16 and c.micro_batch_size_to_train_on == 16
  assert c.ici_parallelism[list(c.mesh_axes).index("fsdp")] == 8       # the -1 default filled with all devices
  assert c.learning_rate_schedule_steps == c.steps


def test_fractional_batch_and_accumulation():
  c = init("per_device_batch_size=0.5", "gradient_accumulation_steps=2", n=8)
  assert c.micro_batch_size_to_train_on == 4 and c.global_batch_size_to_train_on == 8 and c.global_batch_size_to_load == 16


def test_global_parameter_scale():
  c = init("global_parameter_scale=8")
  d = init()
  assert c.emb_dim == 2 * d.emb_dim and c.num_query_heads == 2 * d.num_query_heads and c.num_decoder_layers == 2 * d.num_decoder_layers
  with pytest.raises(ValueError):
    init("global_parameter_scale=3")


def test_unknown_key_and_double_override_are_errors(monkeypatch):
  with pytest.raises(ConfigError):
    init("no_such_key=1")
  with pytest.raises(ConfigError):
    init("steps=1", "steps=2")
  monkeypatch.setenv("M_STEPS", "7")
  assert init().steps == 7
  with pytest.raises(ConfigError):
    init("steps=3")


def test_model_catalog_beats_yaml_and_needs_override_flag():
  with pytest.raises(ConfigError):
    init("model_name=llama3-8b", "base_emb_dim=128")
  c = init("model_name=llama3-8b", "base_emb_dim=128", "override_model_config=true")
  assert c.emb_dim == 128


def test_config_is_read_only_and_replace_recomputes():
  c = init(n=2)
  with pytest.raises(AttributeError):
    c.steps = 5
  d = c.replace(per_device_batch_size=3.0)
  assert d.global_batch_size_to_train_on == 6 and c.global_batch_size_to_train_on == 24


def test_logical_axis_rules_merge_and_override():
  c = init("logical_axis_rules=[['embed', ['fsdp']], ['my_axis', ['tensor']]]")
  rules = [tuple(r) for r in map(lambda r: (r[0], tuple(r[1]) if isinstance(r[1], list) else r[1]), c.logical_axis_rules)]
  assert [r for r in rules if r[0] == "embed"] == [("embed", ("fsdp",))]
  assert ("my_axis", ("tensor",)) in rules and any(r[0] == "mlp" for r in rules)
  o = init("logical_axis_rules=[['embed', ['fsdp']]]", "override_logical_axis_rules=true")
  assert len(o.logical_axis_rules) == 1


def test_custom_mesh_and_rule_and_mesh_fill():
  c = init("custom_mesh_and_rule=pure-fsdp", n=4)
  assert list(c.mesh_axes) == ["fsdp"] and c.mesh_shape == [4]
  c = init("ici_fsdp_parallelism=2", "ici_tensor_parallelism=-1", n=8)
  assert c.tensor_mesh_size == 4 and c.fsdp_mesh_size == 2
  with pytest.raises(ValueError):
    init("ici_fsdp_parallelism=3", n=8)


def test_validators():
  for bad in ("remat_policy=nope", "opt_type=lion", "decoder_block=bert", "quantization=int3", "context_parallel_strategy=zigzag"):
    with pytest.raises(ValueError):
      init(bad)
  with pytest.raises(ValueError):
    init("ici_pipeline_parallelism=2", "ici_fsdp_parallelism=2", "base_num_decoder_layers=3", n=4)
  c = init("ici_pipeline_parallelism=2", "ici_fsdp_parallelism=2", "base_num_decoder_layers=8", "num_layers_per_pipeline_stage=2", n=4)
  assert c.num_pipeline_repeats == 2 and c.num_pipeline_microbatches == 2


def test_yaml_base_config_chain(tmp_path):
  child = tmp_path / "child.yml"
  child.write_text("base_config: base.yml\nsteps: 11\nmodel_name: llama2-7b\n")
  grand = tmp_path / "grand.yml"
  grand.write_text(f"base_config: {child}\nsteps: 12\n")
  c = pyconfig.initialize(["t", str(grand), "log_config=false"], num_devices=1)
  assert c.steps == 12 and c.emb_dim == 4096


def test_legacy_sequence_degree_folds_into_context():
  from helpers import tiny_config
  c = tiny_config("llama3-8b", ["ici_sequence_parallelism=2", "ici_fsdp_parallelism=2"], num_devices=4)
  shape = dict(zip(c.mesh_axes, c.mesh_shape))
  assert shape["context"] == 2 and shape["fsdp"] == 2 and "sequence" not in shape


REJECTED = [
    (["load_parameters_path=/a", "load_full_state_path=/b"], "At most one of"),
    (["enable_emergency_checkpoint=true"], "local_checkpoint_directory"),
    (["enable_emergency_checkpoint=true", "local_checkpoint_directory=/tmp/x", "local_checkpoint_period=0"], "local_checkpoint_period"),
    (["attention_type=chunk", "chunk_attn_window_size=0"], "chunk_attn_window_size"),
    (["attention_type=local_sliding", "sliding_window_size=0"], "sliding_window_size"),
    (["mla_qk_head_chunk_size=3"], "mla_qk_head_chunk_size"),
    (["use_indexer=true"], "attention_type='mla'"),
    (["use_qk_clip=true"], "QK-Clip is only supported"),
    (["share_kv_projections=true", "fused_qkv=true"], "fused_qkv"),
    (["num_kv_shared_layers=1", "fused_qkv=true"], "num_kv_shared_layers"),
    (["quantize_kvcache=true", "kv_quant_axis="], "kv_quant_axis"),
    (["attention_type=block_diffusion", "packing=true"], "does not support packing"),
    (["training_objective=block_diffusion", "packing=false"], "requires `attention_type='block_diffusion'`"),
    (["training_objective=block_diffusion", "attention_type=block_diffusion", "packing=false", "block_diffusion_mask_id=999999"], "block_diffusion_mask_id"),
    (["quantization=fp8", "gradient_accumulation_steps=2"], "gradient accumulation"),
    (["use_batch_split_schedule=true", "quantization=int8"], "fp8_full"),
    (["use_manual_quantization=true"], "use_batch_split_schedule"),
    (["num_experts=4", "num_experts_per_tok=2", "routed_bias=true", "routed_bias_update_rate=0.1"], "Loss-free load balancing"),
    (["num_experts=4", "num_experts_per_tok=2", "num_moe_token_chunks=3", "max_target_length=32"], "num_moe_token_chunks"),
    (["decoder_block=llama4", "num_experts=4", "num_experts_per_tok=2"], "top-1 routing"),
    (["decoder_block=llama4", "num_experts=4", "num_experts_per_tok=1", "capacity_factor=1.0"], "capacity_factor"),
    (["partial_rotary_factor=0.5"], "partial_rotary_factor"),
    (["decoder_block=qwen3_next", "gdn_num_value_heads=3", "gdn_num_key_heads=2"], "gdn_num_value_heads"),
    (["use_multimodal=true"], "Multimodal is only supported"),
    (["use_sft=true", "use_dpo=true", "packing=false"], "Only one of"),
    (["use_dpo=true", "packing=true"], "DPO does not support packing"),
    (["num_vocab_tiling=7"], "vocab tiles"),
    (["ring_scan_unroll=2", "context_parallel_strategy=all_gather"], "ring_scan_unroll"),
    (["dcn_data_parallelism=2"], "dcn degrees"),
    (["enable_streaming_diloco=true", "scan_layers=false"], "scan_layers=True"),
    (["distill_alpha_end=1.5"], "distill_alpha_end must be in [0, 1]"),
    (["distill_temperature_end=0"], "distill_temperature_end must be > 0"),
    (["distill_beta=0.0", "distill_beta_end=0.5"], "distill_beta_end=0.5"),
    (["distill_alpha_schedule=linear"], "distill_alpha_end is None"),
    (["load_full_state_path=/tmp/none", "enable_checkpointing=false"], "enable_checkpointing=True to load"),
    (["enable_multi_tier_checkpointing=true", "local_checkpoint_directory=/tmp/x", "local_checkpoint_period=2"], "Exactly one of"),
    (["elastic_backup_kind=tape"], "elastic_backup_kind"),
    (["use_batch_split_schedule=true", "batch_split_factor=0"], "batch_split_factor"),
    (["context_parallel_strategy=spiral"], "context_parallel_strategy"),
    (["sharding_tolerance=1.5"], "sharding_tolerance"),
    (["indexer_cutoff_threshold=device"], "indexer_cutoff_threshold"),
    (["engram_layers=[1]", "engram_vocab_bases=[50]", "engram_max_ngram_size=3", "tokenizer_type=byte"], "Engram vocab size mismatch"),
    (["use_ring_of_experts=true", "num_experts=4", "num_experts_per_tok=2"], "When EP rank is 1"),
]


import pytest  # noqa: E402


@pytest.mark.parametrize("overrides,fragment", REJECTED, ids=[r[1][:28].replace(" ", "_") for r in REJECTED])
def test_illegal_combinations_are_rejected_at_parse_time(overrides, fragment):
  """One case per cross-field rule: the config layer refuses the combination and names the offending keys."""
  from helpers import tiny_config
  from maxtext_b200.config.types import ConfigValueError
  with pytest.raises((ConfigValueError, ValueError)) as e:
    tiny_config(extra=list(overrides))
  assert fragment in str(e.value), str(e.value)


def test_multi_device_rules_are_rejected_at_parse_time():
  from helpers import tiny_config
  from maxtext_b200.config.types import ConfigValueError
  for over, frag, n in [
      (["ici_tensor_parallelism=4", "ici_fsdp_parallelism=1", "base_num_query_heads=6", "base_num_kv_heads=2"], "num_query_heads", 4),
      (["ici_expert_parallelism=4", "ici_fsdp_parallelism=1", "num_experts=6", "num_experts_per_tok=2"], "num_experts", 4),
      (["ici_tensor_sequence_parallelism=2", "ici_context_parallelism=2", "ici_fsdp_parallelism=1"], "tensor_sequence parallelism cannot", 4),
      (["ici_context_parallelism=2", "ici_fsdp_parallelism=1", "context_parallel_strategy=ulysses", "base_num_kv_heads=1", "base_num_query_heads=4"], "MQA", 2),
  ]:
    with pytest.raises((ConfigValueError, ValueError)) as e:
      tiny_config(extra=over, num_devices=n)
    assert frag in str(e.value), (over, str(e.value))
