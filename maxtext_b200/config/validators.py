"""Cross-field checks of a configuration table: combinations that cannot work are rejected when the config is parsed,
with a message that names the keys, instead of surfacing later as a shape error (or not at all).

The rules are those of the reference's schema that apply to this implementation (src/maxtext/configs/types.py:3694-4418,
`set_derived_and_validate_values` section I); rules about TPU-only kernels, Pathways and JAX plumbing have no meaning
here and are left out. `run_all(t)` is called by `types.derive_and_validate` on the table with its derived values
(`emb_dim`, mesh sizes, batch sizes) already filled in."""
from __future__ import annotations


class ConfigValueError(ValueError):
  pass


def _g(t, key, default=None):
  v = t.get(key, default)
  return default if v is None else v


def _fail(msg: str):
  raise ConfigValueError(msg)


def check_checkpointing(t):
  if _g(t, "load_parameters_path", "") and _g(t, "load_full_state_path", ""):
    _fail("At most one of `load_parameters_path` or `load_full_state_path` should be set.")
  if (_g(t, "enable_emergency_checkpoint", False) or _g(t, "enable_multi_tier_checkpointing", False)):
    if not _g(t, "local_checkpoint_directory", ""):
      _fail("`local_checkpoint_directory` must be set for emergency / multi-tier checkpointing.")
    if int(_g(t, "local_checkpoint_period", 0)) <= 0:
      _fail("`local_checkpoint_period` must be > 0 for emergency / multi-tier checkpointing.")
  if int(_g(t, "checkpoint_period", 1)) <= 0:
    _fail("`checkpoint_period` must be > 0.")


def check_attention(t):
  at = t["attention_type"]
  if at == "chunk" and int(_g(t, "chunk_attn_window_size", 0)) <= 0:
    _fail("`chunk_attn_window_size` must be an integer > 0 for 'chunk' attention.")
  if at == "local_sliding" and int(_g(t, "sliding_window_size", 0)) <= 0:
    _fail("`sliding_window_size` must be an integer > 0 for 'local_sliding' attention.")
  chunk = int(_g(t, "mla_qk_head_chunk_size", 0))
  if chunk > 0 and (chunk > t["num_query_heads"] or t["num_query_heads"] % chunk):
    _fail(f"`mla_qk_head_chunk_size` ({chunk}) must divide `num_query_heads` ({t['num_query_heads']}).")
  if _g(t, "use_indexer", False):
    if at != "mla":
      _fail("`use_indexer=True` requires `attention_type='mla'`: only the MLA indexer produces this mask.")
    if int(_g(t, "q_lora_rank", 0)) == 0:
      _fail("The sparse indexer needs `q_lora_rank` > 0.")
    if float(_g(t, "indexer_loss_scaling_factor", 0.0)) > 0 and int(_g(t, "indexer_topk", 0)) >= int(t["max_target_length"]):
      _fail(f"`indexer_topk` ({t.get('indexer_topk')}) must be < `max_target_length` ({t['max_target_length']}) when the indexer loss is on.")
  if _g(t, "use_qk_clip", False):
    if at != "mla":
      _fail(f"QK-Clip is only supported when attention_type='mla', but found attention_type='{at}'.")
    if float(_g(t, "attn_logits_soft_cap", 0.0) or 0.0) > 0:
      _fail("QK-Clip monitors raw dot products; disable `attn_logits_soft_cap` when using `use_qk_clip`.")
  if _g(t, "share_kv_projections", False) and _g(t, "fused_qkv", False):
    _fail("`share_kv_projections` is not compatible with `fused_qkv`.")
  if int(_g(t, "num_kv_shared_layers", 0)) > 0:
    if _g(t, "fused_qkv", False):
      _fail("`num_kv_shared_layers > 0` is not compatible with `fused_qkv`.")
    if _g(t, "share_kv_projections", False):
      _fail("`num_kv_shared_layers > 0` is not compatible with `share_kv_projections`.")
  if _g(t, "quantize_kvcache", False) and not _g(t, "kv_quant_axis", ""):
    _fail("`kv_quant_axis` cannot be empty when quantize_kvcache is True.")
  for v in _g(t, "compress_ratios", ()) or ():
    if int(v) != 0 and int(v) < 4:
      _fail(f"compress_ratio must be 0 (disabled) or >= 4, got {v}")


def check_block_diffusion(t):
  at = t["attention_type"]
  if at == "block_diffusion" and _g(t, "packing", False):
    _fail("Block-diffusion attention does not support packing; set `packing=False`.")
  if _g(t, "training_objective", "") != "block_diffusion":
    return
  if at != "block_diffusion":
    _fail("`training_objective='block_diffusion'` requires `attention_type='block_diffusion'`.")
  mid = int(_g(t, "block_diffusion_mask_id", -1))
  if mid < 0 or mid >= int(t["vocab_size"]):
    _fail(f"`block_diffusion_mask_id` ({mid}) must satisfy 0 <= block_diffusion_mask_id < vocab_size ({t['vocab_size']}).")
  if int(_g(t, "mtp_num_layers", 0)) > 0:
    _fail("`training_objective='block_diffusion'` is not compatible with MTP.")
  if int(_g(t, "num_vocab_tiling", 1)) > 1:
    _fail("`training_objective='block_diffusion'` is not compatible with vocabulary tiling.")
  if _g(t, "use_dpo", False) or _g(t, "use_sft", False):
    _fail("`training_objective='block_diffusion'` supports pre-training only (no DPO / SFT).")
  if _g(t, "use_multimodal", False):
    _fail("`training_objective='block_diffusion'` supports text-only training.")
  contract = (_g(t, "block_diffusion_logit_alignment", "same_position"), _g(t, "block_diffusion_canvas_policy", "all_masked"))
  if contract not in {("same_position", "all_masked"), ("shifted", "seed_and_mask")}:
    _fail(f"Block-diffusion training supports only `same_position/all_masked` or `shifted/seed_and_mask`; received `{contract[0]}/{contract[1]}`.")
  if contract[1] == "seed_and_mask" and int(_g(t, "causal_block_size", 0)) < 2:
    _fail("`block_diffusion_canvas_policy='seed_and_mask'` requires `causal_block_size >= 2`.")


def check_quantization(t):
  q = _g(t, "quantization", "")
  if q in ("fp8", "nanoo_fp8", "fp8_gpu", "te_fp8_delayedscaling") and int(t["gradient_accumulation_steps"]) > 1:
    _fail("FP8 quantization with delayed scaling state is not compatible with gradient accumulation.")
  if _g(t, "use_batch_split_schedule", False) and q and q != "fp8_full":
    _fail("Batch split quantization only supports `quantization=fp8_full`")
  if _g(t, "use_manual_quantization", False) and not _g(t, "use_batch_split_schedule", False):
    _fail("manual quantization is only used when `use_batch_split_schedule=True`.")
  if _g(t, "use_sliced_mla_proj", False) and q:
    _fail("`use_sliced_mla_proj` is not supported with quantization.")


def check_moe(t):
  if int(t["num_experts"]) <= 1:
    return
  if int(t["moe_mlp_dim"]) <= 0:
    _fail("moe_mlp_dim must be positive for MoE models (num_experts > 1)")
  db = t["decoder_block"]
  if db == "gpt_oss" and not _g(t, "sparse_matmul", True) and float(_g(t, "capacity_factor", -1)) != -1:
    _fail("GPT-OSS MoE only supports dropless (capacity_factor=-1) with dense matmul.")
  if _g(t, "routed_bias", False) and float(_g(t, "routed_bias_update_rate", 0.0)) > 0 and db not in ("deepseek", "deepseek4"):
    _fail("Loss-free load balancing is only supported for the DeepSeek decoder block.")
  ep = int(t.get("expert_mesh_size", 1))
  if ep > 1 and int(t["num_experts"]) % ep:
    _fail(f"num_experts ({t['num_experts']}) must divide by the expert-parallel degree ({ep}).")
  n_chunks = int(_g(t, "num_moe_token_chunks", 1))
  if n_chunks > 1 and int(t["max_target_length"]) % n_chunks:
    _fail(f"num_moe_token_chunks={n_chunks} must evenly divide max_target_length={t['max_target_length']}.")
  if db == "llama4":
    if float(_g(t, "capacity_factor", -1)) >= 0:
      _fail("Llama4 decoder has not been tested with capacity_factor >= 0 -- please set that value to -1 for now!")
    if int(t["num_experts_per_tok"]) > 1:
      _fail("Only top-1 routing is supported for Llama4 for now!")
  if db in ("llama4", "envy"):
    step = max(1, int(_g(t, "interleave_moe_layer_step", 1)))
    if int(t["base_num_decoder_layers"]) % step:
      _fail(f"The number of decoder layers ({t['base_num_decoder_layers']}) must be divisible by interleave moe layer step ({step})")


def check_families(t):
  db = t["decoder_block"]
  if db in ("qwen3_next", "qwen3_5"):
    if int(_g(t, "gdn_num_value_heads", 1)) % max(1, int(_g(t, "gdn_num_key_heads", 1))):
      _fail("gdn_num_value_heads must be divisible by gdn_num_key_heads")
    rot = int(int(t["head_dim"]) * float(_g(t, "partial_rotary_factor", 1.0)))
    if rot % 2:
      _fail(f"Calculated rotary dimension ({rot}) must be a multiple of 2.")
  elif float(_g(t, "partial_rotary_factor", 1.0)) != 1.0:
    _fail("`partial_rotary_factor` is only effective when `decoder_block` is 'qwen3_next' or 'qwen3_5'.")
  if db == "deepseek4" and int(_g(t, "mtp_num_layers", 0)) > 0:
    _fail("DeepSeek4 decoder block currently does not support MTP layers.")
  if _g(t, "use_multimodal", False):
    ok = ("gemma3-4b", "gemma3-12b", "gemma3-27b", "gemma4-26b", "gemma4-31b", "llama4-17b-16e", "llama4-17b-128e", "qwen3-omni-30b-a3b",
          "qwen3-vl-2b", "qwen3-vl-4b", "qwen3-vl-30b-a3b", "qwen3.5-35b-a3b", "qwen3.5-397b-a17b")
    if t["model_name"] not in ok and t["model_name"] != "default":
      _fail(f"Multimodal is only supported for {ok}, not {t['model_name']}")
    if _g(t, "use_sft", False):
      if not _g(t, "sft_train_on_completion_only", False):
        _fail("For multimodal SFT, `sft_train_on_completion_only` must be True.")
      if _g(t, "packing", False):
        _fail("For multimodal SFT, `packing` is not yet supported.")


def check_post_training(t):
  if _g(t, "use_sft", False) and _g(t, "use_dpo", False):
    _fail("Only one of `use_sft` or `use_dpo` can be True.")
  if _g(t, "use_dpo", False):
    if _g(t, "packing", False):
      _fail("DPO does not support packing. Set `packing=False`.")
    if t["dataset_type"] == "tfds":
      _fail("dataset_type=tfds is not supported for DPO training; use dataset_type=grain or dataset_type=hf.")


def check_batch_and_vocab(t):
  pdb = float(t["per_device_batch_size"])
  nvt = int(t["num_vocab_tiling"])
  if pdb > 0 and (pdb * int(t["max_target_length"])) % nvt:
    _fail("Per device batch size times sequence length should be divisible by the number of vocab tiles.")
  if int(t["eval_interval"]) > 0 >= int(t["eval_steps"]) and _g(t, "generate_padding_batch_eval", False):
    _fail("`eval_steps` must be > 0 when `generate_padding_batch_eval` is True.")
  if int(t["max_target_length"]) < 1:
    _fail("max_target_length must be >= 1")


def check_parallelism(t):
  cp = int(t.get("context_mesh_size", 1))
  strat = t["context_parallel_strategy"]
  if strat not in ("ring", "usp") and int(_g(t, "ring_scan_unroll", 1)) != 1:
    _fail(f"ring_scan_unroll={t.get('ring_scan_unroll')} was specified, but is only supported when context_parallel_strategy='ring' or 'usp'.")
  if cp > 1 and strat == "ulysses":
    if int(t["num_kv_heads"]) == 1:
      _fail("Ulysses attention does not support MQA with context parallelism > 1.")
    if int(t["num_kv_heads"]) % cp and cp % int(t["num_kv_heads"]):
      _fail(f"Ulysses attention requires num_kv_heads ({t['num_kv_heads']}) and the context degree ({cp}) to divide one another.")
  if strat == "usp":
    u = int(t.get("context_usp_ulysses_mesh_size", 1))
    if u > 1 and int(t["num_query_heads"]) % u:
      _fail(f"usp: num_query_heads ({t['num_query_heads']}) must divide by ici_context_usp_ulysses_parallelism ({u}).")
  if cp > 1:
    if _g(t, "use_multimodal", False):
      _fail("Context parallelism does not support multimodal attention (bidirectional image blocks).")
    if _g(t, "moba", False):
      _fail("Context parallelism does not support MoBA.")
  tsp = int(t.get("tensor_sequence_mesh_size", 1))
  if tsp > 1:
    if cp > 1 or int(t.get("stage_mesh_size", 1)) > 1:
      _fail("tensor_sequence parallelism cannot be combined with context or pipeline parallelism.")
    if int(_g(t, "mtp_num_layers", 0)) > 0:
      _fail("tensor_sequence parallelism does not support MTP layers.")
    if int(t["max_target_length"]) % tsp:
      _fail(f"max_target_length ({t['max_target_length']}) must divide by the tensor_sequence degree ({tsp}).")
  tp = int(t.get("tensor_mesh_size", 1)) * tsp
  if tp > 1:
    if int(t["num_query_heads"]) % tp:
      _fail(f"num_query_heads ({t['num_query_heads']}) must divide by the tensor-parallel degree ({tp}).")
    if int(t["mlp_dim"]) % tp:
      _fail(f"mlp_dim ({t['mlp_dim']}) must divide by the tensor-parallel degree ({tp}).")
  dcn = 1
  for v in t.get("dcn_parallelism", ()):
    dcn *= int(v)
  if abs(dcn) > 1 and not int(t["num_slices"]) > 1:
    _fail("DCN parallelism requested but only one slice available.")
  if _g(t, "enable_streaming_diloco", False):
    if not _g(t, "scan_layers", True):
      _fail("enable_streaming_diloco=True requires scan_layers=True.")
    frags = _g(t, "num_diloco_fragments", None)
    if frags is not None and int(frags) > 1 and int(t["num_decoder_layers"]) % (int(frags) - 1):
      _fail(f"The number of decoder layers ({t['num_decoder_layers']}) must be divisible by (num_diloco_fragments - 1) ({int(frags) - 1}) "
            "when enable_streaming_diloco is True.")


def _num(v):
  """Optional numeric keys arrive as None, the string 'None', or a number."""
  if v is None or (isinstance(v, str) and v.strip().lower() in ("none", "")):
    return None
  return float(v)


def check_schedules_and_distillation(t):
  """src/maxtext/configs/types.py:3310-3345: the distillation parameter schedules (the WSD phase check lives in `types.py`)."""
  a_end, t_end, b_end = _num(t.get("distill_alpha_end")), _num(t.get("distill_temperature_end")), _num(t.get("distill_beta_end"))
  if a_end is not None and not 0.0 <= a_end <= 1.0:
    _fail(f"distill_alpha_end must be in [0, 1], got {a_end}")
  if t_end is not None and t_end <= 0.0:
    _fail(f"distill_temperature_end must be > 0, got {t_end}")
  if b_end is not None and b_end < 0.0:
    _fail(f"distill_beta_end must be >= 0, got {b_end}")
  if float(_g(t, "distill_beta", 0.0)) == 0.0 and b_end is not None and b_end > 0.0:
    _fail(f"distill_beta=0.0 but distill_beta_end={b_end}. Feature extraction is disabled when distill_beta starts at 0.0.")
  for name, end in (("distill_alpha", a_end), ("distill_temperature", t_end), ("distill_beta", b_end)):
    sched = str(_g(t, f"{name}_schedule", "constant"))
    if sched != "constant" and end is None:
      _fail(f"{name}_schedule is '{sched}' but {name}_end is None. Set {name}_end to a target value or use schedule='constant'.")


def check_misc(t):
  """Single-key ranges and pairings from src/maxtext/configs/types.py:3183-3197, 3356-3420, 3815-3818, 3884-3930, 4280-4330."""
  if _g(t, "load_full_state_path", "") and not _g(t, "enable_checkpointing", True):
    # parameters alone (`load_parameters_path`) load without the checkpoint manager here; a full state needs it
    _fail("You must set enable_checkpointing=True to load a full training state.")
  if _g(t, "enable_multi_tier_checkpointing", False):
    mins, steps = t.get("multi_tier_checkpointing_backup_interval_minutes"), t.get("multi_tier_checkpointing_backup_interval_steps")
    if (_num(mins) is None) == (_num(steps) is None):
      _fail("Exactly one of `multi_tier_checkpointing_backup_interval_minutes` or `multi_tier_checkpointing_backup_interval_steps` must be set.")
    if _num(steps) is not None and _num(steps) <= 0:
      _fail(f"`multi_tier_checkpointing_backup_interval_steps` ({steps}) must be > 0.")
  if str(_g(t, "elastic_backup_kind", "snapshot")) not in ("snapshot", "checkpoint"):
    _fail(f"elastic_backup_kind must be one of 'snapshot' or 'checkpoint', got '{t.get('elastic_backup_kind')}'.")
  tol = float(_g(t, "sharding_tolerance", 0.02))
  if tol > 1.0 or tol < 0.0:
    _fail(f"sharding_tolerance must lie in [0, 1], got {tol}.")
  if not _g(t, "use_indexer", False) and str(_g(t, "indexer_cutoff_threshold", "remat")) != "remat":
    _fail(f"Setting `indexer_cutoff_threshold='{t.get('indexer_cutoff_threshold')}'` is only valid when `use_indexer=True`.")
  chunk = int(_g(t, "mla_qk_head_chunk_size", 0) or 0)
  if chunk > 0 and _g(t, "use_indexer", False) and int(_g(t, "indexer_n_heads", chunk)) % chunk != 0:
    _fail(f"`mla_qk_head_chunk_size` ({chunk}) must divide `indexer_n_heads` ({t.get('indexer_n_heads')}).")
  layers = list(_g(t, "engram_layers", []) or [])
  if layers:
    bases, n = list(_g(t, "engram_vocab_bases", []) or []), int(_g(t, "engram_max_ngram_size", 0))
    if len(bases) != n - 1:
      _fail(f"Engram vocab size mismatch: expected {n - 1} (max_ngram_size - 1), but got {bases}.")
  if str(_g(t, "decoder_block", "")) == "deepseek4" and int(_g(t, "first_num_hash_layers", 0) or 0) > 0 and _g(t, "use_ring_of_experts", False):
    _fail("DeepSeek V4 hash routing is currently not supported with ring of experts.")
  ep = 1
  for k in ("ici_expert_parallelism", "dcn_expert_parallelism"):
    ep *= max(1, int(_g(t, k, 1) or 1))
  if ep == 1 and not _g(t, "override_logical_axis_rules", False):
    for flag, off in (("use_ring_of_experts", False),):            # random routing works on one rank here, the ring needs peers
      if _g(t, flag, off) != off:
        _fail(f"When EP rank is 1, {flag} must be {off} (was {t.get(flag)}).")
  if _g(t, "use_batch_split_schedule", False):
    pp = max(1, int(_g(t, "ici_pipeline_parallelism", 1) or 1)) * max(1, int(_g(t, "dcn_pipeline_parallelism", 1) or 1))
    if pp > 1:
      _fail("`use_batch_split_schedule=True` is not implemented under pipeline parallelism (the pipeline already runs micro-batches).")
    split = int(_g(t, "batch_split_factor", 1))
    if split < 1:
      _fail(f"`batch_split_factor` must be >= 1, got {split}.")
  dpo = t.get("dpo") if isinstance(t.get("dpo"), dict) else None
  if _g(t, "use_dpo", False) and dpo and dpo.get("max_prompt_length") is not None:
    if int(dpo["max_prompt_length"]) >= int(t["max_target_length"]):
      _fail(f"dpo.max_prompt_length ({dpo['max_prompt_length']}) must be less than max_target_length ({t['max_target_length']}).")
  if str(_g(t, "dataset_type", "")) == "tfds" and not _g(t, "dataset_name", "") and not _g(t, "dataset_path", ""):
    _fail("dataset_name can't be empty when dataset_type=tfds")


ALL_CHECKS = (check_checkpointing, check_attention, check_block_diffusion, check_quantization, check_moe, check_families, check_post_training,
              check_batch_and_vocab, check_parallelism, check_schedules_and_distillation, check_misc)


def run_all(t: dict) -> None:
  for fn in ALL_CHECKS:
    fn(t)
