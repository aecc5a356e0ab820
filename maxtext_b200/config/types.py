"""Enumerations, cross-field validation and derived values of the configuration.

Mirrors the behaviour of MaxText's schema (src/maxtext/configs/types.py: enums 83-297, derived
values and validators in `set_derived_and_validate_values` 3162-4418) as plain functions over a
dict: the loader hands in the merged raw table, this module returns the final table with
derived keys (`emb_dim`, `global_batch_size_to_train_on`, `ici_parallelism`, `checkpoint_dir`...).
"""
from __future__ import annotations

import datetime
import math
import os

MESH_AXES_DEFAULT = [
    "diloco", "data", "stage", "fsdp", "fsdp_transpose", "context", "context_usp_ulysses",
    "context_autoregressive", "tensor", "tensor_sequence", "expert", "autoregressive",
]

# mesh axis name -> config suffix ("stage" is spelled "pipeline" in ici_/dcn_ keys)
AXIS_TO_KEY = {a: a for a in MESH_AXES_DEFAULT}
AXIS_TO_KEY["stage"] = "pipeline"
AXIS_TO_KEY["sequence"] = "sequence"

DECODER_BLOCKS = (
    "default", "llama2", "mistral", "mixtral", "deepseek", "gemma", "gemma2", "gemma3", "gemma4",
    "gemma4_small", "qwen2", "qwen3", "qwen3_moe", "qwen3_custom_moe", "qwen3_next", "qwen3_5", "gpt3",
    "gpt_oss", "simple", "simple_mlp", "llama4", "olmo3", "deepseek4", "envy",
)
# families with a model implementation in maxtext_b200.models
IMPLEMENTED_DECODER_BLOCKS = (
    "default", "llama2", "mistral", "mixtral", "deepseek", "gemma", "gemma2", "gemma3", "qwen2", "qwen3",
    "qwen3_moe", "gpt3", "gpt_oss", "olmo3", "simple", "simple_mlp",
)
REMAT_POLICIES = (
    "minimal_with_context", "minimal", "save_dot_with_context_except_mlp", "save_dot_except_mlpwi",
    "save_dot_except_mlp", "save_qkv_proj", "qkv_proj_offloaded", "custom", "minimal_offloaded",
    "save_out_proj", "full", "minimal_flash", "minimal_with_quantization", "minimal_with_context_and_quantization",
)
QUANTIZATIONS = (
    "", "int8", "intmp", "int4", "fp4", "fp8", "fp8_full", "fp8_gpu", "fp8_nanoo", "nanoo_fp8", "fp8_e4m3",
    "fp8_e5m2", "aqt_fp8", "aqt_fp8_full", "te_noscaling", "te_fp8_delayedscaling", "te_fp8_currentscaling",
    "te_mxfp8", "te_nvfp4", "te_nvfp4_no_rht",
)
OPT_TYPES = ("adamw", "adam_pax", "sgd", "muon")
ATTENTION_KERNELS = ("autoselected", "dot_product", "flash", "cudnn_flash_te", "cudnn_flash_jax", "paged", "vllm_rpa")
ATTENTION_TYPES = ("global", "local_sliding", "chunk", "mla", "full", "compressed", "block_diffusion")
DATASET_TYPES = ("synthetic", "hf", "grain", "tfds", "c4_mlperf", "olmo_grain", "tokens")
CP_STRATEGIES = ("all_gather", "ring", "ulysses", "usp")
ROPE_TYPES = ("default", "llama3.1", "yarn")
HARDWARE = ("tpu", "gpu", "gpu_multiprocess", "cpu")
PROFILERS = ("", "xplane", "nsys")
DTYPES = {"bfloat16": "bfloat16", "bf16": "bfloat16", "float32": "float32", "fp32": "float32",
          "float16": "float16", "fp16": "float16", "float8_e4m3fn": "float8_e4m3fn"}


from .validators import ConfigValueError, run_all as _run_validators  # noqa: E402


def detect_num_devices(table: dict) -> int:
  """Device count used for derivation: WORLD_SIZE if launched by a torchrun-style launcher, else the
  reference's launcher variable NNODES (tools/orchestration/gpu_multi_process_run.sh), else 1."""
  if table.get("internal_compile") and int(table.get("internal_compile_num_devices", -1)) > 0:
    return int(table["internal_compile_num_devices"])
  if table.get("compile_topology"):
    from ..utils import topology
    return topology.devices_in(table["compile_topology"]) * max(1, int(table.get("compile_topology_num_slices", 1)))
  for var in ("WORLD_SIZE", "NNODES"):
    if os.environ.get(var):
      try:
        return max(1, int(os.environ[var]))
      except ValueError:
        pass
  return 1


def individual_scales(scale: int):
  if scale <= 0:
    raise ConfigValueError("global_parameter_scale must be a positive power of two")
  lg = int(math.floor(math.log2(scale)))
  if 2 ** lg != scale:
    raise ConfigValueError("global_parameter_scale must be a power of two")
  base, rem = divmod(lg, 3)
  head = base + (1 if rem > 0 else 0)
  emb = base + (1 if rem > 1 else 0)
  return emb, head, head, base  # emb, heads, mlp, layers


def fill_unspecified(parallelism: list[int], target: int, what: str) -> list[int]:
  """Replace the single -1 entry by target / product(others) (src/maxtext/utils/max_utils.py:461)."""
  vals = list(parallelism)
  if vals.count(-1) > 1:
    raise ConfigValueError(f"at most one {what} degree may be -1, got {vals}")
  if -1 in vals:
    known = -int(math.prod(vals))
    if known <= 0 or target % known:
      raise ConfigValueError(f"{what}: cannot fill -1: {target} devices not divisible by product {known} of {vals}")
    vals[vals.index(-1)] = target // known
  if int(math.prod(vals)) != target:
    raise ConfigValueError(f"{what} degrees {vals} multiply to {math.prod(vals)}, expected {target}")
  return vals


def _batch_sizes(pdb: float, expansion: float, ndev: int, accum: int):
  exp = expansion if expansion and expansion > 0 else 1
  if pdb < 1.0:
    micro_load = int(ndev * exp)
  else:
    micro_load = int(ndev * pdb * exp)
  micro_train = int(ndev * pdb)
  return int(micro_load * accum), int(micro_train * accum), micro_train


def _choice(t: dict, key: str, allowed) -> None:
  if t[key] not in allowed:
    raise ConfigValueError(f"{key}={t[key]!r} is not one of {list(allowed)}")


def derive_and_validate(raw: dict, num_devices: int = 1) -> dict:
  t = dict(raw)

  # ---- normalise spelled values
  for k in ("dtype", "weight_dtype", "grad_dtype", "mu_dtype", "dtype_mm", "kv_quant_dtype"):
    v = t.get(k)
    if isinstance(v, str) and v in DTYPES:
      t[k] = DTYPES[v]
  for k in ("max_num_checkpoints_to_keep", "checkpoint_todelete_subdir", "checkpoint_todelete_full_path",
            "muon_consistent_rms", "distill_layer_indices"):
    if t.get(k) in ("None", "none", ""):
      t[k] = None
  if not t.get("mu_dtype"):
    t["mu_dtype"] = t["weight_dtype"]

  _choice(t, "decoder_block", DECODER_BLOCKS)
  _choice(t, "remat_policy", REMAT_POLICIES)
  _choice(t, "opt_type", OPT_TYPES)
  _choice(t, "attention", ATTENTION_KERNELS)
  _choice(t, "attention_type", ATTENTION_TYPES)
  _choice(t, "dataset_type", DATASET_TYPES)
  _choice(t, "context_parallel_strategy", CP_STRATEGIES)
  _choice(t, "rope_type", ROPE_TYPES)
  _choice(t, "hardware", HARDWARE)
  _choice(t, "profiler", PROFILERS)
  _choice(t, "quantization", QUANTIZATIONS)
  _choice(t, "lr_schedule_type", ("cosine", "wsd"))
  _choice(t, "shard_mode", ("auto", "explicit"))
  _choice(t, "decode_sampling_strategy", ("greedy", "weighted", "nucleus", "topk", "composite"))

  # ---- run name / output paths
  if not t.get("run_name"):
    t["run_name"] = os.environ.get("JOBSET_NAME") or f'{t["model_name"]}_{datetime.datetime.now().strftime("%Y-%m-%d-%H-%M")}'
  if t.get("base_output_directory"):
    out = os.path.join(t["base_output_directory"], t["run_name"])
    t["checkpoint_dir"] = os.path.join(out, "checkpoints", "")
    t["metrics_dir"] = os.path.join(out, "metrics", "")
    t["tensorboard_dir"] = os.path.join(out, "tensorboard", "")
  else:
    t["checkpoint_dir"] = t["metrics_dir"] = t["tensorboard_dir"] = None

  # ---- steps / schedule
  if t["learning_rate_schedule_steps"] == -1:
    t["learning_rate_schedule_steps"] = t["steps"]
  if t["steps"] == -1:
    t["steps"] = t["learning_rate_schedule_steps"]
  if t["lr_schedule_type"] == "wsd" and t["warmup_steps_fraction"] + t["wsd_decay_steps_fraction"] > 1.0:
    raise ConfigValueError("warmup_steps_fraction + wsd_decay_steps_fraction must not exceed 1")

  # ---- model dims
  emb_s, head_s, mlp_s, layer_s = individual_scales(int(t["global_parameter_scale"]))
  t["emb_dim"] = (2 ** emb_s) * t["base_emb_dim"]
  t["num_query_heads"] = (2 ** head_s) * t["base_num_query_heads"]
  t["num_kv_heads"] = (2 ** head_s) * t["base_num_kv_heads"]
  t["mlp_dim"] = (2 ** mlp_s) * t["base_mlp_dim"]
  t["moe_mlp_dim"] = (2 ** mlp_s) * t["base_moe_mlp_dim"] if t["base_moe_mlp_dim"] > 0 else t["base_moe_mlp_dim"]
  t["num_decoder_layers"] = (2 ** layer_s) * t["base_num_decoder_layers"]
  if t["num_experts"] > 1 and t["moe_mlp_dim"] <= 0:
    t["moe_mlp_dim"] = t["mlp_dim"]
  if t["num_query_heads"] % max(1, t["num_kv_heads"]):
    raise ConfigValueError("num_query_heads must be a multiple of num_kv_heads")
  if t["num_experts"] > 1 and t["num_experts_per_tok"] > t["num_experts"]:
    raise ConfigValueError("num_experts_per_tok cannot exceed num_experts")

  # ---- devices / slices
  t["num_target_devices"] = int(num_devices)
  if t["num_slices"] in (-1, None):
    t["num_slices"] = max(1, int(t.get("compile_topology_num_slices", -1))) if t.get("compile_topology") else 1

  # ---- mesh degrees in mesh-axis order
  axes = list(t["mesh_axes"])
  for prefix in ("ici", "dcn"):
    # the legacy `sequence` axis is no mesh axis any more: its degree is folded into `context` (base.yml:663,676)
    seq = int(t.get(f"{prefix}_sequence_parallelism", 1) or 1)
    if seq > 1 and "sequence" not in axes and "context" in axes:
      t[f"{prefix}_context_parallelism"] = max(1, int(t.get(f"{prefix}_context_parallelism", 1))) * seq
      t[f"{prefix}_sequence_parallelism"] = 1
  def degree(prefix, axis):
    key = f"{prefix}_{AXIS_TO_KEY.get(axis, axis)}_parallelism"
    return int(t.get(key, 1))
  ici = [degree("ici", a) for a in axes]
  dcn = [degree("dcn", a) for a in axes]
  per_slice = num_devices // t["num_slices"] if num_devices % t["num_slices"] == 0 else num_devices
  if ici.count(-1) == 0 and int(math.prod(ici)) != per_slice and "fsdp" in axes and t.get("custom_mesh_and_rule"):
    pass
  t["ici_parallelism"] = fill_unspecified(ici, per_slice, "ici")
  t["dcn_parallelism"] = fill_unspecified(dcn, t["num_slices"], "dcn")
  t["mesh_shape"] = [i * d for i, d in zip(t["ici_parallelism"], t["dcn_parallelism"])]
  for a, n in zip(axes, t["mesh_shape"]):
    t[f"{a}_mesh_size"] = n

  # ---- batch sizes
  (t["global_batch_size_to_load"], t["global_batch_size_to_train_on"], t["micro_batch_size_to_train_on"]) = _batch_sizes(
      float(t["per_device_batch_size"]), float(t["expansion_factor_real_data"]), num_devices,
      int(t["gradient_accumulation_steps"]))
  (t["global_batch_size_to_load_eval"], t["global_batch_size_to_eval_on"], t["micro_batch_size_to_eval_on"]) = _batch_sizes(
      float(t["eval_per_device_batch_size"]) or float(t["per_device_batch_size"]), float(t["expansion_factor_real_data"]),
      num_devices, 1)
  if t["micro_batch_size_to_train_on"] < 1:
    raise ConfigValueError("per_device_batch_size x devices gives an empty batch")
  if t["enable_rampup_batch_size"]:
    start, _, _ = _batch_sizes(float(t["per_device_batch_size_start"]), float(t["expansion_factor_real_data"]),
                               num_devices, int(t["gradient_accumulation_steps"]))
    inc, _, _ = _batch_sizes(float(t["per_device_batch_size_increment"]), float(t["expansion_factor_real_data"]),
                             num_devices, int(t["gradient_accumulation_steps"]))
    t["global_batch_size_to_load_start"] = start
    t["global_batch_size_to_load_increment"] = inc
    diff = t["global_batch_size_to_load"] - start
    if inc <= 0 or diff < 0 or diff % inc:
      raise ConfigValueError("ramp-up: (end - start) batch must be a non-negative multiple of the increment")
    t["rampup_end_step"] = diff // inc
    t["rampup_samples_per_increment_to_load"] = t["global_rampup_samples"] / max(1, t["rampup_end_step"])

  # ---- pipeline (src/maxtext/configs/types.py:3565-3659)
  stages = t.get("stage_mesh_size", 1)
  t["using_pipeline_parallelism"] = stages > 1
  if stages > 1:
    lps = int(t["num_layers_per_pipeline_stage"])
    pp_layers = t["num_decoder_layers"] if t["pipeline_parallel_layers"] == -1 else int(t["pipeline_parallel_layers"])
    t["pipeline_parallel_layers"] = pp_layers
    if pp_layers % (stages * lps):
      raise ConfigValueError(f"pipelined layers ({pp_layers}) must divide by stages x layers_per_stage ({stages * lps})")
    t["num_pipeline_repeats"] = pp_layers // (stages * lps)
    if t["num_pipeline_microbatches"] == -1:
      t["num_pipeline_microbatches"] = stages
    if t["num_pipeline_microbatches"] % stages:
      raise ConfigValueError("num_pipeline_microbatches must be a multiple of the number of stages")
    mb = t["micro_batch_size_to_train_on"]
    if mb % t["num_pipeline_microbatches"]:
      raise ConfigValueError("micro batch must divide evenly into pipeline microbatches")
  else:
    if t["num_pipeline_repeats"] == -1:
      t["num_pipeline_repeats"] = 1
    if t["num_pipeline_microbatches"] == -1:
      t["num_pipeline_microbatches"] = 1

  # ---- context parallel checks (src/maxtext/configs/types.py:4004-4147)
  cp = t.get("context_mesh_size", 1)
  if cp > 1:
    if t["max_target_length"] % (2 * cp if t["context_parallel_load_balance"] else cp):
      raise ConfigValueError("max_target_length must divide by (2x when load-balanced) the context parallel degree")
    if t["context_parallel_strategy"] in ("ulysses",) and t["num_query_heads"] % cp:
      raise ConfigValueError("ulysses context parallelism needs num_query_heads divisible by the context degree")
  if t.get("context_usp_ulysses_mesh_size", 1) > 1 and t["context_parallel_strategy"] != "usp":
    raise ConfigValueError("ici_context_usp_ulysses_parallelism > 1 requires context_parallel_strategy=usp")

  # ---- tensor parallel vs kv heads (src/maxtext/layers/attentions.py:576)
  tp = t.get("tensor_mesh_size", 1) * t.get("tensor_sequence_mesh_size", 1)
  if tp > 1 and t["attention_type"] != "mla" and t["num_kv_heads"] % tp and tp % t["num_kv_heads"]:
    raise ConfigValueError(f"num_kv_heads={t['num_kv_heads']} incompatible with tensor parallel degree {tp}")

  if t["gradient_accumulation_steps"] < 1:
    raise ConfigValueError("gradient_accumulation_steps must be >= 1")
  if t["num_vocab_tiling"] < 1:
    raise ConfigValueError("num_vocab_tiling must be >= 1")
  if t["attention_type"] == "mla" and t["share_kv_projections"]:
    raise ConfigValueError("share_kv_projections is not compatible with attention_type=mla")

  # custom remat: collect the named tensors (src/maxtext/configs/types.py:3538-3563)
  names = ("context", "mlpwi", "mlpwi_0", "mlpwi_1", "mlpwo", "moe_mlpwi_0", "moe_mlpwi_1", "moe_mlpwo", "query_proj",
           "key_proj", "value_proj", "kv_proj", "qkv_proj", "out_proj", "query_wa_proj", "kv_wa_proj", "mla_q", "mla_kv",
           "attention_out", "engram", "decoder_layer_input", "indexer_cutoff_threshold")
  t["tensors_on_device"] = [n for n in names if t.get(n) == "device"]
  t["tensors_to_offload"] = [n for n in names if t.get(n) == "offload"]

  # expert / context axis helpers
  t["ep_enabled"] = t.get("expert_mesh_size", 1) > 1
  _run_validators(t)
  return t
