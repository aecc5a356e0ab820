"""Named benchmark recipes for B200 nodes: model + parallelism + tuning keys, the counterpart of the reference's per-chip
recipe tables (benchmarks/maxtext_trillium_model_configs.py, maxtext_v5p_model_configs.py: `MaxTextModel(model_name,
model_type, tuning_params, xla_flags)`). XLA flag lists have no equivalent here; what a recipe tunes instead are the
framework's own knobs (remat policy, batch, parallel degrees, collective implementation, quantisation)."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class Recipe:
  name: str
  model: str
  gpus: int
  tuning: dict = field(default_factory=dict)
  note: str = ""

  def overrides(self) -> list[str]:
    base = {"model_name": self.model, "dataset_type": "synthetic", "enable_checkpointing": "false", "dtype": "bfloat16",
            "weight_dtype": "float32", "attention": "flash", "steps": 20, "log_period": 5}
    base.update(self.tuning)
    return [f"{k}={str(v).lower() if isinstance(v, bool) else v}" for k, v in base.items()]


RECIPES = {r.name: r for r in [
    Recipe("llama3_8b_8192_1gpu", "llama3-8b", 1, dict(per_device_batch_size=2, max_target_length=8192, remat_policy="full"),
           "headline configuration on one GPU"),
    Recipe("llama3_8b_8192_fsdp8", "llama3-8b", 8, dict(per_device_batch_size=2, max_target_length=8192, remat_policy="full",
                                                        ici_fsdp_parallelism=8), "headline configuration, one node"),
    Recipe("llama3_8b_8192_fsdp8_save_qkv", "llama3-8b", 8, dict(per_device_batch_size=2, max_target_length=8192, remat_policy="save_qkv_proj",
                                                                 ici_fsdp_parallelism=8), "less recompute: 180 GB of HBM leaves room"),
    Recipe("llama3_8b_8192_fp8_fsdp8", "llama3-8b", 8, dict(per_device_batch_size=2, max_target_length=8192, remat_policy="full",
                                                            ici_fsdp_parallelism=8, quantization="fp8"), "fp8 linear layers"),
    Recipe("llama3_70b_8192_fsdp4_tp2", "llama3-70b", 8, dict(per_device_batch_size=1, max_target_length=8192, remat_policy="full",
                                                              ici_fsdp_parallelism=4, ici_tensor_parallelism=2, weight_dtype="bfloat16",
                                                              mu_dtype="bfloat16"),
           "70B on one node needs bf16 master weights and first moments to fit 180 GB per GPU"),
    Recipe("mixtral_8x7b_8192_ep8", "mixtral-8x7b", 8, dict(per_device_batch_size=2, max_target_length=8192, remat_policy="full",
                                                            ici_fsdp_parallelism=1, ici_expert_parallelism=8, weight_dtype="bfloat16"),
           "experts spread over the node, peer-memory dispatch"),
    Recipe("deepseek2_16b_4096_ep8", "deepseek2-16b", 8, dict(per_device_batch_size=4, max_target_length=4096, remat_policy="full",
                                                              ici_fsdp_parallelism=1, ici_expert_parallelism=8), "MLA + shared/routed experts"),
    Recipe("qwen3_30b_a3b_4096_ep8", "qwen3-30b-a3b", 8, dict(per_device_batch_size=4, max_target_length=4096, remat_policy="full",
                                                              ici_fsdp_parallelism=1, ici_expert_parallelism=8), "128 experts, top-8"),
    Recipe("gemma2_9b_8192_fsdp8", "gemma2-9b", 8, dict(per_device_batch_size=1, max_target_length=8192, remat_policy="full",
                                                        ici_fsdp_parallelism=8), "local/global attention pairs, soft-capped logits"),
    Recipe("llama3_8b_32k_cp4_fsdp2", "llama3-8b", 8, dict(per_device_batch_size=1, max_target_length=32768, remat_policy="full",
                                                           ici_fsdp_parallelism=2, ici_context_parallelism=4,
                                                           context_parallel_strategy="ulysses"), "long context: head/sequence all-to-all"),
]}
