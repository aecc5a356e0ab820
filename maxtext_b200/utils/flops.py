"""Model-FLOPs accounting used for TFLOP/s and MFU.

The formula is the one MaxText reports with (src/maxtext/utils/maxtext_utils.py:1149-1392): per device
and per step, forward FLOPs of every matmul family (qkv, attention with the causal half, output
projection, gated FFN or routed experts counted by active experts, un-embedding), times 3 for
forward + backward, times gradient_accumulation_steps. Rematerialisation recompute is not counted.
"""
from __future__ import annotations


def _ffn(bs, d, f, n_act=2):
  return 2 * bs * d * f * n_act + 2 * bs * f * d


def training_tflops_per_device(c, batch_per_device: float | None = None) -> tuple[float, float, float]:
  """Returns (total, learnable-weight, attention) TFLOPs per device per optimizer step."""
  B = float(batch_per_device if batch_per_device is not None else c.per_device_batch_size)
  S = c.max_target_length
  bs = B * S
  d, L = c.emb_dim, c.num_decoder_layers
  n_act = len(c.mlp_activations)
  if c.attention_type == "mla":
    qk = c.qk_nope_head_dim + c.qk_rope_head_dim
    if c.q_lora_rank > 0:
      q = 2 * bs * (d * c.q_lora_rank + c.q_lora_rank * c.num_query_heads * qk)
    else:
      q = 2 * bs * d * c.num_query_heads * qk
    kv = 2 * bs * (d * (c.kv_lora_rank + c.qk_rope_head_dim) + c.kv_lora_rank * c.num_query_heads * (c.qk_nope_head_dim + c.v_head_dim))
    qkv = q + kv
    attn = 2 * bs * S * c.num_query_heads * (qk + c.v_head_dim) / 2
    proj = 2 * bs * d * c.num_query_heads * c.v_head_dim
  else:
    qkv = 2 * bs * d * (c.num_query_heads + 2 * c.num_kv_heads) * c.head_dim
    attn = 4 * bs * S * c.num_query_heads * c.head_dim / 2
    proj = 2 * bs * d * c.num_query_heads * c.head_dim
  if c.num_experts > 1:
    gate = 2 * bs * d * c.num_experts
    moe = gate + _ffn(bs, d, c.moe_mlp_dim, n_act) * c.num_experts_per_tok
    if c.shared_experts > 0:
      moe += _ffn(bs, d, c.moe_mlp_dim * c.shared_experts, n_act)
    nd = c.first_num_dense_layers if c.decoder_block == "deepseek" else 0
    ffn_total = nd * _ffn(bs, d, c.mlp_dim, n_act) + (L - nd) * moe
  else:
    ffn_total = L * _ffn(bs, d, c.mlp_dim, n_act)
  blocks = 2 if c.decoder_block == "gemma2" else 1
  weight = (ffn_total + L * (qkv + proj)) * blocks + 2 * bs * d * c.vocab_size
  attention = L * attn * blocks
  g = c.gradient_accumulation_steps
  return 3 * (weight + attention) * g / 1e12, 3 * weight * g / 1e12, 3 * attention * g / 1e12


def tokens_per_device(c, batch_per_device: float | None = None) -> float:
  B = float(batch_per_device if batch_per_device is not None else c.per_device_batch_size)
  return B * c.max_target_length * c.gradient_accumulation_steps
