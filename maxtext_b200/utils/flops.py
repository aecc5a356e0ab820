"""Model-FLOPs accounting used for TFLOP/s and MFU.

The formula is the one MaxText reports with (src/maxtext/utils/maxtext_utils.py:1149-1392): per device
and per step, forward FLOPs of every matmul family (qkv, attention with the causal half, output
projection, gated FFN or routed experts counted by active experts, un-embedding), times 3 for
forward + backward, times gradient_accumulation_steps. Rematerialisation recompute is not counted.
"""
from __future__ import annotations


def _ffn(bs, d, f, n_act=2):
  return 2 * bs * d * f * n_act + 2 * bs * f * d


def _mhc(bs, d, k):
  """One hyper-connection wrapper: the [k*D -> k], [k*D -> k], [k*D -> k*k] read-outs, the stream contraction, the write-back and
  the k x k stream mix (src/maxtext/utils/maxtext_utils.py:992-1009)."""
  return 2 * bs * (k * d) * k * 2 + 2 * bs * (k * d) * k * k + 2 * bs * k * d + bs * k * d + 2 * bs * k * k * d


def _deepseek4(c, B, S, ffn_total, unembed):
  """DeepSeek-V4 (src/maxtext/utils/maxtext_utils.py:1012-1147): low-rank query, one key = value head, grouped low-rank output map;
  per layer kind: the sliding-window triangle (S * W - W^2 / 2 pairs), plus S / 128 pooled entries for the heavy kind, plus for the
  sparse kind the indexer (projections, scoring and head reduction over S / 4 entries at the causal half, its own poolers) and
  attention over the chosen top-k entries; the poolers and two hyper-connection wrappers per layer count as weights."""
  bs, d, H, dh = B * S, c.emb_dim, c.num_query_heads, c.head_dim
  ratios = [int(r) for r in (c.compress_ratios or [])][:c.num_decoder_layers]
  n_win, n_hca, n_csa = (ratios.count(0), ratios.count(128), ratios.count(4)) if ratios else (2, 20, 21)
  L = c.num_decoder_layers
  q = 2 * bs * (d * c.q_lora_rank + c.q_lora_rank * H * dh)
  kv = 2 * bs * d * c.num_kv_heads * dh
  per_group = H * dh // c.o_groups
  out = 2 * bs * c.o_groups * per_group * c.o_lora_rank + 2 * bs * c.o_groups * c.o_lora_rank * d
  W = c.sliding_window_size
  window = 4 * B * (S * W - 0.5 * W * W) * H * dh
  hca = window + 2 * bs * (S / 128) * H * dh
  n4 = S // 4
  k_sel = min(int(c.indexer_topk), n4)
  frac = (k_sel / n4) - 0.5 * (k_sel / n4) ** 2 if n4 else 0.0
  indexer = (2 * bs * (c.q_lora_rank * c.indexer_n_heads * c.indexer_head_dim + d * c.indexer_n_heads)
             + bs * (S / 4) * c.indexer_n_heads * c.indexer_head_dim + bs * (S / 4) * c.indexer_n_heads
             + 4 * bs * d * 2 * c.indexer_head_dim)
  csa = window + 4 * B * S * (S / 4) * H * dh * frac + indexer
  attention = n_win * window + n_hca * hca + n_csa * csa
  k = int(getattr(c, "mhc_expansion_rate", 1) or 1)
  weight = (L * (q + kv + out) + (2 * L * _mhc(bs, d, k) if k > 1 else 0) + n_hca * 4 * bs * d * dh + n_csa * 4 * bs * d * 2 * dh
            + ffn_total + unembed)
  return weight, attention


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
  if c.decoder_block == "deepseek4":
    weight, attention = _deepseek4(c, B, S, ffn_total, 2 * bs * d * c.vocab_size)
    g = c.gradient_accumulation_steps
    return 3 * (weight + attention) * g / 1e12, 3 * weight * g / 1e12, 3 * attention * g / 1e12
  blocks = 2 if c.decoder_block == "gemma2" else 1
  weight = (ffn_total + L * (qkv + proj)) * blocks + 2 * bs * d * c.vocab_size
  attention = L * attn * blocks
  g = c.gradient_accumulation_steps
  return 3 * (weight + attention) * g / 1e12, 3 * weight * g / 1e12, 3 * attention * g / 1e12


def tokens_per_device(c, batch_per_device: float | None = None) -> float:
  B = float(batch_per_device if batch_per_device is not None else c.per_device_batch_size)
  return B * c.max_target_length * c.gradient_accumulation_steps
