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
  from ..models import families
  if c.decoder_block == "deepseek4":
    ffn_total = L * (2 * bs * d * c.num_experts + _ffn(bs, d, c.moe_mlp_dim, n_act) * c.num_experts_per_tok
                     + (_ffn(bs, d, c.moe_mlp_dim * c.shared_experts, n_act) if c.shared_experts > 0 else 0))
    weight, attention = _deepseek4(c, B, S, ffn_total, 2 * bs * d * c.vocab_size)
  else:
    # walk the layer plans: every block contributes its own projections, feed-forward kind and attention pattern, so families with
    # mixed layers (local / global, chunked, dense / routed, gated-delta) are counted layer by layer
    weight, attention = 2 * bs * d * c.vocab_size, 0.0
    for plan in families.layer_plans(c):
      for bp in plan.blocks:
        w_, a_ = _block(c, bp, B, S, n_act)
        weight += w_
        attention += a_
  g = c.gradient_accumulation_steps
  return 3 * (weight + attention) * g / 1e12, 3 * weight * g / 1e12, 3 * attention * g / 1e12


def _block(c, bp, B, S, n_act):
  """(weight FLOPs, attention FLOPs) of one block, forward."""
  bs, d = B * S, c.emb_dim
  if bp.attention == "mla":
    qk = c.qk_nope_head_dim + c.qk_rope_head_dim
    if c.q_lora_rank > 0:
      q = 2 * bs * (d * c.q_lora_rank + c.q_lora_rank * c.num_query_heads * qk)
    else:
      q = 2 * bs * d * c.num_query_heads * qk
    kv = 2 * bs * (d * (c.kv_lora_rank + c.qk_rope_head_dim) + c.kv_lora_rank * c.num_query_heads * (c.qk_nope_head_dim + c.v_head_dim))
    proj_w = q + kv + 2 * bs * d * c.num_query_heads * c.v_head_dim
    attn = 2 * bs * S * c.num_query_heads * (qk + c.v_head_dim) / 2
  elif bp.attention == "gdn":
    # gated delta network (src/maxtext/utils/maxtext_utils.py:772-820): projections, short convolution, 8 FLOPs per state element and token
    kd, vd = c.gdn_num_key_heads * c.gdn_key_head_dim, c.gdn_num_value_heads * c.gdn_value_head_dim
    proj_w = 2 * bs * d * (2 * kd + 2 * vd + 2 * c.gdn_num_value_heads) + 2 * bs * d * vd + 2 * bs * c.gdn_conv_kernel_dim * (2 * kd + vd)
    attn = bs * c.gdn_num_value_heads * c.gdn_key_head_dim * c.gdn_value_head_dim * 8
  else:
    dh = int(bp.head_dim or c.head_dim)
    hkv = int(bp.kv_heads or c.num_kv_heads)
    n_kv_proj = 1 if bp.share_kv else 2
    proj_w = 2 * bs * d * (c.num_query_heads + n_kv_proj * hkv) * dh + 2 * bs * d * c.num_query_heads * dh
    if bp.window and bp.window > 0:
      w = min(int(bp.window), S)
      attn = 4 * B * (S * w - 0.5 * w * w) * c.num_query_heads * dh              # causal band of width w
    elif bp.chunk and 0 < bp.chunk < S:
      n, rem = divmod(S, int(bp.chunk))
      attn = 4 * B * (n * bp.chunk ** 2 + rem ** 2) * c.num_query_heads * dh / 2   # causal triangles of the chunks
    else:
      attn = 4 * bs * S * c.num_query_heads * dh / 2
  if bp.mlp in ("moe", "moe_shared", "gemma4_moe"):
    ffn = 2 * bs * d * c.num_experts + _ffn(bs, d, c.moe_mlp_dim, n_act) * c.num_experts_per_tok
    if bp.mlp == "moe_shared" and c.shared_experts > 0:
      ffn += _ffn(bs, d, c.moe_mlp_dim * c.shared_experts, n_act)
    if bp.mlp == "gemma4_moe":
      ffn += _ffn(bs, d, c.mlp_dim, n_act)                                         # the dense MLP next to the routed experts
  else:
    ffn = _ffn(bs, d, int(bp.mlp_hidden or c.mlp_dim), n_act)
  return proj_w + ffn, attn


def tokens_per_device(c, batch_per_device: float | None = None) -> float:
  B = float(batch_per_device if batch_per_device is not None else c.per_device_batch_size)
  return B * c.max_target_length * c.gradient_accumulation_steps


def prefill_tflops_per_device(c, num_parameters: int, prefill_length: int, num_devices: int = 1) -> tuple[float, float, float]:
  """(total, weight, causal attention) TFLOPs of one prefill pass (src/maxtext/utils/maxtext_utils.py:1396-1420): two FLOPs per
  parameter and token, plus the causal half of the attention products."""
  weight = 2.0 * num_parameters * prefill_length / num_devices / 1e12
  attention = 4.0 * c.num_query_heads * c.num_decoder_layers * c.head_dim * prefill_length ** 2 / num_devices / 1e12 / 2
  return weight + attention, weight, attention
