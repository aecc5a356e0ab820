"""Sparse-attention indexer of DeepSeek-V3.2 (src/maxtext/layers/attention_mla.py:84-436) and its training loss
(src/maxtext/layers/attention_mla.py:1117-1229).

For every query the indexer scores all keys with a small multi-query ReLU attention,

  score[t, s] = sum_h  w[t, h] * relu(q[t, h, :] . k[s, :]),   w = weights_proj(x) * n_heads^-1/2 * head_dim^-1/2

keeps the `indexer_topk` best keys among those the attention mask allows, and hands the main attention a mask restricted to
them. It reads detached inputs (the language-model loss never reaches its weights); it learns from a KL term that pulls
softmax(score) towards the head-summed, L1-normalised attention probabilities of the main model. Sequences no longer than
`indexer_topk` are passed through unmasked.
"""
from __future__ import annotations

import torch

from ..ops import functional as F
from ..ops import reference as ref
from . import blocks as L


class Indexer:
  def __init__(self, b: L.Builder, config, rope_inv_ts, name="indexer"):
    c = config
    assert c.q_lora_rank > 0, "use_indexer needs the latent query (q_lora_rank > 0)"
    self.c = c
    self.h, self.d, self.topk, self.rope_d = int(c.indexer_n_heads), int(c.indexer_head_dim), int(c.indexer_topk), int(c.qk_rope_head_dim)
    self.inv_ts = rope_inv_ts
    ib = b.sub(name)
    self.wq_b = ib.sub("wq_b").linear("kernel", (c.q_lora_rank,), (self.h, self.d), ("q_lora", "q_heads", "kv"), init="fan_in_normal")
    self.wk = ib.sub("wk").linear("kernel", (c.emb_dim,), (self.d,), ("embed", "kv"), init="fan_in_normal")
    self.k_norm = L.Norm(ib, "k_norm", self.d, 1e-6, kind="layernorm", axes=(None,))
    self.weights_proj = ib.sub("weights_proj").linear("kernel", (c.emb_dim,), (self.h,), ("embed", "q_heads"), init="fan_in_normal")
    self.exact = bool(c.indexer_mask_exact_topk)

  def _rope(self, t, positions):
    """Rotary embedding on the FIRST rope_d features, halves layout (the main MLA rotates its last features, interleaved)."""
    pe = F.rope(t[..., :self.rope_d].contiguous(), positions, self.inv_ts, False)
    return torch.cat([pe, t[..., self.rope_d:]], dim=-1)

  def scores(self, x, low_rank_q, positions):
    """x [B,S,D], low_rank_q [B,S,q_lora] -> score [B,S,S] fp32 (before any mask). Inputs are detached."""
    x, low_rank_q = x.detach(), low_rank_q.detach()
    B, S, _ = x.shape
    q = self._rope(F.linear(low_rank_q, self.wq_b).view(B, S, self.h, self.d), positions)
    k = self.k_norm(F.linear(x, self.wk))
    k = self._rope(k.view(B, S, 1, self.d), positions).view(B, S, self.d)
    w = torch.matmul(x.float(), self.weights_proj.leaf().float().t()) * (self.h ** -0.5) * (self.d ** -0.5)     # fp32, never quantised
    score = torch.zeros(B, S, S, dtype=torch.float32, device=x.device)
    step = max(1, int(getattr(self.c, "mla_qk_head_chunk_size", 0)) or self.h)      # heads per pass bound the [B,S,S,h] temporary
    kf = k.float()
    for h0 in range(0, self.h, step):
      logits = torch.relu(torch.einsum("bthd,bsd->bhts", q[:, :, h0:h0 + step].float(), kf))
      score = score + torch.einsum("bhts,bth->bts", logits, w[..., h0:h0 + step])
    return score

  def select(self, score, allowed):
    """score [B,S,S], allowed bool [B,S,S] -> bool mask of the top-k allowed keys per query (all allowed keys where a query has
    fewer than k of them). Ties at the threshold are cut in key order when `indexer_mask_exact_topk`."""
    neg = torch.finfo(torch.float32).min
    s = score.masked_fill(~allowed, neg)
    kth = s.topk(self.topk, dim=-1).values[..., -1:]
    if not self.exact:
      return (s >= kth) & allowed
    greater, equal = s > kth, s == kth
    g_rank, e_rank = greater.int().cumsum(-1), equal.int().cumsum(-1)
    kept = greater & (g_rank <= self.topk)
    room = self.topk - g_rank[..., -1:].clamp(max=self.topk)
    return (kept | (equal & (e_rank <= room))) & allowed

  def __call__(self, x, low_rank_q, positions, segment_ids):
    """-> (mask bool [B,1,S,S] or None when every key is kept, score [B,S,S] or None, allowed [B,1,S,S] or None)."""
    S = x.shape[1]
    if S <= self.topk:
      return None, None, None
    allowed = ref.attention_mask(positions, positions, segment_ids, segment_ids, True, 0, 0)
    score = self.scores(x, low_rank_q, positions)
    return self.select(score, allowed[:, 0])[:, None], score, allowed

  def loss(self, score, q, k, allowed, mask, scale_q: float = 1.0):
    """KL(target || softmax(score)) averaged over queries, times `indexer_loss_scaling_factor`. target = L1-normalised sum over
    heads of the main model's attention probabilities (q, k detached), under the sparse mask in the sparse-training stage and
    under the plain attention mask in the dense warm-up stage."""
    c = self.c
    eps = 1e-9
    sparse = bool(c.indexer_sparse_training)
    use = mask if sparse else allowed
    neg = torch.finfo(torch.float32).min
    ind = score.masked_fill(~use[:, 0], neg) if sparse else score
    ind_p = torch.softmax(ind.float(), dim=-1)
    logits = torch.einsum("bthd,bshd->bhts", q.detach().float() * scale_q, k.detach().float()).masked_fill(~use, neg)
    tgt = torch.softmax(logits, dim=-1).sum(1)
    tgt = tgt / (tgt.sum(-1, keepdim=True) + eps)
    kl = (tgt * (torch.log(tgt + eps) - torch.log(ind_p + eps))).sum(-1)
    return kl.mean() * float(c.indexer_loss_scaling_factor)
