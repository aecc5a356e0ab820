"""Engram n-gram memory: canonical ids, the multi-head hash, the layer against a direct restatement, and a model that trains."""
import math

import numpy as np
import torch

from helpers import batch_of, make_engine, tiny_config

EXTRA = ["engram_layers=[1]", "engram_vocab_bases=[50,70]", "engram_max_ngram_size=3", "engram_num_heads=2", "engram_head_dim=8",
         "engram_kernel_size=3", "tokenizer_type=byte", "vocab_size=260"]


class _Tok:
  vocab_size = 8
  words = ["Apple", " apple", "APPLE", "café", "cafe", " ", "\n\n", "x"]

  def decode(self, ids):
    return "".join(self.words[i] for i in ids)


def test_canonical_ids_merge_case_accent_and_whitespace_variants():
  from maxtext_b200.layers.engram import CompressedTokenizer, normalize_token_text
  assert normalize_token_text("  APPLE ") == "apple" and normalize_token_text("Café") == "cafe" and normalize_token_text(" ") == " "
  ct = CompressedTokenizer(_Tok())
  t = ct.table_np
  assert t[0] == t[1] == t[2] and t[3] == t[4] and t[5] == t[6] and len({t[0], t[3], t[5], t[7]}) == 4 and len(ct) == 4
  ids = torch.tensor([[0, 2, -1, 7]])
  assert ct(ids).tolist() == [[int(t[0]), int(t[0]), -1, int(t[7])]]


def test_hashes_follow_the_published_formula_with_distinct_primes():
  from maxtext_b200.layers.engram import NgramHashMapping, _is_prime
  hm = NgramHashMapping([50, 70], 3, 2, [1, 4], _Tok(), pad_id=7, seed=3)
  primes = hm.vocab_sizes(1) + hm.vocab_sizes(4)
  assert len(set(primes)) == 8 and all(_is_prime(p) for p in primes) and min(hm.vocab_sizes(1)[:2]) >= 50 and min(hm.vocab_sizes(1)[2:]) >= 70
  assert all(int(m) % 2 == 1 for m in hm.multipliers[1])
  ids = torch.tensor([[0, 3, 5, 7, 1, 4]])
  got = hm(ids)[1][0]
  c = hm.ct(ids)[0].tolist()
  m = [int(v) for v in hm.multipliers[1]]
  i32 = lambda v: ((v + 2 ** 31) % 2 ** 32) - 2 ** 31  # noqa: E731
  for t in range(6):
    prev = lambda k: c[t - k] if t - k >= 0 else hm.pad  # noqa: E731
    h2 = i32(c[t] * m[0]) ^ i32(prev(1) * m[1])
    h3 = h2 ^ i32(prev(2) * m[2])
    want = [h2 % p for p in hm.primes[1][0]] + [h3 % p for p in hm.primes[1][1]]
    assert got[t].tolist() == want, t
  assert (got >= 0).all()


def test_layer_matches_direct_restatement():
  from maxtext_b200.layers import blocks as L
  from maxtext_b200.layers.engram import Engram
  cfg = tiny_config("deepseek2-16b", EXTRA + ["mhc_expansion_rate=2"])
  b = L.Builder(cfg, "u", None, None)
  vocab = [53, 59, 71, 73]
  en = Engram(b, cfg, vocab)
  g = torch.Generator().manual_seed(0)
  for p in b.params:
    p.data = torch.randn(p.shape, generator=g) * 0.3
  B, S, G, D = 1, 7, 2, cfg.emb_dim
  h = torch.randn(B, S, G, D, generator=g)
  ids = torch.stack([torch.randint(0, v, (B, S), generator=g) for v in vocab], -1)
  with torch.no_grad():
    got = en(h, ids)
    off = np.cumsum([0] + vocab[:-1])
    e = torch.cat([en.table.data[ids[..., i] + int(off[i])] for i in range(4)], -1)               # [B,S,E]
    rms = lambda x, s: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.normalization_layer_epsilon) * s  # noqa: E731
    key = rms((e @ en.key_proj.data.t()).view(B, S, G, D) + en.key_bias.data, en.k_scale.data)
    q = rms(h, en.q_scale.data)
    gate = (q * key).sum(-1) / math.sqrt(D)
    gate = torch.sigmoid(gate.abs().clamp(min=1e-6).sqrt() * gate.sign())
    v = gate[..., None] * (e @ en.value_proj.data.t() + en.value_bias.data)[:, :, None]
    xn = rms(v, en.conv_scale.data).reshape(B, S, G * D)
    w = en.conv_kernel.data.reshape(3, G * D)
    y = torch.zeros_like(xn)
    for t in range(S):
      for j in range(3):
        src = t - (2 - j) * 3                                                                        # dilation = max n-gram size
        if src >= 0:
          y[:, t] += xn[:, src] * w[j]
    want = v + torch.nn.functional.silu(y).view(B, S, G, D)
  assert torch.allclose(got, want, atol=1e-5)


def test_deepseek_with_an_engram_layer_trains():
  cfg = tiny_config("deepseek2-16b", EXTRA + ["steps=5"])
  eng = make_engine(cfg)
  names = [p.name for u in eng.store.units.values() for p in u.params]
  assert any("engram/multi_head_embedding/embedding" in n for n in names) and any(n.endswith("engram_layer_norm/scale") for n in names)
  # only the configured layer (global index 1 = the first MoE layer) has the memory
  assert any(n.startswith("moe_layers_0/engram") for n in names)
  assert not any(n.startswith(("dense_layers_0/engram", "moe_layers_1/engram")) for n in names)
  batch = batch_of(cfg)
  losses = [float(eng.train_step(batch)["learning/loss"]) for _ in range(5)]
  assert all(math.isfinite(v) for v in losses) and losses[-1] < losses[0]
  table = [p for u in eng.store.units.values() for p in u.params if p.name.endswith("multi_head_embedding/embedding/embedding")]
  conv = [p for u in eng.store.units.values() for p in u.params if p.name.endswith("short_conv/conv/kernel")][0]
  assert table and float(eng.store.full_master(conv).abs().max()) > 0       # the zero-initialised convolution received gradient
