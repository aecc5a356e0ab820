"""DeepSeek-V4: compressed attention against a per-query restatement, causality of the whole model, training."""
import math

import pytest
import torch

from helpers import tiny_config

V4 = ["base_num_decoder_layers=5", "compress_ratios=[0,4,8,8,4]", "first_num_hash_layers=1", "tokenizer_type=byte", "max_target_length=64",
      "vocab_size=256", "sliding_window_size=8", "qk_rope_head_dim=8", "indexer_head_dim=16", "indexer_topk=3", "dtype=float32",
      "per_device_batch_size=2", "learning_rate=2e-3"]


def _layer(ratio, extra=()):
  from maxtext_b200.layers import blocks as L
  from maxtext_b200.layers.attention_compressed import CompressedAttention
  from maxtext_b200.layers.context import LayerCtx
  cfg = tiny_config("deepseek4-tiny", V4 + list(extra))
  b = L.Builder(cfg, "u", None, None)
  att = CompressedAttention(b, cfg, "self_attention", ratio, int(cfg.sliding_window_size))
  g = torch.Generator().manual_seed(ratio + 1)
  for p in b.params:
    p.data = torch.randn(p.shape, generator=g) * (0.3 if p.data is None or p.pdef.init != "ones" else 0.0) + (1.0 if p.pdef.init == "ones" else 0.0)
  return cfg, att, LayerCtx


def test_pair_rotation_is_a_rotation_and_reverses():
  from maxtext_b200.layers.attention_compressed import rope_pairs
  x = torch.randn(2, 5, 3, 16)
  pos = torch.arange(5)[None].expand(2, 5) * 7
  y = rope_pairs(x, pos, 10000.0, 8)
  assert torch.equal(y[..., :8], x[..., :8])
  assert torch.allclose(y.pow(2).sum(-1), x.pow(2).sum(-1), atol=1e-5)
  assert torch.allclose(rope_pairs(y, pos, 10000.0, 8, reverse=True), x, atol=1e-5)
  # pair (2i, 2i + 1) turns by pos * theta^(-2i / dim), like a complex number
  z = torch.view_as_complex(x[..., 8:].reshape(2, 5, 3, 4, 2).contiguous())
  ang = pos[..., None].float() * 10000.0 ** (-2.0 * torch.arange(4) / 8)
  want = torch.view_as_real(z * torch.polar(torch.ones_like(ang), ang)[:, :, None]).flatten(-2)
  assert torch.allclose(y[..., 8:], want, atol=1e-5)
  # a 3-D input (pooled entries) takes the same path
  assert torch.allclose(rope_pairs(x[:, :, 0], pos, 10000.0, 8), y[:, :, 0], atol=1e-6)


def _naive_pool(pool, x, positions, theta, rope_dim, overlap):
  from maxtext_b200.layers.attention_compressed import rope_pairs
  from maxtext_b200.ops import functional as F
  B, S, _ = x.shape
  r, d = pool.r, pool.dim
  kv = F.linear(x, pool.kv_proj).float()
  gate = F.linear(x, pool.gate_proj).float()
  out = torch.zeros(B, S // r, d)
  for b in range(B):
    for j in range(S // r):
      rows, gates = [], []
      if overlap and j > 0 and int(positions[b, j * r]) == int(positions[b, (j - 1) * r]) + r:
        for t in range(r):
          rows.append(kv[b, (j - 1) * r + t, :d])
          gates.append(gate[b, (j - 1) * r + t, :d] + pool.position_bias.leaf()[t, :d])
      lo = d if overlap else 0
      for t in range(r):
        rows.append(kv[b, j * r + t, lo:lo + d])
        gates.append(gate[b, j * r + t, lo:lo + d] + pool.position_bias.leaf()[t, lo:lo + d])
      w = torch.softmax(torch.stack(gates), 0)
      out[b, j] = (torch.stack(rows) * w).sum(0)
  out = pool.kv_norm(out)
  return rope_pairs(out, positions[:, :(S // r) * r:r], theta, rope_dim)


def _naive_layer(att, x, positions, seg):
  """One query at a time: window keys, visible pooled entries (top-k for the sparse kind), sink in the denominator."""
  from maxtext_b200.layers.attention_compressed import rope_pairs
  from maxtext_b200.ops import functional as F
  B, S, _ = x.shape
  q, kv, qn = att.project(x, positions)
  r = att.r
  ent = None
  if r:
    ent = _naive_pool(att.hca if att.hca is not None else att.csa, x, positions, att.theta, att.rope_dim, att.hca is None)
    if att.indexer is not None:
      sc = att.indexer.scores(x, qn, positions, att.theta, att.rope_dim)
  out = torch.zeros(B, S, att.H, att.dh)
  for b in range(B):
    for s in range(S):
      keys = []
      for t in range(S):
        ok = 0 <= int(positions[b, s]) - int(positions[b, t]) < att.window
        if seg is not None:
          ok = ok and int(seg[b, s]) == int(seg[b, t]) and int(seg[b, t]) != 0
        if ok:
          keys.append(kv[b, t])
      if r:
        vis = []
        for j in range(S // r):
          ok = int(positions[b, j * r]) + r <= int(positions[b, s]) + 1
          if seg is not None:
            blk = seg[b, j * r:(j + 1) * r]
            ok = ok and bool((blk == blk[0]).all()) and int(blk[0]) == int(seg[b, s])
          if ok:
            vis.append(j)
        if att.indexer is not None and len(vis) > att.indexer.topk:
          vis = sorted(vis, key=lambda j: -float(sc[b, s, j]))[:att.indexer.topk]
        keys += [ent[b, j] for j in vis]
      if not keys:
        continue
      K = torch.stack(keys).float()
      logits = torch.einsum("hd,kd->hk", q[b, s].float(), K)
      full = torch.cat([logits, att.sinks.leaf().float()[:, None]], 1)
      p = torch.softmax(full, -1)[:, :-1]
      out[b, s] = p @ K
  out = rope_pairs(out, positions, att.theta, att.rope_dim, reverse=True)
  grouped = torch.einsum("bsgi,gio->bsgo", out.reshape(B, S, att.g, att.per_group), att.o_a.leaf())
  return F.linear(grouped.reshape(B, S, -1), att.o_b)


@pytest.mark.parametrize("ratio", [0, 4, 8])
@pytest.mark.parametrize("packed", [False, True])
def test_layer_matches_per_query_restatement(ratio, packed):
  cfg, att, LayerCtx = _layer(ratio)
  B, S = 2, 40
  # fixed inputs: with two index scores within rounding of each other the vectorised top-k and the per-query sort could pick
  # different blocks, which is a legitimate tie, not an error
  x = torch.randn(B, S, cfg.emb_dim, generator=torch.Generator().manual_seed(100 + ratio + int(packed)))
  if packed:
    # two documents per row; the boundary (18) cuts through a block of 4 and of 8
    seg = torch.cat([torch.ones(B, 18), torch.full((B, 22), 2.0)], 1).long()
    pos = torch.cat([torch.arange(18), torch.arange(22)])[None].expand(B, S).contiguous()
  else:
    seg, pos = None, torch.arange(S)[None].expand(B, S).contiguous()
  ctx = LayerCtx(cfg, pos, seg)
  with torch.no_grad():
    got = att(x, ctx)
    want = _naive_layer(att, x, pos, seg)
  assert torch.allclose(got, want, atol=2e-4, rtol=2e-4), float((got - want).abs().max())


def test_query_chunking_does_not_change_values_or_gradients(monkeypatch):
  from maxtext_b200.layers import attention_compressed as ac
  cfg, att, LayerCtx = _layer(4)
  x = torch.randn(1, 48, cfg.emb_dim, generator=torch.Generator().manual_seed(7)).requires_grad_(True)
  pos = torch.arange(48)[None]
  a = att(x, LayerCtx(cfg, pos, None))
  ga, = torch.autograd.grad(a.sum(), x)
  monkeypatch.setattr(ac, "Q_CHUNK", 16)
  b = att(x, LayerCtx(cfg, pos, None))
  gb, = torch.autograd.grad(b.sum(), x)
  assert torch.allclose(a, b, atol=1e-5) and torch.allclose(ga, gb, atol=1e-5)


def test_sparse_layer_keeps_at_most_topk_blocks():
  cfg, att, LayerCtx = _layer(4)
  x = torch.randn(2, 64, cfg.emb_dim, generator=torch.Generator().manual_seed(8))
  pos = torch.arange(64)[None].expand(2, 64)
  with torch.no_grad():
    _, _, qn = att.project(x, pos)
    ent, allowed = att.pooled(x, qn, pos, None)
  assert ent.shape == (2, 16, cfg.head_dim) and allowed.shape == (2, 64, 16)
  assert int(allowed.sum(-1).max()) == 3 and not allowed[:, :3].any()          # nothing is visible before the first block closes
  assert allowed[:, 3, 0].all()


def _model(extra=()):
  from maxtext_b200.models.transformer import Transformer
  cfg = tiny_config("deepseek4-tiny", V4 + list(extra))
  m = Transformer(cfg, None, torch.device("cpu"))
  m.store.initialize(seed=0)
  return cfg, m


def test_model_is_causal_through_window_pooled_entries_and_hyper_connections():
  cfg, m = _model()
  names = {p.pdef.name.split("/")[0] for p in m.all_params()}
  assert {"layers_0", "scanned_blocks_0", "scanned_blocks_1"} <= names
  assert any("hc_head" in p.pdef.name for p in m.all_params()) and any("tid2eid" in p.pdef.name or "hash" in p.pdef.name.lower() for p in m.layers[0].params)
  t = torch.randint(1, 200, (2, 64))
  with torch.no_grad():
    a = m.forward(t)
    t2 = t.clone()
    t2[:, 40] = (t2[:, 40] + 1) % 200
    b = m.forward(t2)
  assert torch.isfinite(a).all()
  assert torch.allclose(a[:, :40], b[:, :40], atol=1e-5) and not torch.allclose(a[:, 40:], b[:, 40:])
  # far beyond the window the change is still felt: it travels through the pooled entries
  assert not torch.allclose(a[:, 60:], b[:, 60:], atol=1e-6)


def test_engine_trains_deepseek4():
  from maxtext_b200.input_pipeline.synthetic import SyntheticDataIterator
  from maxtext_b200.train.engine import TrainEngine
  cfg = tiny_config("deepseek4-tiny", V4)
  eng = TrainEngine(cfg, None, torch.device("cpu"))
  batch = next(SyntheticDataIterator(cfg, pin=False))
  losses = [float(eng.train_step(dict(batch))["learning/loss"]) for _ in range(5)]
  assert all(math.isfinite(v) for v in losses) and losses[-1] < losses[0], losses


def test_sqrt_softplus_router_weights_are_positive_and_normalised():
  from maxtext_b200.layers import blocks as L
  from maxtext_b200.layers import moe as M
  cfg = tiny_config("deepseek4-tiny", V4)
  b = L.Builder(cfg, "u", None, None)
  moe = M.RoutedMoE(b, cfg, "MoeBlock_0", deepseek_style=True)
  g = torch.Generator().manual_seed(0)
  for p in b.params:
    p.data = torch.randn(p.shape, generator=g) * 0.5
  x = torch.randn(2, 16, cfg.emb_dim)
  x2 = x.reshape(-1, cfg.emb_dim)
  logits = x2 @ moe.gate.data.t()
  with torch.no_grad():
    wts, idx, _ = moe.route(x2, 2, 16, None)
  assert (wts > 0).all()
  assert torch.allclose(wts.sum(-1), torch.full((32,), float(cfg.routed_scaling_factor)), atol=1e-5)
  want = torch.sqrt(torch.nn.functional.softplus(logits.float())) + moe.gate_bias.data.float()
  assert torch.equal(idx.sort(-1).values, want.topk(int(cfg.num_experts_per_tok), -1).indices.sort(-1).values)


def test_flops_accounting_counts_each_layer_kind():
  from maxtext_b200.utils import flops
  base = V4 + ["max_target_length=1024", "per_device_batch_size=1", "sliding_window_size=128", "indexer_topk=16", "mhc_expansion_rate=1"]
  def att(ratios):
    cfg = tiny_config("deepseek4-tiny", [e for e in base if not e.startswith(("compress_ratios", "base_num_decoder_layers", "first_num_hash"))] +
                      [f"compress_ratios={ratios}", f"base_num_decoder_layers={len(ratios)}", "first_num_hash_layers=1"])
    return cfg, flops.training_tflops_per_device(cfg)
  cfg, (t0, w0, a0) = att([0, 0, 0])
  B, S, W, H, dh = 1, 1024, 128, cfg.num_query_heads, cfg.head_dim
  window = 4 * B * (S * W - 0.5 * W * W) * H * dh
  assert abs(a0 - 3 * 3 * window / 1e12) < 1e-12 and abs(t0 - (w0 + a0)) < 1e-12
  _, (_, w1, a1) = att([0, 128, 128])
  assert abs((a1 - a0) - 3 * 2 * (2 * B * S * (S / 128) * H * dh) / 1e12) < 1e-12          # two heavy layers add S / 128 entries each
  assert abs((w1 - w0) - 3 * 2 * (4 * B * S * cfg.emb_dim * dh) / 1e12) < 1e-12            # and their kv / gate poolers
  _, (_, w2, a2) = att([0, 4, 4])
  assert a2 > a0 and w2 > w1                                                                 # sparse layers: indexer + wider poolers
