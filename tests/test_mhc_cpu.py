"""Manifold-constrained hyper-connections: properties of the three maps, the layer against a direct fp32 restatement of the
published formula, and a DeepSeek-style model that trains with k = 4 residual streams."""
import math

import torch

from helpers import batch_of, make_engine, tiny_config


def test_sinkhorn_is_doubly_stochastic_and_lite_map_is_a_mixture_of_permutations():
  from maxtext_b200.layers import mhc
  torch.manual_seed(0)
  t = mhc.sinkhorn(torch.randn(3, 5, 4, 4), 20)
  assert torch.allclose(t.sum(-1), torch.ones(3, 5, 4), atol=5e-3) and torch.allclose(t.sum(-2), torch.ones(3, 5, 4), atol=5e-3)
  P = mhc.permutation_matrices(3)
  assert P.shape == (6, 3, 3) and torch.equal(P.sum(-1), torch.ones(6, 3)) and torch.equal(P.sum(-2), torch.ones(6, 3))
  assert len({tuple(p.flatten().tolist()) for p in P}) == 6


def _layer(lite):
  from maxtext_b200.layers import blocks as L, mhc
  cfg = tiny_config("deepseek2-16b", ["mhc_expansion_rate=3", f"enable_mhc_lite={'true' if lite else 'false'}", "sinkhorn_iterations=8"])
  b = L.Builder(cfg, "u", None, None)
  hc = mhc.HyperConnection(b, cfg, "mhc_attention", 16)
  g = torch.Generator().manual_seed(1)
  for p in b.params:
    p.data = torch.randn(p.shape, generator=g) * (0.3 if len(p.shape) > 1 else 0.5)
  return cfg, hc


def test_layer_matches_direct_restatement():
  from maxtext_b200.layers import mhc
  for lite in (False, True):
    cfg, hc = _layer(lite)
    k, D = 3, 16
    torch.manual_seed(2)
    x = torch.randn(2, 5, k, D)
    branch = torch.nn.Linear(D, D)
    with torch.no_grad():
      got = hc(None, branch, x)
      # direct restatement, token by token
      flat = x.reshape(2, 5, k * D)
      nx = flat * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + cfg.normalization_layer_epsilon) * hc.norm.scale.data
      want = torch.empty_like(x)
      for bi in range(2):
        for si in range(5):
          v = nx[bi, si]
          pre = torch.sigmoid(hc.pre_alpha_scale.data * (hc.pre_alpha.data @ v) + hc.pre_beta.data) + 1e-6
          post = 2 * torch.sigmoid(hc.post_alpha_scale.data * (hc.post_alpha.data @ v) + hc.post_beta.data)
          hr = hc.res_alpha_scale.data * (hc.res_alpha.data @ v)
          if lite:
            w = torch.softmax(hr + hc.res_beta.data, -1)
            res = (w[:, None, None] * mhc.permutation_matrices(k)).sum(0)
          else:
            res = mhc.sinkhorn((hr.reshape(k, k) + hc.res_beta.data)[None], 8)[0]
          inp = (pre[:, None] * x[bi, si]).sum(0)
          out = branch(inp)
          want[bi, si] = res.t() @ x[bi, si] + post[:, None] * out[None]
    assert torch.allclose(got, want, atol=1e-4), (lite, float((got - want).abs().max()))


def test_deepseek_with_four_streams_trains_and_round_trips_parameter_names():
  cfg = tiny_config("deepseek2-16b", ["mhc_expansion_rate=4", "steps=6"])
  eng = make_engine(cfg)
  names = [p.name for u in eng.store.units.values() for p in u.params]
  assert any(n.endswith("mhc_attention/res_alpha") for n in names) and any(n.endswith("mhc_mlp/mhc_norm/scale") for n in names)
  res = [p for u in eng.store.units.values() for p in u.params if p.name.endswith("mhc_attention/res_alpha")][0]
  assert res.pdef.ref_shape == (4 * cfg.emb_dim, 16)
  batch = batch_of(cfg)
  losses = [float(eng.train_step(batch)["learning/loss"]) for _ in range(6)]
  assert all(math.isfinite(v) for v in losses) and losses[-1] < losses[0]
  # the plain forward sees the same model: logits have the vocabulary width, one row per token
  with torch.no_grad():
    logits = eng.model.forward(batch["inputs"])
  assert logits.shape == (*batch["inputs"].shape, cfg.vocab_size)


def test_hyper_head_collapses_streams():
  from maxtext_b200.layers import blocks as L, mhc
  cfg = tiny_config("deepseek2-16b", ["mhc_expansion_rate=4"])
  b = L.Builder(cfg, "u", None, None)
  head = mhc.HyperHead(b, cfg)
  for p in b.params:
    p.data = torch.randn(p.shape) * 0.1
  x = torch.randn(2, 3, 4, cfg.emb_dim)
  with torch.no_grad():
    y = head(x)
  assert y.shape == (2, 3, cfg.emb_dim)
  flat = x.reshape(2, 3, -1)
  flat = flat * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + 1e-6)
  pre = torch.sigmoid(flat @ head.hc_fn.data.t() * head.hc_scale.data + head.hc_base.data) + 1e-6
  assert torch.allclose(y, (pre[..., None] * x).sum(2), atol=1e-5)
