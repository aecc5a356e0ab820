"""DeepSeek-V3.2 sparse-attention indexer: selection rule, gradient isolation and a model that trains with it."""
import math

import torch

from helpers import batch_of, make_engine, tiny_config

EXTRA = ["use_indexer=true", "indexer_topk=8", "indexer_n_heads=4", "indexer_head_dim=16", "indexer_loss_scaling_factor=0.1"]


def _indexer(extra=()):
  from maxtext_b200.layers import blocks as L
  from maxtext_b200.layers.indexer import Indexer
  cfg = tiny_config("deepseek3-tiny", EXTRA + list(extra))
  b = L.Builder(cfg, "u", None, None)
  inv = 1.0 / (10000.0 ** (torch.arange(0, cfg.qk_rope_head_dim, 2).float() / cfg.qk_rope_head_dim))
  ix = Indexer(b, cfg, inv)
  g = torch.Generator().manual_seed(0)
  for p in b.params:
    p.data = torch.randn(p.shape, generator=g) * 0.3
  return cfg, ix, b


def test_selection_keeps_top_k_allowed_keys_and_cuts_ties_in_key_order():
  cfg, ix, _ = _indexer()
  B, S = 2, 20
  torch.manual_seed(1)
  x, lq = torch.randn(B, S, cfg.emb_dim), torch.randn(B, S, cfg.q_lora_rank)
  pos = torch.arange(S)[None].expand(B, S)
  seg = torch.ones(B, S, dtype=torch.int32)
  seg[1, 12:] = 2
  with torch.no_grad():
    mask, score, allowed = ix(x, lq, pos, seg)
  assert mask.shape == (B, 1, S, S) and score.shape == (B, S, S)
  assert not (mask & ~allowed).any()                                        # never a key the attention mask forbids
  n_allowed = allowed[:, 0].sum(-1)
  assert torch.equal(mask[:, 0].sum(-1), n_allowed.clamp(max=8))            # exactly k, or all of them when fewer are visible
  # the kept keys are the best-scored allowed ones
  s = score.masked_fill(~allowed[:, 0], -1e30)
  best = s.topk(8, -1).indices
  for b in range(B):
    for t in range(S):
      if n_allowed[b, t] >= 8:
        assert set(best[b, t].tolist()) == set(mask[b, 0, t].nonzero().flatten().tolist())
  # ties: equal scores everywhere -> the first k allowed keys
  with torch.no_grad():
    tie = ix.select(torch.zeros(1, S, S), allowed[:1, 0])
  assert torch.equal(tie[0, 15].nonzero().flatten(), torch.arange(8))
  # short sequences pass through untouched
  with torch.no_grad():
    assert ix(x[:, :8], lq[:, :8], pos[:, :8], None) == (None, None, None)


def test_scores_follow_the_definition():
  cfg, ix, _ = _indexer()
  B, S = 1, 12
  torch.manual_seed(2)
  x, lq = torch.randn(B, S, cfg.emb_dim), torch.randn(B, S, cfg.q_lora_rank)
  pos = torch.zeros(B, S, dtype=torch.long)                                  # position 0: the rotation is the identity
  with torch.no_grad():
    got = ix.scores(x, lq, pos)
    q = (lq @ ix.wq_b.data.t()).view(B, S, 4, 16)
    k = torch.nn.functional.layer_norm(x @ ix.wk.data.t(), (16,), ix.k_norm.scale.data, ix.k_norm.bias.data, 1e-6)
    w = (x @ ix.weights_proj.data.t()) * (4 ** -0.5) * (16 ** -0.5)
    want = torch.einsum("btsh,bth->bts", torch.relu(torch.einsum("bthd,bsd->btsh", q, k)), w)
  assert torch.allclose(got, want, atol=1e-4)


def test_model_trains_and_the_indexer_learns_only_from_its_own_loss():
  cfg = tiny_config("deepseek3-tiny", EXTRA + ["steps=4"])
  eng = make_engine(cfg)
  batch = batch_of(cfg)
  m0 = eng.train_step(batch)
  assert math.isfinite(float(m0["learning/loss"]))
  ix = [p for u in eng.store.units.values() for p in u.params if "/indexer/" in p.name]
  assert len(ix) >= 4 * cfg.num_decoder_layers
  # with the loss switched off the indexer still masks, but nothing reaches its weights
  cfg2 = tiny_config("deepseek3-tiny", [e for e in EXTRA if not e.startswith("indexer_loss")] + ["steps=4"])
  eng2 = make_engine(cfg2)
  before = {p.name: p.data.clone() for u in eng2.store.units.values() for p in u.params if "/indexer/" in p.name and "k_norm" not in p.name}
  eng2.train_step(batch_of(cfg2))
  after = {p.name: p.data for u in eng2.store.units.values() for p in u.params if p.name in before}
  wd = 1.0 - float(cfg2.learning_rate) * float(cfg2.adam_weight_decay)
  for n, b in before.items():
    assert torch.allclose(after[n], b * wd, atol=1e-6) or torch.allclose(after[n], b, atol=1e-6), n
  # with the loss on, they move
  moved = [p for p in ix if "wq_b" in p.name]
  eng.train_step(batch)
  eng3 = make_engine(cfg)
  ref0 = {p.name: p.data.clone() for u in eng3.store.units.values() for p in u.params if "indexer/wq_b" in p.name}
  assert any(not torch.allclose(p.data, ref0[p.name], atol=1e-5) for p in moved)


def test_hash_routed_prefix_layers_pick_experts_from_the_token_table():
  """`first_num_hash_layers`: the experts of a token come from a frozen [vocab, k] table; the router supplies the weights only."""
  cfg = tiny_config("deepseek3-tiny", ["first_num_hash_layers=2", "first_num_dense_layers=0", "n_routing_groups=0", "topk_routing_group=0", "steps=3"])
  eng = make_engine(cfg)
  tabs = [p for u in eng.store.units.values() for p in u.params if p.name.endswith("tid2eid")]
  assert len(tabs) == 2 and all(p.pdef.frozen and p.pdef.shape == (cfg.vocab_size, 2) for p in tabs)       # layers 0 and 1 only
  table = (torch.arange(cfg.vocab_size)[:, None] * 3 + torch.tensor([0, 5])) % cfg.num_experts
  for p in tabs:
    eng.store.load_full(p.name, table.float())
  eng.store.sync_compute_from_master()
  moe = eng.model.layers[0].blocks[0].mlp.routed
  batch = batch_of(cfg)
  tokens = batch["inputs"]
  ctx = eng.model.make_ctx(torch.arange(tokens.shape[1])[None].expand_as(tokens), None, "train", tokens)
  x2 = torch.randn(tokens.numel(), cfg.emb_dim)
  with torch.no_grad():
    wts, idx, _ = moe.route(x2, tokens.shape[0], tokens.shape[1], ctx)
  assert torch.equal(idx, table[tokens.reshape(-1).long()])
  assert wts.shape == idx.shape and bool((wts > 0).all())
  before = eng.store.full_master(tabs[0]).clone()
  losses = [float(eng.train_step(batch)["learning/loss"]) for _ in range(3)]
  assert all(math.isfinite(v) for v in losses) and losses[-1] < losses[0]
  assert torch.equal(eng.store.full_master(tabs[0]), before)                                                 # the table is not trained
