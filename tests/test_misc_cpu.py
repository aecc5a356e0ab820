"""Schedules, FLOPs accounting, synthetic data, metric logger, op-level reference identities."""
import json
import math

import pytest
import torch

from helpers import tiny_config
from maxtext_b200.ops import reference as ref


def test_cosine_schedule_pieces():
  from maxtext_b200.optimizers.schedules import make_schedule
  c = tiny_config("llama3-8b", ["steps=120", "learning_rate_schedule_steps=100", "learning_rate=1.0", "warmup_steps_fraction=0.1",
                                "learning_rate_final_fraction=0.1"])
  s = make_schedule(c)
  assert s(0) == 0.0 and abs(s(5) - 0.5) < 1e-9 and abs(s(10) - 1.0) < 1e-9          # linear warm-up, then cosine from its step 0
  assert abs(s(99) - 0.1) < 1e-9                                                    # last cosine step reaches the final fraction
  mid = 10 + 89 / 2
  assert abs(s(int(mid)) - (0.5 * (1 + math.cos(math.pi * (int(mid) - 10) / 89)) * 0.9 + 0.1)) < 1e-9
  assert s(100) == 0.0 and s(119) == 0.0                                            # zero tail


def test_wsd_schedule():
  from maxtext_b200.optimizers.schedules import make_schedule
  c = tiny_config("llama3-8b", ["steps=100", "learning_rate=2.0", "lr_schedule_type=wsd", "warmup_steps_fraction=0.1",
                                "wsd_decay_steps_fraction=0.2", "learning_rate_final_fraction=0.5"])
  s = make_schedule(c)
  assert s(9) == pytest.approx(1.8) and s(10) == 2.0 and s(79) == 2.0 and s(99) == pytest.approx(1.0)


def test_flops_formula_llama3_8b():
  from maxtext_b200.utils import flops
  from maxtext_b200.config import pyconfig
  from helpers import BASE_YML
  c = pyconfig.initialize(["t", BASE_YML, "model_name=llama3-8b", "per_device_batch_size=2", "max_target_length=8192", "log_config=false"],
                          num_devices=1)
  total, weights, attn = flops.training_tflops_per_device(c)
  B, S, D, F, L, V, H, KV, Dh = 2, 8192, 4096, 14336, 32, 128256, 32, 8, 128
  per_layer = 2 * B * S * D * F * 3 + 2 * B * S * D * (H + 2 * KV) * Dh + 2 * B * S * D * H * Dh
  want_w = 3 * (L * per_layer + 2 * B * S * D * V) / 1e12
  want_a = 3 * L * (4 * B * S * S * H * Dh / 2) / 1e12
  assert weights == pytest.approx(want_w) and attn == pytest.approx(want_a) and total == pytest.approx(want_w + want_a)
  assert total / (B * S) * 1e3 == pytest.approx(51.5, rel=0.02)      # GFLOP per token


def test_flops_moe_counts_active_experts_only():
  from maxtext_b200.utils import flops
  a = flops.training_tflops_per_device(tiny_config("mixtral-8x7b", ["num_experts=8", "num_experts_per_tok=2"]))[0]
  b = flops.training_tflops_per_device(tiny_config("mixtral-8x7b", ["num_experts=16", "num_experts_per_tok=2"]))[0]
  assert b > a and (b - a) / a < 0.05     # only the router grows


def test_synthetic_iterator_contract():
  from maxtext_b200.input_pipeline.synthetic import SyntheticDataIterator
  c = tiny_config("llama3-8b", ["per_device_batch_size=4"])
  it = SyntheticDataIterator(c, pin=False)
  b1, b2 = next(it), next(it)
  assert b1 is b2 and b1["inputs"].shape == (4, 32)
  assert torch.equal(b1["inputs"][:, 1:], b1["targets"][:, :-1])
  assert int(b1["inputs"].max()) < c.vocab_size and (b1["inputs_segmentation"] == 1).all()
  halves = [SyntheticDataIterator(c, r, 2, pin=False).batch["inputs"] for r in (0, 1)]
  assert torch.equal(torch.cat(halves), b1["inputs"])                # ranks read disjoint rows of the same global batch


def test_metric_logger_line_file_and_nan_abort(tmp_path, capsys):
  from maxtext_b200.utils.metric_logger import MetricLogger, TrainingAborted
  c = tiny_config("llama3-8b", [f"metrics_file={tmp_path}/m.jsonl"])
  lg = MetricLogger(c)
  lg.record(0, {"learning/loss": torch.tensor(2.5), "learning/lm_loss": torch.tensor(2.5), "learning/total_weights": torch.tensor(64.)}, 0.5)
  lg.record(1, {"learning/loss": torch.tensor(float("nan")), "learning/total_weights": torch.tensor(64.)}, 0.5)   # writes step 0
  out = capsys.readouterr().out
  assert "completed step: 0, seconds: 0.500, TFLOP/s/device:" in out and "loss: 2.500" in out
  with pytest.raises(TrainingAborted):
    lg.flush()
  rows = [json.loads(l) for l in open(f"{tmp_path}/m.jsonl")]
  assert rows[0]["step"] == 0 and rows[0]["perf/step_time_seconds"] == 0.5 and math.isnan(rows[1]["learning/loss"])


def test_rope_layouts_and_inverse():
  x = torch.randn(2, 5, 3, 16)
  pos = torch.arange(5)[None].expand(2, 5)
  inv = ref.rope_inv_timescale(16, 1, 10000)
  for inter in (False, True):
    y = ref.apply_rope(x, pos, inv, inter)
    assert torch.allclose(ref.apply_rope(y, pos, inv, inter, inverse=True), x, atol=1e-5)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
  # interleaved layout == rotate-half layout applied to de-interleaved lanes
  perm = torch.cat([torch.arange(0, 16, 2), torch.arange(1, 16, 2)])
  assert torch.allclose(ref.apply_rope(x, pos, inv, True)[..., perm], ref.apply_rope(x[..., perm], pos, inv, False), atol=1e-5)
  scaled = ref.rope_inv_timescale(128, 1, 500000, rope_type="llama3.1")
  plain = ref.rope_inv_timescale(128, 1, 500000)
  assert torch.allclose(scaled[:20], plain[:20]) and torch.allclose(scaled[-1], plain[-1] / 8)


def test_cross_entropy_gradient_identity():
  lg = torch.randn(7, 50, requires_grad=True)
  tg = torch.randint(0, 50, (7,))
  w = torch.rand(7)
  loss, _ = ref.cross_entropy(lg, tg, 1e-3)
  (loss * w).sum().backward()
  assert torch.allclose(lg.grad, ref.cross_entropy_dlogits(lg.detach(), tg, w, 1e-3), atol=1e-5)


def test_adamw_matches_torch_optimizer():
  p = torch.randn(100)
  g = torch.randn(100)
  ref_p = torch.nn.Parameter(p.clone())
  opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
  m, v = torch.zeros(100), torch.zeros(100)
  q = p.clone()
  for step in (1, 2, 3):
    ref_p.grad = g.clone()
    opt.step()
    ref.adamw_step(q, g, m, v, 1e-2, 0.9, 0.95, 1e-8, 0.0, 0.1, step)
  assert torch.allclose(q, ref_p.detach(), atol=2e-5)


def test_adam_pax_matches_praxis_formula():
  """adam_pax: bias correction folded into the decays (reference optimizers.py:289-346)."""
  import torch
  from maxtext_b200.ops import functional as F
  torch.manual_seed(0)
  n, b1, b2, eps, epsr, wd, lr = 64, 0.9, 0.95, 1e-8, 1e-12, 0.1, 1e-2
  p = torch.randn(n); m = torch.zeros(n); v = torch.zeros(n)
  rp, rm, rv = p.clone(), m.clone(), v.clone()
  for step in range(1, 5):
    g = torch.randn(n)
    F.adamw_flat(p, g.clone(), m, v, None, lr, b1, b2, eps, epsr, wd, step, torch.ones(1), pax=True)
    t = float(step)
    d1 = b1 * (1 - b1 ** (t - 1)) / (1 - b1 ** t)
    d2 = b2 * (1 - b2 ** (t - 1)) / (1 - b2 ** t)
    rm = (1 - d1) * g + d1 * rm
    rv = (1 - d2) * g * g + d2 * rv
    rp = rp - lr * (rm / (torch.sqrt(rv + epsr) + eps) + wd * rp)
    assert torch.allclose(p, rp, atol=1e-6)


def test_int8_quantization_numerics_and_training():
  """quantization=int8: forward and input-gradient products on symmetric per-channel int8 operands, weight gradient in the
  compute dtype; checked against the definition and by a short training run."""
  import torch
  from helpers import tiny_config, make_engine, batch_of
  from maxtext_b200.ops import quantization as Q
  torch.manual_seed(0)
  x, w = torch.randn(12, 32), torch.randn(20, 32) * 0.3
  sx, sw = x.abs().amax(1, keepdim=True) / 127, w.abs().amax(1, keepdim=True) / 127
  want = (torch.round(x / sx).clamp(-127, 127) * sx) @ (torch.round(w / sw).clamp(-127, 127) * sw).t()
  got = Q.int8_linear_fwd(x, w)
  assert (got - want).abs().max() < 1e-4 and 1e-4 < (got - x @ w.t()).abs().max() < 0.2      # quantised, and close to the exact product
  dy = torch.randn(12, 20)
  dx = Q.int8_linear_dx(dy, w)
  assert (dx - dy @ w).abs().max() < 0.3 and (dx - dy @ w).abs().max() > 1e-5
  try:
    eng = make_engine(tiny_config("llama3-8b", ["quantization=int8"]))
    assert Q.mode() == "int8"
    b = batch_of(eng.config)
    losses = [float(eng.train_step(b)["learning/loss"]) for _ in range(5)]
    assert losses[-1] < losses[0], losses
    ref = make_engine(tiny_config("llama3-8b"))          # resets the mode
    assert Q.mode() == ""
    l0 = float(ref.train_step(b)["learning/loss"])
    assert abs(l0 - losses[0]) < 0.05 and l0 != losses[0]
  finally:
    Q.set_mode("")


def test_muon_newton_schulz_and_training():
  import torch
  from helpers import tiny_config, make_engine, batch_of
  from maxtext_b200.optimizers.muon import newton_schulz
  torch.manual_seed(0)
  for shape in ((32, 64), (64, 32), (3, 16, 24)):
    o = newton_schulz(torch.randn(*shape), steps=8)
    sv = torch.linalg.svdvals(o)
    assert o.shape == shape and float(sv.max()) < 1.3 and float(sv.min()) > 0.5, (shape, sv.min(), sv.max())
  eng = make_engine(tiny_config("llama3-8b", ["opt_type=muon"]))
  b = batch_of(eng.config)
  losses = [float(eng.train_step(b)["learning/loss"]) for _ in range(5)]
  assert losses[-1] < losses[0], losses


def test_moe_capacity_factor_drops_overflow_and_random_routing_runs():
  import torch
  from helpers import tiny_config, make_engine, batch_of
  from maxtext_b200.models.transformer import Transformer
  base = ["num_experts=4", "num_experts_per_tok=2", "base_moe_mlp_dim=64", "weight_init=normal"]
  full = Transformer(tiny_config("mixtral-8x7b", base), None, "cpu")
  tight = Transformer(tiny_config("mixtral-8x7b", base + ["capacity_factor=0.5"]), None, "cpu")
  loose = Transformer(tiny_config("mixtral-8x7b", base + ["capacity_factor=8.0"]), None, "cpu")
  for m_ in (full, tight, loose):
    m_.store.initialize(seed=0)
  toks = torch.randint(0, 256, (2, 32))
  a, b, c = full.forward(toks), tight.forward(toks), loose.forward(toks)
  assert torch.allclose(a, c, atol=1e-6)                        # capacity above the load: nothing dropped
  assert (a - b).abs().max() > 1e-4                            # half the fair share: some assignments dropped
  # the mask itself: capacity = ceil(S k / E) * cf per sequence, arrival order over (token, choice)
  moe = tight.layers[0].blocks[0].mlp
  x2 = torch.randn(2 * 32, 64)
  wts, idx, _ = moe.route(x2, 2, 32)
  cap = int(max(-(-32 * 2 // 4) * 0.5, 0.5))
  for row in range(2):
    cnt = {}
    for t in range(32):
      for j in range(2):
        e = int(idx[row * 32 + t, j])
        cnt[e] = cnt.get(e, 0) + 1
        assert (float(wts[row * 32 + t, j]) == 0.0) == (cnt[e] > cap)
  eng = make_engine(tiny_config("mixtral-8x7b", base + ["use_random_routing=true", "capacity_factor=1.0"]))
  bt = batch_of(eng.config)
  assert torch.isfinite(torch.as_tensor(float(eng.train_step(bt)["learning/loss"])))


def test_small_config_switches():
  """use_untrainable_positional_embedding, qk_norm_with_scale=false, reuse_example_batch."""
  import torch
  from helpers import tiny_config, make_engine, batch_of, TINY, BASE_YML
  from maxtext_b200.train import train as T
  eng = make_engine(tiny_config("llama3-8b", ["use_untrainable_positional_embedding=true"]))
  ref_ = make_engine(tiny_config("llama3-8b"))
  toks = torch.randint(0, 256, (1, 8))
  pos = torch.arange(8)[None]
  d = eng.model.embed(toks, pos) - ref_.model.embed(toks, pos)
  half = 32
  inv = torch.exp(torch.arange(half).float() * -(torch.log(torch.tensor(10000.0)) / (half - 1)))
  want = torch.cat([torch.sin(pos.float()[..., None] * inv), torch.cos(pos.float()[..., None] * inv)], -1)
  assert torch.allclose(d, want, atol=1e-5)
  q = make_engine(tiny_config("qwen3-8b", ["qk_norm_with_scale=false"]))
  assert not any("query_norm" in n or "key_norm" in n for n in q.store.params)
  b = batch_of(q.config)
  ls = [float(q.train_step(b)["learning/loss"]) for _ in range(4)]
  assert ls[-1] < ls[0]
  args = [a for a in TINY if not a.startswith("steps")] + ["model_name=llama3-8b", "steps=4", "reuse_example_batch=1"]
  _, hist = T.main(["train", BASE_YML] + args)
  losses = [h["learning/loss"] for h in hist]
  assert all(b_ < a_ for a_, b_ in zip(losses, losses[1:])), losses        # the same batch every step: monotone at this size


def test_moba_mask_matches_a_per_query_restatement_and_trains():
  import torch
  from helpers import tiny_config, make_engine, batch_of
  from maxtext_b200.ops import reference as ref
  torch.manual_seed(0)
  B, S, Hq, Hkv, D, chunk, topk = 1, 22, 4, 2, 8, 4, 2
  q, k = torch.randn(B, S, Hq, D), torch.randn(B, S, Hkv, D)
  pos = torch.arange(S)[None]
  m = ref.moba_block_mask(q, k, pos, chunk, topk)
  g, nb = Hq // Hkv, -(-S // chunk)
  for h in range(Hq):
    kv = h // g
    for t in range(S):
      scores = []
      for n in range(nb):
        blk = k[0, n * chunk:(n + 1) * chunk, kv].float().mean(0)
        sc = float(q[0, t, h].float() @ blk)
        if n > t // chunk:
          sc = float("-inf")
        if n == t // chunk:
          sc = float("inf")
        scores.append(sc)
      best = sorted(range(nb), key=lambda n: -scores[n])[: min(topk, nb)]
      best = [n for n in best if scores[n] > float("-inf")]
      want = torch.tensor([(j // chunk in best) and j <= t for j in range(S)])
      assert torch.equal(m[0, kv, h % g, t], want), (h, t)
  # with top-k covering all blocks the result is plain causal attention
  v = torch.randn(B, S, Hkv, D)
  full = ref.moba_attention(q, k, v, pos, chunk, nb, 0.3)
  causal = ref.attention(q, k, v, ref.attention_mask(pos, pos), 0.3)
  assert torch.allclose(full, causal.to(full.dtype), atol=1e-5)
  eng = make_engine(tiny_config("llama3-8b", ["moba=true", "moba_chunk_size=8", "moba_topk=2"]))
  b = batch_of(eng.config)
  ls = [float(eng.train_step(b)["learning/loss"]) for _ in range(4)]
  assert ls[-1] < ls[0]


def test_prometheus_endpoint_serves_step_metrics():
  import socket
  import urllib.request
  from helpers import tiny_config
  from maxtext_b200.utils.metric_logger import MetricLogger
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
  ml = MetricLogger(tiny_config("llama3-8b", [f"prometheus_port={port}"]))
  ml.record(0, {"learning/loss": 2.5}, 0.1)
  ml.flush()
  body = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=10).read().decode()
  assert "maxtext_learning_loss 2.5" in body and "maxtext_perf_step_time_seconds" in body
  ml.close()


def test_convergence_recipe_resolves_samples_and_tokens_into_steps():
  from maxtext_b200.benchmarks.convergence import C4_MLPERF, ConvergenceSpec, convergence_recipe
  from maxtext_b200.benchmarks.recipes import RECIPES
  spec = ConvergenceSpec(warmup_samples=1000, decay_end_samples=10000, total_tokens_to_train=64 * 8192 * 500, learning_rate_per_sample=1e-6,
                         eval_interval_tokens=64 * 8192 * 50, target_eval_loss=2.7)
  r = convergence_recipe(RECIPES["llama3_8b_8192_fsdp8"], C4_MLPERF, spec, gpus=8, global_batch=64)
  t = r.tuning
  assert t["steps"] == 500 and t["per_device_batch_size"] == 8.0 and abs(t["learning_rate"] - 6.4e-5) < 1e-12
  assert t["learning_rate_schedule_steps"] == 157 and abs(t["warmup_steps_fraction"] - 16 / 157) < 1e-9
  assert t["eval_interval"] == 50 and t["eval_steps"] == -(-24567 * 2048 // (64 * 8192)) and t["dataset_type"] == "c4_mlperf"
  assert t["target_eval_loss"] == 2.7 and r.gpus == 8 and r.name.endswith("-c4mlperf")
  over = r.overrides()
  assert "steps=500" in over and "dataset_type=c4_mlperf" in over and "eval_split=validation_24567exp" in over
  # the same specification on another machine size keeps the token budget
  r2 = convergence_recipe(RECIPES["llama3_8b_8192_fsdp8"], C4_MLPERF, spec, gpus=4, global_batch=32)
  assert r2.tuning["steps"] == 1000 and r2.tuning["per_device_batch_size"] == 8.0


def test_results_database_keeps_runs_and_ignores_throttled_ones(tmp_path):
  from maxtext_b200.benchmarks.results_db import ResultsDB, main
  db = ResultsDB(str(tmp_path / "runs.sqlite"))
  line = {"metric": "tokens/sec", "value": 15436.0, "unit": "tokens/s", "n_gpus": 1, "ms_per_step": 1061.4, "dtype": "bf16",
          "config": {"model": "llama3-8b", "parallelism": "fsdp1"}, "clocks": {"sm_mhz": 1470, "reasons": ["sw_power_cap"]},
          "e2e": {"value": 15428.0}}
  a = db.add(line)
  b = db.add({**line, "value": 17000.0, "clocks": {"sm_mhz": 900, "reasons": ["hw_thermal_slowdown"]}})
  c = db.add({**line, "value": 118000.0, "n_gpus": 8, "config": {"model": "llama3-8b", "parallelism": "fsdp8"}})
  assert (a, b, c) == (1, 2, 3) and len(db.query(model="llama3-8b")) == 3 and len(db.query(gpus=8)) == 1
  assert db.best(model="llama3-8b", gpus=1)["id"] == a                      # the faster run was throttled
  assert db.best(model="llama3-8b", gpus=1, ignore_throttled=False)["id"] == b
  assert db.record(c)["config"]["parallelism"] == "fsdp8" and db.best(model="other") is None
  import pytest
  with pytest.raises(ValueError):
    db.add({"value": 1})
  db.close()
  assert main(["best", str(tmp_path / "runs.sqlite"), "--gpus", "8"]) == 0
