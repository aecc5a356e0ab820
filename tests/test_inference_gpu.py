"""Decode on the GPU: the kernel path (split-KV decode attention, no host sync) against the CPU reference engine, and the
CUDA-graph replay against eager decoding."""
import pytest
import torch

pytestmark = pytest.mark.gpu

ARGS = ["base_emb_dim=256", "base_num_query_heads=4", "base_num_kv_heads=2", "head_dim=64", "base_mlp_dim=512", "base_num_decoder_layers=3",
        "vocab_size=512", "max_target_length=160", "max_prefill_predict_length=64", "per_device_batch_size=3", "weight_init=normal"]


def _run(cfg, device, steps=12, weights=None):
  from maxtext_b200.inference.maxengine import MaxEngine
  eng = MaxEngine(cfg, device=device)
  eng.load_params(seed=3)
  if weights is not None:              # the initialiser draws from the device's own generator: share one set of weights
    eng.model.store.master.copy_(weights.to(device))
    eng.model.store.sync_compute_from_master()
  state = eng.init_decode_state(3)
  g = torch.Generator().manual_seed(0)
  for s, n in enumerate((5, 17, 40)):
    toks = torch.randint(1, cfg.vocab_size, (n,), generator=g)
    p, _ = eng.prefill(toks, n)
    state = eng.insert(p, state, s)
  out = []
  for _ in range(steps):
    state, res = eng.generate(state)
    out.append(res.data[:, 0].cpu())
  return torch.stack(out), eng


def test_gpu_decode_matches_cpu_reference_and_graph_replay():
  from helpers import tiny_config
  cpu_cfg = tiny_config(extra=ARGS + ["dtype=float32", "hardware=cpu"])
  want, cpu_eng = _run(cpu_cfg, "cpu")
  w = cpu_eng.model.store.master.clone()
  gpu_cfg = tiny_config(extra=ARGS + ["dtype=bfloat16", "hardware=gpu"])
  got, eng = _run(gpu_cfg, "cuda", weights=w)
  # bf16 vs fp32 can flip a near-tie; the first tokens of every slot must agree and most of the rest
  assert torch.equal(got[0], want[0])
  assert (got == want).float().mean() > 0.8
  graph_cfg = tiny_config(extra=ARGS + ["dtype=bfloat16", "hardware=gpu", "cuda_graphs=true"])
  got_g, eng_g = _run(graph_cfg, "cuda", weights=w)
  assert any(v is not False for v in eng_g._graphs.values()), "graph capture fell back to eager"
  assert torch.equal(got_g, got)


def test_sampling_kernel_matches_the_pytorch_definition():
  """Greedy is the arg-max; top-k and nucleus draws stay inside the support PyTorch's masks give; the empirical frequencies of
  many rows with the same logits follow softmax(kept / temperature); the same uniform numbers give the same tokens."""
  import torch
  from maxtext_b200.inference import inference_utils as U
  from maxtext_b200.ops import backend
  E = backend.ext(required=True)
  torch.manual_seed(0)
  big = torch.randn(64, 128256, device="cuda") * 3
  assert torch.equal(U.sampling(big, "greedy"), big.argmax(-1))
  assert torch.equal(U.sampling(big.bfloat16(), "greedy"), big.bfloat16().float().argmax(-1))
  g = torch.Generator(device="cuda").manual_seed(5)
  tk = U.sampling(big, "topk", topk=40, temperature=0.8, generator=g)
  kth = big.topk(40, -1).values[:, -1]
  assert (big.gather(1, tk[:, None])[:, 0] >= kth).all()
  g.manual_seed(5)
  assert torch.equal(tk, U.sampling(big, "topk", topk=40, temperature=0.8, generator=g))          # reproducible under a seed
  keep = torch.isfinite(U._mask_nucleus(big.float(), 0.6))
  g.manual_seed(6)
  nu = U.sampling(big, "nucleus", nucleus_p=0.6, generator=g)
  assert keep.gather(1, nu[:, None]).all()
  keep_c = torch.isfinite(U._mask_nucleus(U._mask_topk(big.float(), 50), 0.9))
  co = U.sampling(big, "composite", topk=50, nucleus_p=0.9, temperature=1.3, generator=g)
  assert keep_c.gather(1, co[:, None]).all()
  # frequencies: 40 000 rows of the same 16 logits
  base = torch.tensor([2.0, 1.5, 1.0, 0.5, 0.0, -0.5, -1.0, -1.5, 3.0, -3.0, 0.2, 0.1, -0.1, 2.5, -2.0, 1.2], device="cuda")
  rows = base[None].expand(40000, 16).contiguous()
  for strategy, kw in (("weighted", dict(temperature=0.7)), ("topk", dict(topk=5, temperature=1.0)), ("nucleus", dict(nucleus_p=0.8)),
                       ("composite", dict(topk=8, nucleus_p=0.9, temperature=1.5))):
    toks = U.sampling(rows, strategy, generator=g, **kw)
    lf = base.float()[None]
    if strategy in ("topk", "composite"):
      lf = U._mask_topk(lf, kw.get("topk", 0))
    if strategy in ("nucleus", "composite"):
      lf = U._mask_nucleus(lf, kw.get("nucleus_p", -1.0))
    want = torch.softmax(lf / kw.get("temperature", 1.0), -1)[0]
    got = torch.bincount(toks, minlength=16).float() / toks.numel()
    assert (got - want).abs().max() < 0.012, (strategy, got, want)
    assert (got[want == 0] == 0).all()
