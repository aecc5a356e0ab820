"""MoE kernels on the GPU against plain PyTorch fp32 references: padded stable sort, gather/combine, grouped GEMMs, and the
whole routed FFN (forward and gradients) against the per-expert loop."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ext():
  from maxtext_b200.ops import backend
  return backend.ext(required=True)


def _plan(idx, E):
  from maxtext_b200.ops.moe_ops import GroupPlan
  return GroupPlan(idx, E)


@pytest.mark.parametrize("T,k,E", [(512, 2, 8), (1000, 4, 64), (4096, 8, 256), (64, 2, 16)])
def test_sort_is_stable_and_padded(T, k, E):
  torch.manual_seed(0)
  idx = torch.randint(0, E, (T, k), device="cuda")
  if E == 16:
    idx[idx == 3] = 4                     # an empty expert
  p = _plan(idx, E)
  flat = idx.reshape(-1)
  sizes = torch.bincount(flat, minlength=E)
  assert torch.equal(p.sizes.long(), sizes)
  padded = (sizes + 127) // 128 * 128
  offs = torch.cat([torch.zeros(1, dtype=torch.long, device="cuda"), padded.cumsum(0)])
  assert torch.equal(p.offs.long(), offs)
  order = torch.argsort(flat, stable=True)               # stable sort oracle
  starts = offs[:-1]
  want_dest = torch.empty_like(flat)
  rank = torch.arange(flat.numel(), device="cuda") - torch.repeat_interleave(sizes.cumsum(0) - sizes, sizes)
  want_dest[order] = (starts[flat[order]] + rank)
  assert torch.equal(p.dest.long(), want_dest)
  rp = p.row_pair.long()
  used = int(offs[-1])
  assert torch.equal(rp[want_dest], torch.arange(flat.numel(), device="cuda"))
  assert int((rp[:used] < 0).sum()) == used - flat.numel()
  blk = p.blk_expert.long()[: used // 128]
  want_blk = torch.repeat_interleave(torch.arange(E, device="cuda"), padded // 128)
  assert torch.equal(blk, want_blk)


def test_gather_combine_roundtrip_and_grads():
  from maxtext_b200.ops import moe_ops
  torch.manual_seed(1)
  T, k, E, D = 768, 2, 8, 256
  x = torch.randn(T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
  idx = torch.randint(0, E, (T, k), device="cuda")
  w = torch.rand(T, k, device="cuda", requires_grad=True)
  plan = _plan(idx, E)
  rows = moe_ops._GatherRowsFn.apply(x, plan)
  out = moe_ops._CombineFn.apply(rows * 1.0, w, plan)
  want = (x.float()[:, None, :] * w[:, :, None]).sum(1)
  assert torch.allclose(out.float(), want, atol=2e-2, rtol=2e-2)
  g = torch.randn_like(out)
  out.backward(g)
  want_dx = g.float() * w.sum(1, keepdim=True)
  assert torch.allclose(x.grad.float(), want_dx, atol=3e-2, rtol=3e-2)
  want_dw = (g.float()[:, None, :] * x.float()[:, None, :]).sum(-1).expand(T, k)
  assert torch.allclose(w.grad, want_dw, atol=0.3, rtol=3e-2)


@pytest.mark.parametrize("T,k,E,D,Fd", [(1024, 2, 8, 512, 1024), (2048, 4, 16, 256, 384), (300, 2, 4, 128, 128)])
def test_grouped_gemm_modes(T, k, E, D, Fd):
  torch.manual_seed(2)
  ext = _ext()
  idx = torch.randint(0, E, (T, k), device="cuda")
  if E == 4:
    idx[idx == 2] = 1                     # empty group: its weight gradient must come out zero
  plan = _plan(idx, E)
  R = plan.rows_max
  used = int(plan.offs[-1])
  blk = plan.blk_expert.long()
  row_e = torch.repeat_interleave(blk, 128)[:R]
  x = torch.randn(R, D, device="cuda", dtype=torch.bfloat16) * 0.5
  valid = (plan.row_pair >= 0)
  x[~valid] = 0
  W = torch.randn(E, Fd, D, device="cuda", dtype=torch.bfloat16) * 0.05
  # mode 1
  y = torch.empty(R, Fd, device="cuda", dtype=torch.bfloat16)
  ext.grouped_gemm(1, x, W, y, plan.offs, plan.blk_expert, False)
  want = torch.einsum("rd,rfd->rf", x.float(), W.float()[row_e])
  assert torch.allclose(y[:used].float(), want[:used], atol=3e-2, rtol=3e-2)
  # mode 1 into a column slice of a wider buffer
  wide = torch.zeros(R, 2 * Fd, device="cuda", dtype=torch.bfloat16)
  ext.grouped_gemm(1, x, W, wide[:, Fd:], plan.offs, plan.blk_expert, False)
  assert torch.equal(wide[:used, Fd:], y[:used]) and float(wide[:, :Fd].abs().max()) == 0
  # mode 2
  dy = torch.randn(R, Fd, device="cuda", dtype=torch.bfloat16) * 0.5
  dy[~valid] = 0
  dx = torch.empty(R, D, device="cuda", dtype=torch.bfloat16)
  ext.grouped_gemm(2, dy, W, dx, plan.offs, plan.blk_expert, False)
  want = torch.einsum("rf,rfd->rd", dy.float(), W.float()[row_e])
  assert torch.allclose(dx[:used].float(), want[:used], atol=5e-2, rtol=3e-2)
  # mode 3 (+ accumulate)
  dW = torch.full((E, Fd, D), 7.0, device="cuda")
  ext.grouped_gemm(3, dy, x, dW, plan.offs, plan.blk_expert, False)
  want = torch.zeros(E, Fd, D, device="cuda")
  want.index_add_(0, row_e[:used], torch.einsum("rf,rd->rfd", dy[:used].float(), x[:used].float())) if R * Fd * D < 2e9 else None
  assert torch.allclose(dW, want, atol=0.15, rtol=3e-2)
  ext.grouped_gemm(3, dy, x, dW, plan.offs, plan.blk_expert, True)
  assert torch.allclose(dW, 2 * want, atol=0.3, rtol=3e-2)
  assert ext.kernel_status(True) == 0


def test_routed_moe_layer_matches_per_expert_loop():
  """Mixtral-style block: padded-group kernels vs the reference composition (fp32 math), forward and all gradients."""
  from helpers import tiny_config
  from maxtext_b200.models.transformer import Transformer
  torch.manual_seed(3)
  cfg = tiny_config("mixtral-8x7b", extra=["base_emb_dim=256", "base_mlp_dim=512", "base_moe_mlp_dim=512", "num_experts=8", "num_experts_per_tok=2",
                                           "base_num_decoder_layers=1", "dtype=bfloat16", "hardware=gpu", "max_target_length=256",
                                           "per_device_batch_size=4", "base_num_query_heads=4", "base_num_kv_heads=2", "head_dim=64"])
  model = Transformer(cfg, None, "cuda")
  model.store.initialize(seed=0)
  moe = model.layers[0].blocks[0].mlp
  from maxtext_b200.ops import moe_ops
  B, S, D = 4, 256, 256
  x = (torch.randn(B, S, D, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
  ctx = model.make_ctx(torch.arange(S, device="cuda")[None].expand(B, S), None, "train")
  model.store.begin_step()
  y = moe(x, ctx)
  g = torch.randn_like(y)
  y.backward(g)
  got_dx = x.grad.clone()
  got_dw = {n: p.main_grad.clone().float() for n, p in (("wi_0", moe.wi_0), ("wi_1", moe.wi_1), ("wo", moe.wo))}
  # reference: same routing, fp32 per-expert math
  x32 = x.detach().float().requires_grad_(True)
  x2 = x32.reshape(-1, D)
  _, idx, _ = moe.route(x.detach().reshape(-1, D), B, S)
  gate_w = moe.gate.leaf().detach().float()
  wts = torch.softmax((x2 @ gate_w.T).gather(1, idx), -1)         # differentiable router weights (Mixtral: softmax over the top-k logits)
  W0, W1, Wo = (p.data.detach().float().requires_grad_(True) for p in (moe.wi_0, moe.wi_1, moe.wo))
  out = torch.zeros_like(x2)
  for e in range(moe.E):
    for c in range(moe.k):
      m = idx[:, c] == e
      if m.any():
        h = torch.nn.functional.silu(x2[m] @ W0[e].T) * (x2[m] @ W1[e].T)
        out = out.index_add(0, m.nonzero()[:, 0], (h @ Wo[e].T) * wts[m, c, None].float())
  out.backward(g.reshape(-1, D).float())
  rel = lambda a, b: float((a.float() - b).abs().max() / (b.abs().max() + 1e-6))  # noqa: E731
  assert rel(y.reshape(-1, D), out) < 2e-2, rel(y.reshape(-1, D), out)
  assert rel(got_dx, x32.grad) < 2e-2, rel(got_dx, x32.grad)
  for n, w in (("wi_0", W0), ("wi_1", W1), ("wo", Wo)):
    err = (got_dw[n] - w.grad).abs().max() / (w.grad.abs().max() + 1e-6)
    assert err < 3e-2, (n, float(err))


@pytest.mark.parametrize("E,k,mode,sig,raw,use_bias", [(8, 2, 0, False, False, False), (128, 8, 0, False, False, True), (16, 1, 0, False, True, False),
                                                      (64, 6, 1, False, False, True), (64, 6, 1, True, False, True), (160, 6, 1, True, False, False)])
def test_router_kernel_matches_pytorch_forward_and_backward(E, k, mode, sig, raw, use_bias):
  """Scores, top-k, routing weights and the expert histogram from one launch; gradients w.r.t. the logits through both
  outputs (weights and full probabilities) against autograd of the plain PyTorch formulas."""
  from maxtext_b200.ops import moe_ops
  torch.manual_seed(E + k)
  T = 777
  logits = (torch.randn(T, E, device="cuda") * 2.0).requires_grad_(True)
  bias = (torch.randn(E, device="cuda") * 0.5) if use_bias else None
  scaling = 2.5 if mode == 1 else 1.0
  idx, wts, probs, counts = moe_ops.router_topk(logits, bias, k, mode, sig, raw, scaling)
  ref_l = logits.detach().clone().requires_grad_(True)
  if mode == 1:
    scores = torch.sigmoid(ref_l) if sig else torch.softmax(ref_l, -1)
    sel = scores + bias if bias is not None else scores
    ridx = sel.topk(k, -1).indices
    rw = scores.gather(-1, ridx)
    if sig:
      rw = rw / (rw.sum(-1, keepdim=True) + 1e-20)
    rw, rp = rw * scaling, scores
  else:
    lg = ref_l + bias if bias is not None else ref_l
    vals, ridx = lg.topk(k, -1)
    rw = vals if raw else torch.softmax(vals, -1)
    rp = torch.softmax(lg, -1)
  assert torch.equal(idx, ridx)
  assert torch.allclose(wts, rw, atol=1e-5, rtol=1e-4) and torch.allclose(probs, rp, atol=1e-6, rtol=1e-4)
  assert torch.equal(counts.long(), torch.bincount(ridx.reshape(-1), minlength=E))
  gw, gp = torch.randn_like(wts), torch.randn_like(probs)
  ((wts * gw).sum() + (probs * gp).sum()).backward()
  ((rw * gw).sum() + (rp * gp).sum()).backward()
  assert torch.allclose(logits.grad, ref_l.grad, atol=2e-5, rtol=1e-3), (logits.grad - ref_l.grad).abs().max()
