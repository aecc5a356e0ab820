"""Each memory-bound CUDA kernel against the PyTorch definition in ops.reference."""
import pytest
import torch

from maxtext_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


def _E():
  from maxtext_b200.ops import backend
  return backend.ext(required=True)


@pytest.mark.parametrize("rows,D", [(64, 4096), (37, 1024), (300, 128), (5, 8192), (129, 264)])
def test_rmsnorm_fwd_bwd(rows, D):
  E = _E()
  x = torch.randn(rows, D, device="cuda").bfloat16()
  scale = (1 + 0.1 * torch.randn(D, device="cuda")).bfloat16()
  y = torch.empty_like(x)
  rstd = torch.empty(rows, device="cuda")
  E.rmsnorm_fwd(x, scale, 1e-5, 0.0, y, rstd)
  yr = ref.rmsnorm(x, scale, 1e-5)
  assert (y.float() - yr.float()).abs().max() <= 2e-2
  dy = torch.randn(rows, D, device="cuda").bfloat16()
  dx = torch.empty_like(x)
  ds = torch.zeros(D, device="cuda")
  E.rmsnorm_bwd(dy, x, scale, rstd, 0.0, dx, ds)
  dxr, dsr = ref.rmsnorm_bwd(dy, x, scale, 1e-5)
  assert (dx.float() - dxr.float()).abs().max() <= 3e-2
  assert (ds - dsr).abs().max() <= 2e-2 * max(1.0, dsr.abs().max().item())


@pytest.mark.parametrize("interleaved", [False, True])
def test_rope_roundtrip_and_reference(interleaved):
  E = _E()
  B, S, H, Dh = 2, 96, 6, 128
  x = torch.randn(B, S, H, Dh, device="cuda").bfloat16()
  pos = torch.arange(S, device="cuda", dtype=torch.int32)[None].expand(B, S).contiguous()
  inv = ref.rope_inv_timescale(Dh, 1, 500000).cuda()
  want = ref.apply_rope(x[:, :, :4], pos, inv, interleaved)
  y = x.clone()
  E.rope_inplace(y.view(B * S, H, Dh), pos.reshape(-1), inv, 4, interleaved, False, Dh)
  assert (y[:, :, :4].float() - want.float()).abs().max() <= 3e-2
  assert torch.equal(y[:, :, 4:], x[:, :, 4:])
  E.rope_inplace(y.view(B * S, H, Dh), pos.reshape(-1), inv, 4, interleaved, True, Dh)
  assert (y.float() - x.float()).abs().max() <= 5e-2


@pytest.mark.parametrize("act,code", [("silu", 0), ("gelu", 1)])
def test_gated_act(act, code):
  E = _E()
  torch.manual_seed(0)
  gu = torch.randn(200, 2 * 1408, device="cuda").bfloat16()
  out = torch.empty(200, 1408, device="cuda", dtype=torch.bfloat16)
  E.gated_act_fwd(gu, out, code)
  want = ref.gated_act(gu, act).float()
  assert bool(((out.float() - want).abs() <= 1e-2 + want.abs() / 64).all())          # within two bf16 ulps of the reference
  dy = torch.randn_like(out)
  dgu = torch.empty_like(gu)
  E.gated_act_bwd(dy, gu, dgu, code)
  wantg = ref.gated_act_bwd(dy, gu, act).float()
  assert bool(((dgu.float() - wantg).abs() <= 2e-2 + wantg.abs() / 64).all())


@pytest.mark.parametrize("V", [32000, 128256, 1003 * 8])
def test_xent_fwd_bwd(V):
  E = _E()
  rows = 33
  logits = (3 * torch.randn(rows, V, device="cuda")).bfloat16()
  tg = torch.randint(0, V, (rows,), device="cuda", dtype=torch.int32)
  w = (torch.rand(rows, device="cuda") > 0.2).float()
  want, wz = ref.cross_entropy(logits, tg.long(), 1e-4)
  wd = ref.cross_entropy_dlogits(logits, tg.long(), w, 1e-4)
  loss = torch.empty(rows, device="cuda")
  z = torch.empty(rows, device="cuda")
  work = logits.clone()
  E.xent_fwd_bwd(work, tg, w, 1e-4, loss, z, True)
  assert (loss - want).abs().max() <= 2e-3 * want.abs().max()
  assert (z - wz).abs().max() <= 1e-3 * max(1.0, wz.abs().max().item())
  assert (work.float() - wd).abs().max() <= 1e-2


def test_adamw_and_sumsq():
  E = _E()
  n = 1 << 20
  p = torch.randn(n, device="cuda")
  g = torch.randn(n, device="cuda")
  m = torch.zeros(n, device="cuda")
  v = torch.zeros(n, device="cuda")
  sh = torch.empty(n, device="cuda", dtype=torch.bfloat16)
  pr, mr, vr = p.clone(), m.clone(), v.clone()
  gs = torch.tensor([0.5], device="cuda")
  for step in (1, 2, 3):
    E.adamw(p, g, m, v, sh, 1e-2, 0.9, 0.95, 1e-8, 0.0, 0.1, 1 - 0.9 ** step, 1 - 0.95 ** step, gs)
    ref.adamw_step(pr, g, mr, vr, 1e-2, 0.9, 0.95, 1e-8, 0.0, 0.1, step, 0.5)
  assert (p - pr).abs().max() <= 1e-5
  assert (sh.float() - pr).abs().max() <= 2e-2
  out = torch.zeros(1, device="cuda")
  E.sumsq(g, out)
  assert abs(out.item() - g.double().pow(2).sum().item()) <= 1e-4 * n
  out2 = torch.zeros(1, device="cuda")
  E.sumsq(g, out2)
  assert out.item() == out2.item()   # fixed reduction order


def test_embedding():
  E = _E()
  V, D, T = 1000, 256, 513
  table = torch.randn(V, D, device="cuda").bfloat16()
  tok = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
  out = torch.empty(T, D, device="cuda", dtype=torch.bfloat16)
  E.embedding_fwd(tok, table, out)
  assert torch.equal(out, table[tok.long()])
  dy = torch.randn(T, D, device="cuda").bfloat16()
  dt = torch.zeros(V, D, device="cuda")
  E.embedding_bwd(tok, dy, dt)
  want = torch.zeros(V, D, device="cuda").index_add_(0, tok.long(), dy.float())
  assert (dt - want).abs().max() <= 1e-3


@pytest.mark.gpu
def test_muon_newton_schulz_on_the_repository_gemm():
  """The GPU path runs the iteration in bf16 on this repository's GEMM; it must orthogonalise like the fp32 definition."""
  from maxtext_b200.optimizers.muon import newton_schulz
  torch.manual_seed(0)
  for shape in ((256, 512), (512, 256)):
    x = torch.randn(*shape)
    want = newton_schulz(x, steps=5)
    got = newton_schulz(x.cuda(), steps=5).float().cpu()
    assert (got - want).abs().max() < 0.05 * want.abs().max() + 0.02, (got - want).abs().max()
    sv = torch.linalg.svdvals(got)
    assert float(sv.max()) < 1.3 and float(sv.min()) > 0.4
