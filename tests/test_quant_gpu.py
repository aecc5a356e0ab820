"""FP8 path on the GPU: quantisation kernels against torch's float8 casts, the 8-bit GEMM against an fp32 product of the
de-quantised operands, the quantised linear layer against bf16, and a short fp8 training run."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ext():
  from maxtext_b200.ops import backend
  return backend.ext(required=True)


@pytest.mark.parametrize("fmt,dtype,fmax", [(0, torch.float8_e4m3fn, 448.0), (1, torch.float8_e5m2, 57344.0)])
def test_quantize_matches_torch_cast(fmt, dtype, fmax):
  E = _ext()
  torch.manual_seed(0)
  x = (torch.randn(256, 384, device="cuda") * 3).bfloat16()
  q, qt, deq = E.quantize_fp8(x, fmt, True, True)
  amax = x.float().abs().max()
  assert torch.allclose(deq, (amax / fmax).reshape(1))
  want = (x.float() * (fmax / amax)).to(dtype)
  assert torch.equal(q.view(dtype).float(), want.float())
  assert torch.equal(qt, q.t().contiguous())
  q2, qt2, _ = E.quantize_fp8(x, fmt, False, True)
  assert q2 is None and torch.equal(qt2, qt)


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (1024, 768, 512), (384, 128, 1152)])
def test_gemm_fp8_matches_dequantised_product(M, N, K):
  E = _ext()
  torch.manual_seed(1)
  a = torch.randn(M, K, device="cuda").bfloat16()
  b = torch.randn(N, K, device="cuda").bfloat16()
  aq, _, sa = E.quantize_fp8(a, 0, True, False)
  bq, _, sb = E.quantize_fp8(b, 1, True, False)
  ref = (aq.view(torch.float8_e4m3fn).float() * sa) @ (bq.view(torch.float8_e5m2).float() * sb).t()
  out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
  E.gemm_fp8(aq, bq, out, 0, 1, sa, sb, False)
  assert torch.allclose(out.float(), ref, atol=0.05 * float(ref.abs().max()) / 16, rtol=1e-2)
  acc = torch.full((M, N), 2.0, device="cuda")
  E.gemm_fp8(aq, bq, acc, 0, 1, sa, sb, True)
  assert torch.allclose(acc, ref + 2.0, atol=1e-3 * float(ref.abs().max()), rtol=1e-4)
  assert E.kernel_status(True) == 0


def test_fp8_linear_close_to_bf16():
  from maxtext_b200.ops import quantization as Q
  torch.manual_seed(2)
  x = (torch.randn(512, 1024, device="cuda") * 0.5).bfloat16()
  w = (torch.randn(768, 1024, device="cuda") * 0.05).bfloat16()
  dy = (torch.randn(512, 768, device="cuda") * 0.1).bfloat16()
  Q.set_mode("fp8")
  try:
    assert Q.supported(x, w)
    y = Q.linear_fwd(x, w)
    g = torch.zeros(768, 1024, device="cuda")
    dx = Q.linear_bwd(dy, x, w, True, g, False)
  finally:
    Q.set_mode("")
  rel = lambda a, b: float((a.float() - b).norm() / b.norm())  # noqa: E731
  assert rel(y, x.float() @ w.float().t()) < 0.06
  assert rel(dx, dy.float() @ w.float()) < 0.08
  assert rel(g, dy.float().t() @ x.float()) < 0.08


def test_fp8_training_reduces_loss():
  from helpers import tiny_config
  from maxtext_b200.train import train as train_lib
  cfg = tiny_config(extra=["quantization=fp8", "base_emb_dim=256", "base_mlp_dim=512", "head_dim=64", "vocab_size=512", "max_target_length=128",
                           "per_device_batch_size=4", "dtype=bfloat16", "hardware=gpu", "steps=12", "learning_rate=3e-3"])
  try:
    _, hist = train_lib.train_loop(cfg)
  finally:
    from maxtext_b200.ops import quantization as Q
    Q.set_mode("")
  assert hist[-1]["learning/loss"] < hist[0]["learning/loss"] - 0.3


def test_delayed_scaling_uses_history_maximum():
  from maxtext_b200.ops import quantization as Q
  E = _ext()
  torch.manual_seed(5)
  x1 = (torch.randn(128, 128, device="cuda")).bfloat16()
  x2 = (torch.randn(128, 128, device="cuda") * 0.1).bfloat16()          # much smaller than the history's maximum
  Q.set_delayed_scaling(4)
  try:
    owner = object()
    _, _, s1 = Q._quantize(x1, 0, True, False, (id(owner), "x"))
    q2, _, s2 = Q._quantize(x2, 0, True, False, (id(owner), "x"))
    assert torch.allclose(s2, s1)                                        # the scale still comes from the first tensor's amax
    want = (x2.float() / s1).to(torch.float8_e4m3fn)
    assert torch.equal(q2.view(torch.float8_e4m3fn).float(), want.float())
    ring = Q._HISTORY[(id(owner), "x")][0]
    assert torch.allclose(ring[0], x2.float().abs().max())                # ...and x2's amax entered the history
  finally:
    Q.set_delayed_scaling(0)


@pytest.mark.gpu
def test_int8_products_on_gpu_match_the_definition():
  """quantization=int8 on the GPU (integer product through the library) against the float emulation of the same integers."""
  from maxtext_b200.ops import quantization as Q
  torch.manual_seed(0)
  x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
  w = (torch.randn(384, 512, device="cuda") * 0.1).bfloat16()
  dy = torch.randn(256, 384, device="cuda", dtype=torch.bfloat16)
  y, dx = Q.int8_linear_fwd(x, w), Q.int8_linear_dx(dy, w)
  y_ref, dx_ref = Q.int8_linear_fwd(x.cpu().float(), w.cpu().float()), Q.int8_linear_dx(dy.cpu().float(), w.cpu().float())
  assert (y.float().cpu() - y_ref).abs().max() < 0.02 * y_ref.abs().max() + 0.05
  assert (dx.float().cpu() - dx_ref).abs().max() < 0.02 * dx_ref.abs().max() + 0.05


# ------------------------------------------------------------------------------------------------ block-scaled fp8
def _deq_rows(q, s_t):
  """q [R, C] e4m3 bytes with scales_t [C/128 blocks, R] -> fp32."""
  R, C = q.shape
  s = s_t.t().repeat_interleave(128, dim=1)[:, :C]
  return q.view(torch.float8_e4m3fn).float() * s


def _deq_blocks(q, s):
  """q [G, R, C] with scales [G, R/128 blocks, C/128 blocks] -> fp32."""
  G, R, C = q.shape
  full = s.repeat_interleave(128, dim=1)[:, :R].repeat_interleave(128, dim=2)[:, :, :C]
  return q.view(torch.float8_e4m3fn).float() * full


def test_block_quantisation_kernels_match_the_definition():
  E = _ext()
  torch.manual_seed(5)
  x = (torch.randn(300, 400, device="cuda") * torch.logspace(-2, 2, 400, device="cuda")).bfloat16()
  q, s_t = E.quant_fp8_rows(x)
  blocks = torch.nn.functional.pad(x.float(), (0, 112)).reshape(300, 4, 128)
  amax = blocks.abs().amax(-1)
  assert torch.allclose(s_t.t(), torch.where(amax > 0, amax / 448.0, torch.ones_like(amax)))
  want = (blocks * (448.0 / amax).unsqueeze(-1)).reshape(300, 512)[:, :400].to(torch.float8_e4m3fn)
  got = q.view(torch.float8_e4m3fn).float()
  assert float((got != want.float()).float().mean()) < 1e-3          # a product that lands on a rounding tie may go either way
  assert torch.allclose(got, want.float(), rtol=0.13, atol=2 ** -9)
  # a strided view quantises like its contiguous copy
  wide = torch.randn(64, 512, device="cuda").bfloat16()
  qa, sa = E.quant_fp8_rows(wide[:, 256:])
  qb, sb = E.quant_fp8_rows(wide[:, 256:].contiguous())
  assert torch.equal(qa, qb) and torch.equal(sa, sb)

  w = (torch.randn(3, 272, 144, device="cuda") * 0.3).bfloat16()
  wq, wt, sw = E.quant_fp8_blocks(w, True, True)
  assert sw.shape == (3, 3, 2) and torch.equal(wt, wq.transpose(1, 2).contiguous())
  rel = (_deq_blocks(wq, sw) - w.float()).abs().max() / w.float().abs().max()
  assert rel < 0.07
  pad = torch.nn.functional.pad(w.float(), (0, 112, 0, 112)).reshape(3, 3, 128, 2, 128).abs().amax((2, 4))
  assert torch.allclose(sw, pad / 448.0)


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (1000, 768, 1152), (384, 144, 400), (4096, 2048, 7168)])
def test_block_scaled_gemm_matches_dequantised_product(M, N, K):
  E = _ext()
  torch.manual_seed(6)
  a = (torch.randn(M, K, device="cuda") * torch.logspace(-1, 1, K, device="cuda")).bfloat16()
  b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
  aq, sa = E.quant_fp8_rows(a)
  bq, bt, sb = E.quant_fp8_blocks(b, True, True)
  ref = _deq_rows(aq, sa) @ _deq_blocks(bq, sb)[0].t()
  out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
  E.gemm_fp8_block(aq, sa, bq, sb, False, out, None, None)
  assert E.kernel_status(True) == 0
  tol = 8e-3 * float(ref.abs().max())
  assert torch.allclose(out.float(), ref, atol=tol, rtol=8e-3)
  # the whole product stays close to the bf16 one: block scales keep the wide dynamic range of `a`
  exact = a.float() @ b.float().t()
  assert float((out.float() - exact).norm() / exact.norm()) < 0.05
  # input-gradient form: dy [M, N] times the transposed 8-bit copy, scale table read transposed
  dy = torch.randn(M, N, device="cuda").bfloat16()
  gq, sg = E.quant_fp8_rows(dy)
  dx = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
  E.gemm_fp8_block(gq, sg, bt, sb, True, dx, None, None)
  assert E.kernel_status(True) == 0
  ref2 = _deq_rows(gq, sg) @ _deq_blocks(bq, sb)[0]
  assert torch.allclose(dx.float(), ref2, atol=8e-3 * float(ref2.abs().max()), rtol=8e-3)


def test_block_scaled_grouped_gemm_matches_per_expert_products():
  from maxtext_b200.ops import moe_ops
  E = _ext()
  torch.manual_seed(7)
  n_exp, T, k, D, Fd = 6, 700, 2, 256, 384
  idx = torch.randint(0, n_exp, (T, k), device="cuda", dtype=torch.int32)
  idx[idx == 4] = 3                                              # one expert without tokens
  plan = moe_ops.GroupPlan(idx, n_exp)
  rows = torch.zeros(plan.rows_max, D, device="cuda", dtype=torch.bfloat16)
  offs = plan.offs.tolist()
  sizes = plan.sizes.tolist()
  for e in range(n_exp):
    rows[offs[e]:offs[e] + sizes[e]] = torch.randn(sizes[e], D, device="cuda").bfloat16()
  w = (torch.randn(n_exp, Fd, D, device="cuda") * 0.1).bfloat16()
  rq, sr = E.quant_fp8_rows(rows)
  wq, _, sw = E.quant_fp8_blocks(w, True, False)
  out = torch.zeros(plan.rows_max, Fd, device="cuda", dtype=torch.bfloat16)
  E.gemm_fp8_block(rq, sr, wq, sw, False, out, plan.offs, plan.blk_expert)
  assert E.kernel_status(True) == 0
  a = _deq_rows(rq, sr)
  wd = _deq_blocks(wq, sw)
  for e in range(n_exp):
    sl = slice(offs[e], offs[e] + sizes[e])
    ref = a[sl] @ wd[e].t()
    if sizes[e]:
      assert torch.allclose(out[sl].float(), ref, atol=8e-3 * float(ref.abs().max()), rtol=8e-3), e


def test_block_scaled_linear_and_expert_ffn_close_to_bf16():
  """The autograd paths under quantization=fp8 with block scaling: dense linear and the padded expert FFN."""
  from maxtext_b200.ops import functional as F, moe_ops, quantization as Q
  from maxtext_b200.parallel.param_store import Param, ParamDef
  torch.manual_seed(8)

  def make(shape):
    q = Param(ParamDef(name="w", unit="u", shape=tuple(shape), ref_path=("w",), ref_shape=tuple(shape), logical_axes=(None,) * len(shape)))
    q.data = (torch.randn(*shape, device="cuda") * 0.05).bfloat16()
    q.main_grad = torch.zeros(*shape, device="cuda")
    return q

  def run(block):
    Q.set_mode("fp8" if block else "")
    Q.set_block_scaling(block)
    try:
      torch.manual_seed(9)
      x = (torch.randn(384, 512, device="cuda") * 0.5).bfloat16().requires_grad_()
      p = make((256, 512))
      y = F.linear(x, p)
      y.float().square().sum().backward()
      n_exp, Fd = 4, 256
      ws = [make(shape) for shape in ((n_exp, Fd, 512), (n_exp, Fd, 512), (n_exp, 512, Fd))]
      x2 = (torch.randn(384, 512, device="cuda") * 0.5).bfloat16().requires_grad_()
      idx = torch.randint(0, n_exp, (384, 2), device="cuda", dtype=torch.int32)
      wts = torch.rand(384, 2, device="cuda")
      o = moe_ops.moe_ffn_padded(x2, wts, idx, ws[0], ws[1], ws[2], n_exp, "silu")
      o.float().square().sum().backward()
      return [y.detach().float(), x.grad.float(), p.main_grad.clone(), o.detach().float(), x2.grad.float()] + [q.main_grad.clone() for q in ws]
    finally:
      Q.set_mode("")
      Q.set_block_scaling(False)

  ref, got = run(False), run(True)
  E = _ext()
  assert E.kernel_status(True) == 0
  for i, (r, g) in enumerate(zip(ref, got)):
    rel = float((r - g).norm() / r.norm())
    assert rel < 0.08, (i, rel)
    assert rel > 0 or i in (2,), i          # the 8-bit path really ran (the weight gradient of the dense layer stays bf16-exact only by chance)
