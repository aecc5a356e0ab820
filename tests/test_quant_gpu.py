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
