"""tcgen05 GEMM vs an fp32 PyTorch reference: every operand layout, both output types, accumulate,
ragged sizes (not multiples of the 128 x 256 x 64 tile)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ext():
  from maxtext_b200.ops import backend
  return backend.ext(required=True)


def _run(M, N, K, ta, tb, out_dtype, accumulate=False, seed=0, pair=False):
  E = _ext()
  g = torch.Generator(device="cuda").manual_seed(seed)
  a = torch.randn((K, M) if ta else (M, K), device="cuda", generator=g).bfloat16()
  b = torch.randn((N, K) if tb else (K, N), device="cuda", generator=g).bfloat16()
  ref = (a.float().t() if ta else a.float()) @ (b.float().t() if tb else b.float())
  if accumulate:
    out = torch.randn(M, N, device="cuda", generator=g, dtype=out_dtype)
    ref = ref + out.float()
  else:
    out = torch.full((M, N), float("nan"), device="cuda", dtype=out_dtype)
  assert E.gemm_supported(a, b, out, ta, tb)
  (E.gemm_pair if pair else E.gemm)(a, b, out, ta, tb, accumulate)
  torch.cuda.synchronize()
  assert E.kernel_status(True) == 0, "a bounded wait inside the GEMM kernel timed out"
  err = (out.float() - ref).abs().max().item()
  scale = ref.abs().max().item()
  tol = (2e-2 if out_dtype == torch.bfloat16 else 2e-3) * max(scale, 1.0)
  assert err <= tol, f"M={M} N={N} K={K} ta={ta} tb={tb} {out_dtype}: max err {err} (scale {scale})"


def test_gemm_smallest_first():
  # the first launch of the kernel in a process: one tile, one k-block pass
  _run(128, 256, 64, False, True, torch.bfloat16)


@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_layouts(ta, tb, out_dtype):
  _run(512, 768, 320, ta, tb, out_dtype)


@pytest.mark.parametrize("M,N,K", [(136, 264, 72), (1000, 520, 200), (128, 128, 64), (4096, 1536, 1024), (2048, 14336, 512)])
def test_gemm_ragged_and_large(M, N, K):
  _run(M, N, K, False, True, torch.bfloat16)
  _run(M, N, K, True, False, torch.float32)


@pytest.mark.parametrize("M", [2526, 619, 131])
def test_gemm_row_count_not_a_multiple_of_eight(M):
  """Rows are the strided dimension of a non-transposed A and of the output: any count works (per-expert token groups)."""
  _run(M, 1408, 2048, False, True, torch.bfloat16)
  _run(M, 512, 256, False, False, torch.bfloat16)
  if M >= 512:
    _run(M, 512, 256, False, True, torch.bfloat16, pair=True)


def test_gemm_accumulate_fp32():
  _run(640, 512, 384, True, False, torch.float32, accumulate=True)
  _run(384, 1024, 256, False, True, torch.float32, accumulate=True)


def test_gemm_many_tiles_persistent():
  # more tiles than SMs: every CTA walks several tiles through both TMEM accumulator buffers
  _run(8192, 4096, 256, False, True, torch.bfloat16)


def test_gemm_strided_views():
  E = _ext()
  big = torch.randn(512, 1024, device="cuda").bfloat16()
  a = big[:, 256:768]           # [512, 512] view with leading stride 1024
  w = torch.randn(384, 512, device="cuda").bfloat16()
  out = torch.empty(512, 384, device="cuda", dtype=torch.bfloat16)
  E.gemm(a, w, out, False, True, False)
  torch.cuda.synchronize()
  assert E.kernel_status(True) == 0
  ref = a.float() @ w.float().t()
  assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()


def test_gemm_pair_smallest_first():
  # CTA-pair (cta_group::2) variant: one 256 x 256 tile, one k-block
  _run(256, 256, 64, False, True, torch.bfloat16, pair=True)


@pytest.mark.parametrize("ta,tb,out_dtype", [(False, True, torch.bfloat16), (False, False, torch.bfloat16), (True, False, torch.float32),
                                             (False, True, torch.float32)])
def test_gemm_pair_layouts(ta, tb, out_dtype):
  _run(512, 768, 320, ta, tb, out_dtype, pair=True)


@pytest.mark.parametrize("M,N,K", [(384, 384, 192), (1000, 640, 72), (4096, 4096, 1024), (8192, 1536, 4096)])
def test_gemm_pair_ragged_and_large(M, N, K):
  _run(M, N, K, False, True, torch.bfloat16, pair=True)


def test_gemm_pair_accumulate_fp32():
  _run(512, 512, 256, True, False, torch.float32, accumulate=True, pair=True)


@pytest.mark.parametrize("M", [1, 5, 8, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("N,K", [(16, 64), (100, 192), (4096, 4096), (1000, 1024)])
def test_small_m_weight_streaming_gemm(M, N, K):
  """Decode-sized products (M <= 64): out = x @ W.T against an fp32 reference, all activation-tile counts, ragged N."""
  E = _ext()
  g = torch.Generator(device="cuda").manual_seed(M * 1000 + N)
  x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
  w = torch.randn(N, K, device="cuda", generator=g).bfloat16()
  out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
  assert E.gemm_small_m_supported(x, w, out)
  E.gemm_small_m(x, w, out)
  torch.cuda.synchronize()
  ref = x.float() @ w.float().t()
  err = (out.float() - ref).abs().max().item()
  assert err <= 2e-2 * max(ref.abs().max().item(), 1.0), f"M={M} N={N} K={K}: max err {err}"


def test_small_m_gemm_strided_views_and_dispatch():
  """Row-strided activations / weights / outputs, and `functional.mm` routing M <= 64 to the streaming kernel (no library call)."""
  from maxtext_b200.ops import functional as F
  E = _ext()
  g = torch.Generator(device="cuda").manual_seed(3)
  xb = torch.randn(12, 640, device="cuda", generator=g).bfloat16()
  wb = torch.randn(300, 640, device="cuda", generator=g).bfloat16()
  ob = torch.zeros(12, 512, device="cuda", dtype=torch.bfloat16)
  x, w, out = xb[:, 128:512], wb[:, 256:640], ob[:, :300]
  assert E.gemm_small_m_supported(x, w, out)
  E.gemm_small_m(x, w, out)
  ref = x.float() @ w.float().t()
  assert (out.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
  assert float(ob[:, 300:].abs().max()) == 0.0                 # nothing is written past N
  before = F.gemm_fallbacks()
  y = F.mm(xb, wb, False, True)
  assert F.gemm_fallbacks() == before
  ref2 = xb.float() @ wb.float().t()
  assert (y.float() - ref2).abs().max().item() <= 2e-2 * ref2.abs().max().item()
  # K not a multiple of 64 is not covered: the caller falls back and counts it
  assert not E.gemm_small_m_supported(xb[:, :40].contiguous(), wb[:, :40].contiguous(), torch.empty(12, 300, device="cuda", dtype=torch.bfloat16))
