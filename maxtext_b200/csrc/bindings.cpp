// PyTorch bindings for the sm_100a kernel library. Kernels live in plain .cu files with C launchers
// (raw pointers + stream); this file only validates tensors and forwards them.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>
#include <atomic>

extern "C" {
int mt_gemm_bf16(const void* a, const void* b, void* c, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int a_mn, int b_mn,
                 int out_f32, int accumulate, int* status, int num_sms, cudaStream_t stream);
int mt_rmsnorm_fwd(const void* x, const void* scale, float eps, float offset, void* y, float* rstd, int rows, int D, cudaStream_t st);
int mt_rmsnorm_bwd(const void* dy, const void* x, const void* scale, const float* rstd, float offset, void* dx, float* dscale,
                   float* partial, int rows, int D, int sms, cudaStream_t st);
int mt_rmsnorm_bwd_partial_rows(int rows, int D, int sms);
int mt_rope(void* x, const int* pos, const float* inv_ts, long tokens, int heads, int dh, int n_rot, int rot_dim, int interleaved,
            int inverse, cudaStream_t st);
int mt_gated_act_fwd(const void* gu, void* out, long rows, int F, int code, int sms, cudaStream_t st);
int mt_gated_act_bwd(const void* dy, const void* gu, void* dgu, long rows, int F, int code, int sms, cudaStream_t st);
int mt_embedding_fwd(const int* tok, const void* table, void* out, long tokens, int D, int V, cudaStream_t st);
int mt_embedding_bwd(const int* tok, const void* dy, float* dtable, long tokens, int D, int V, cudaStream_t st);
int mt_xent(void* logits, const int* targets, const float* weights, float z_loss, float* loss_out, float* z_out, long rows, long ld,
            int V, int write_grad, cudaStream_t st);
int mt_adamw(float* p, const float* g, void* m, int m_is_bf16, float* v, void* shadow, long n, float lr, float b1, float b2, float eps,
             float eps_root, float wd, float bc1, float bc2, const float* grad_scale, int sms, cudaStream_t st);
int mt_amax(const void* x, long n, float* amax, int sms, cudaStream_t st);
int mt_quantize_fp8(const void* x, int R, int C, const float* amax, int fmt, void* q, void* qt, float* dequant, cudaStream_t st);
int mt_gemm_fp8(const void* a, const void* b, void* c, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int a_fmt, int b_fmt,
                int out_f32, int accumulate, const float* scale_a, const float* scale_b, int* status, int num_sms, cudaStream_t stream);
int mt_gemm_set_group_m(int v);
int mt_gemm_set_raster(int v);
int mt_gemm_bf16_pair(const void* a, const void* b, void* c, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int a_mn, int b_mn,
                      int out_f32, int accumulate, int* status, int num_sms, cudaStream_t stream);
int mt_gemm_fp8_pair(const void* a, const void* b, void* c, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int a_fmt, int b_fmt,
                     int out_f32, int accumulate, const float* scale_a, const float* scale_b, int* status, int num_sms, cudaStream_t stream);
int mt_sumsq_num_partials(long n, int sms);
int mt_sumsq(const float* x, long n, float* partials, float* out, int sms, cudaStream_t st);
}

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int num_sms() {
  static int sms[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && sms[dev]) return sms[dev];
  int n = 0;
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (dev < 64) sms[dev] = n;
  return n;
}

// one status word per device, written by kernels whose bounded waits ran out
torch::Tensor& status_tensor() {
  static std::vector<torch::Tensor> st(64);
  int dev = 0;
  cudaGetDevice(&dev);
  if (!st[dev].defined()) st[dev] = torch::zeros({1}, torch::dtype(torch::kInt32).device(torch::kCUDA, dev));
  return st[dev];
}

// kernels launched through this module since load (benchmarks report the count of a timed region)
std::atomic<int64_t> g_launches{0};

void check(int rc, const char* what, int launches = 1) {
  TORCH_CHECK(rc == 0, what, " failed with code ", rc);
  g_launches.fetch_add(launches, std::memory_order_relaxed);
}

int64_t launch_count() { return g_launches.load(std::memory_order_relaxed); }

bool is2d_rowmajor(const torch::Tensor& t, int align_elems) {
  return t.dim() == 2 && t.stride(1) == 1 && t.stride(0) % align_elems == 0 && t.stride(0) >= t.size(1) &&
         (reinterpret_cast<uintptr_t>(t.data_ptr()) % 16) == 0;
}

// C[M,N] (+)= op(a) op(b): op(a) = a^T if ta (a stored [K,M]), op(b) = b^T if tb (b stored [N,K]).
bool gemm_supported(const torch::Tensor& a, const torch::Tensor& b, const torch::Tensor& out, bool ta, bool tb) {
  if (!a.is_cuda() || a.scalar_type() != torch::kBFloat16 || b.scalar_type() != torch::kBFloat16) return false;
  if (out.scalar_type() != torch::kBFloat16 && out.scalar_type() != torch::kFloat32) return false;
  if (!is2d_rowmajor(a, 8) || !is2d_rowmajor(b, 8)) return false;
  if (!is2d_rowmajor(out, out.scalar_type() == torch::kFloat32 ? 4 : 8)) return false;
  const int64_t M = ta ? a.size(1) : a.size(0), K = ta ? a.size(0) : a.size(1), N = tb ? b.size(0) : b.size(1);
  if ((tb ? b.size(1) : b.size(0)) != K || out.size(0) != M || out.size(1) != N) return false;
  // M is a contiguous dimension only of a transposed A; elsewhere TMA clips the ragged last row block
  return M >= 128 && N >= 128 && K >= 64 && (!ta || M % 8 == 0) && N % 8 == 0 && K % 8 == 0;
}

extern "C" int mt_gemm_small_m_supported(int M, int N, int K, long ldx, long ldw, long ldo);
extern "C" int mt_gemm_small_m(const void* x, const void* w, void* out, int M, int N, int K, long ldx, long ldw, long ldo, int num_sms, cudaStream_t stream);

// out[M, N] = x[M, K] w[N, K]^T for M <= 64 (decode): the weight-streaming kernel of gemm_small_m.cu
bool gemm_small_m_supported(const torch::Tensor& x, const torch::Tensor& w, const torch::Tensor& out) {
  if (!x.is_cuda() || x.scalar_type() != torch::kBFloat16 || w.scalar_type() != torch::kBFloat16 || out.scalar_type() != torch::kBFloat16) return false;
  if (x.dim() != 2 || w.dim() != 2 || out.dim() != 2 || x.stride(1) != 1 || w.stride(1) != 1 || out.stride(1) != 1) return false;
  if (x.size(1) != w.size(1) || out.size(0) != x.size(0) || out.size(1) != w.size(0)) return false;
  if (reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 || reinterpret_cast<uintptr_t>(w.data_ptr()) % 16) return false;
  return mt_gemm_small_m_supported((int)x.size(0), (int)w.size(0), (int)x.size(1), x.stride(0), w.stride(0), out.stride(0)) != 0;
}

void gemm_small_m(const torch::Tensor& x, const torch::Tensor& w, torch::Tensor& out) {
  TORCH_CHECK(gemm_small_m_supported(x, w, out), "gemm_small_m: unsupported operands");
  c10::cuda::CUDAGuard guard(x.device());
  check(mt_gemm_small_m(x.data_ptr(), w.data_ptr(), out.data_ptr(), (int)x.size(0), (int)w.size(0), (int)x.size(1), x.stride(0), w.stride(0),
                        out.stride(0), num_sms(), cur_stream()),
        "mt_gemm_small_m");
}

// CTA-pair (cta_group::2) kernel for shapes it covers: measured 3-10 % faster than the single-CTA kernel under sustained load
bool g_use_pair = true;

void gemm(const torch::Tensor& a, const torch::Tensor& b, torch::Tensor& out, bool ta, bool tb, bool accumulate) {
  TORCH_CHECK(gemm_supported(a, b, out, ta, tb), "gemm: unsupported operands");
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = ta ? a.size(1) : a.size(0), K = ta ? a.size(0) : a.size(1), N = tb ? b.size(0) : b.size(1);
  const bool f32 = out.scalar_type() == torch::kFloat32;
  TORCH_CHECK(!accumulate || f32, "gemm: accumulate requires an fp32 output");
  if (g_use_pair && N % 256 == 0 && M >= 512) {
    int rc = mt_gemm_bf16_pair(a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), b.stride(0), out.stride(0),
                               ta ? 1 : 0, tb ? 0 : 1, f32 ? 1 : 0, accumulate ? 1 : 0, status_tensor().data_ptr<int>(), num_sms(),
                               cur_stream());
    check(rc, "mt_gemm_bf16_pair");
    return;
  }
  int rc = mt_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), b.stride(0), out.stride(0),
                        ta ? 1 : 0, tb ? 0 : 1, f32 ? 1 : 0, accumulate ? 1 : 0, status_tensor().data_ptr<int>(), num_sms(), cur_stream());
  check(rc, "mt_gemm_bf16");
}

// x [R, C] bf16 -> (q [R, C] uint8 or None, qt [C, R] uint8 or None, dequant scale [1]); fmt 0 = E4M3, 1 = E5M2. Current scaling:
// the scale comes from this tensor's own absolute maximum, computed on the device.
std::tuple<c10::optional<torch::Tensor>, c10::optional<torch::Tensor>, torch::Tensor, torch::Tensor> quantize_fp8_with(
    const torch::Tensor& x, int64_t fmt, bool want_q, bool want_t, const c10::optional<torch::Tensor>& amax_for_scale);

std::tuple<c10::optional<torch::Tensor>, c10::optional<torch::Tensor>, torch::Tensor> quantize_fp8(const torch::Tensor& x, int64_t fmt,
                                                                                                     bool want_q, bool want_t) {
  auto r = quantize_fp8_with(x, fmt, want_q, want_t, c10::nullopt);
  return {std::get<0>(r), std::get<1>(r), std::get<2>(r)};
}

// As quantize_fp8, but the scale may come from `amax_for_scale` (delayed scaling: the maximum of an amax history) instead of
// this tensor's own maximum; the tensor's own amax is always computed and returned last, for the caller's history.
std::tuple<c10::optional<torch::Tensor>, c10::optional<torch::Tensor>, torch::Tensor, torch::Tensor> quantize_fp8_with(
    const torch::Tensor& x, int64_t fmt, bool want_q, bool want_t, const c10::optional<torch::Tensor>& amax_for_scale) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && x.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(x.size(0) % 64 == 0 && x.size(1) % 64 == 0, "quantize_fp8: dims must be multiples of 64");
  c10::cuda::CUDAGuard guard(x.device());
  auto fo = torch::dtype(torch::kFloat32).device(x.device());
  auto amax = torch::zeros({1}, fo);
  auto deq = torch::empty({1}, fo);
  check(mt_amax(x.data_ptr(), x.numel(), amax.data_ptr<float>(), num_sms(), cur_stream()), "mt_amax");
  c10::optional<torch::Tensor> q, qt;
  auto bo = torch::dtype(torch::kUInt8).device(x.device());
  if (want_q) q = torch::empty({x.size(0), x.size(1)}, bo);
  if (want_t) qt = torch::empty({x.size(1), x.size(0)}, bo);
  if (amax_for_scale) TORCH_CHECK(amax_for_scale->is_cuda() && amax_for_scale->scalar_type() == torch::kFloat32 && amax_for_scale->numel() == 1);
  const float* scale_src = amax_for_scale ? amax_for_scale->data_ptr<float>() : amax.data_ptr<float>();
  check(mt_quantize_fp8(x.data_ptr(), (int)x.size(0), (int)x.size(1), scale_src, (int)fmt, q ? q->data_ptr() : nullptr,
                        qt ? qt->data_ptr() : nullptr, deq.data_ptr<float>(), cur_stream()),
        "mt_quantize_fp8");
  return {q, qt, deq, amax};
}

// out [M, N] (+)= a [M, K] . b [N, K]^T * sa * sb, a / b uint8 holding E4M3 (fmt 0) or E5M2 (fmt 1)
void gemm_fp8(const torch::Tensor& a, const torch::Tensor& b, torch::Tensor& out, int64_t a_fmt, int64_t b_fmt, const torch::Tensor& sa,
              const torch::Tensor& sb, bool accumulate) {
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == torch::kUInt8 && b.scalar_type() == torch::kUInt8 && a.dim() == 2 && b.dim() == 2);
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && a.size(1) == b.size(1) && out.size(0) == a.size(0) && out.size(1) == b.size(0));
  TORCH_CHECK(a.size(1) % 128 == 0 && a.size(0) % 128 == 0 && b.size(0) % 128 == 0, "gemm_fp8: dims must be multiples of 128");
  const bool f32 = out.scalar_type() == torch::kFloat32;
  TORCH_CHECK((f32 || out.scalar_type() == torch::kBFloat16) && out.stride(1) == 1 && (!accumulate || f32));
  TORCH_CHECK(sa.scalar_type() == torch::kFloat32 && sb.scalar_type() == torch::kFloat32);
  c10::cuda::CUDAGuard guard(a.device());
  auto fn = (g_use_pair && b.size(0) % 256 == 0 && a.size(0) >= 512) ? mt_gemm_fp8_pair : mt_gemm_fp8;
  check(fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)a.size(0), (int)b.size(0), (int)a.size(1), a.stride(0), b.stride(0),
                    out.stride(0), (int)a_fmt, (int)b_fmt, f32 ? 1 : 0, accumulate ? 1 : 0, sa.data_ptr<float>(), sb.data_ptr<float>(),
                    status_tensor().data_ptr<int>(), num_sms(), cur_stream()),
        "mt_gemm_fp8");
}

// the CTA-pair (cta_group::2) variant of `gemm`; N must be a multiple of 128
void gemm_pair(const torch::Tensor& a, const torch::Tensor& b, torch::Tensor& out, bool ta, bool tb, bool accumulate) {
  TORCH_CHECK(gemm_supported(a, b, out, ta, tb), "gemm_pair: unsupported operands");
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = ta ? a.size(1) : a.size(0), K = ta ? a.size(0) : a.size(1), N = tb ? b.size(0) : b.size(1);
  TORCH_CHECK(N % 128 == 0 && M >= 256, "gemm_pair: N must be a multiple of 128 and M at least 256");
  const bool f32 = out.scalar_type() == torch::kFloat32;
  TORCH_CHECK(!accumulate || f32, "gemm_pair: accumulate requires an fp32 output");
  int rc = mt_gemm_bf16_pair(a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), b.stride(0), out.stride(0),
                             ta ? 1 : 0, tb ? 0 : 1, f32 ? 1 : 0, accumulate ? 1 : 0, status_tensor().data_ptr<int>(), num_sms(), cur_stream());
  check(rc, "mt_gemm_bf16_pair");
}

int64_t kernel_status(bool reset) {
  auto& st = status_tensor();
  int64_t v = st.item<int>();
  if (reset && v != 0) st.zero_();
  return v;
}

void rmsnorm_fwd(const torch::Tensor& x, const c10::optional<torch::Tensor>& scale, double eps, double offset, torch::Tensor& y,
                 const c10::optional<torch::Tensor>& rstd) {
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && x.dim() == 2);
  c10::cuda::CUDAGuard guard(x.device());
  check(mt_rmsnorm_fwd(x.data_ptr(), scale ? scale->data_ptr() : nullptr, (float)eps, (float)offset, y.data_ptr(),
                       rstd ? rstd->data_ptr<float>() : nullptr, (int)x.size(0), (int)x.size(1), cur_stream()),
        "mt_rmsnorm_fwd");
}

void rmsnorm_bwd(const torch::Tensor& dy, const torch::Tensor& x, const c10::optional<torch::Tensor>& scale, const torch::Tensor& rstd,
                 double offset, torch::Tensor& dx, const c10::optional<torch::Tensor>& dscale) {
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous() && dx.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  torch::Tensor partial;
  if (dscale) partial = torch::empty({mt_rmsnorm_bwd_partial_rows((int)x.size(0), (int)x.size(1), num_sms()), x.size(1)},
                                     torch::TensorOptions().dtype(torch::kFloat32).device(x.device()));
  check(mt_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), scale ? scale->data_ptr() : nullptr, rstd.data_ptr<float>(), (float)offset,
                       dx.data_ptr(), dscale ? dscale->data_ptr<float>() : nullptr, dscale ? partial.data_ptr<float>() : nullptr,
                       (int)x.size(0), (int)x.size(1), num_sms(), cur_stream()),
        "mt_rmsnorm_bwd");
}

void rope_inplace(torch::Tensor& x, const torch::Tensor& pos, const torch::Tensor& inv_ts, int64_t n_rot, bool interleaved, bool inverse,
                  int64_t rot_dim) {
  TORCH_CHECK(x.is_contiguous() && x.dim() == 3 && pos.scalar_type() == torch::kInt32 && inv_ts.scalar_type() == torch::kFloat32);
  TORCH_CHECK(pos.numel() == x.size(0) && inv_ts.numel() >= rot_dim / 2 && n_rot <= x.size(1) && rot_dim <= x.size(2));
  c10::cuda::CUDAGuard guard(x.device());
  check(mt_rope(x.data_ptr(), pos.data_ptr<int>(), inv_ts.data_ptr<float>(), x.size(0), (int)x.size(1), (int)x.size(2), (int)n_rot,
                (int)rot_dim, interleaved, inverse, cur_stream()),
        "mt_rope");
}

void gated_act_fwd(const torch::Tensor& gu, torch::Tensor& out, int64_t code) {
  TORCH_CHECK(gu.is_contiguous() && out.is_contiguous() && gu.size(1) == 2 * out.size(1));
  c10::cuda::CUDAGuard guard(gu.device());
  check(mt_gated_act_fwd(gu.data_ptr(), out.data_ptr(), gu.size(0), (int)out.size(1), (int)code, num_sms(), cur_stream()), "gated_act_fwd");
}

void gated_act_bwd(const torch::Tensor& dy, const torch::Tensor& gu, torch::Tensor& dgu, int64_t code) {
  TORCH_CHECK(gu.is_contiguous() && dy.is_contiguous() && dgu.is_contiguous());
  c10::cuda::CUDAGuard guard(gu.device());
  check(mt_gated_act_bwd(dy.data_ptr(), gu.data_ptr(), dgu.data_ptr(), gu.size(0), (int)dy.size(1), (int)code, num_sms(), cur_stream()),
        "gated_act_bwd");
}

void embedding_fwd(const torch::Tensor& tok, const torch::Tensor& table, torch::Tensor& out) {
  TORCH_CHECK(tok.scalar_type() == torch::kInt32 && table.is_contiguous() && out.is_contiguous());
  c10::cuda::CUDAGuard guard(table.device());
  check(mt_embedding_fwd(tok.data_ptr<int>(), table.data_ptr(), out.data_ptr(), tok.numel(), (int)table.size(1), (int)table.size(0),
                         cur_stream()),
        "embedding_fwd");
}

void embedding_bwd(const torch::Tensor& tok, const torch::Tensor& dy, torch::Tensor& dtable) {
  TORCH_CHECK(tok.scalar_type() == torch::kInt32 && dy.is_contiguous() && dtable.is_contiguous() &&
              dtable.scalar_type() == torch::kFloat32);
  c10::cuda::CUDAGuard guard(dy.device());
  check(mt_embedding_bwd(tok.data_ptr<int>(), dy.data_ptr(), dtable.data_ptr<float>(), tok.numel(), (int)dtable.size(1),
                         (int)dtable.size(0), cur_stream()),
        "embedding_bwd");
}

void xent_fwd_bwd(torch::Tensor& logits, const torch::Tensor& targets, const torch::Tensor& weights, double z_loss, torch::Tensor& loss,
                  torch::Tensor& z, bool write_grad) {
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && logits.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(targets.scalar_type() == torch::kInt32 && weights.scalar_type() == torch::kFloat32);
  c10::cuda::CUDAGuard guard(logits.device());
  check(mt_xent(logits.data_ptr(), targets.data_ptr<int>(), weights.data_ptr<float>(), (float)z_loss, loss.data_ptr<float>(),
                z.data_ptr<float>(), logits.size(0), logits.stride(0), (int)logits.size(1), write_grad, cur_stream()),
        "mt_xent");
}

void adamw(torch::Tensor& p, const torch::Tensor& g, torch::Tensor& m, torch::Tensor& v, const c10::optional<torch::Tensor>& shadow,
           double lr, double b1, double b2, double eps, double eps_root, double wd, double bc1, double bc2,
           const torch::Tensor& grad_scale) {
  TORCH_CHECK(p.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous());
  TORCH_CHECK(p.numel() == g.numel() && p.numel() == m.numel() && p.numel() == v.numel());
  c10::cuda::CUDAGuard guard(p.device());
  check(mt_adamw(p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr(), m.scalar_type() == torch::kBFloat16, v.data_ptr<float>(),
                 shadow ? shadow->data_ptr() : nullptr, p.numel(), (float)lr, (float)b1, (float)b2, (float)eps, (float)eps_root,
                 (float)wd, (float)bc1, (float)bc2, grad_scale.data_ptr<float>(), num_sms(), cur_stream()),
        "mt_adamw");
}

void sumsq(const torch::Tensor& x, torch::Tensor& out) {
  TORCH_CHECK(x.is_contiguous() && x.scalar_type() == torch::kFloat32 && out.scalar_type() == torch::kFloat32);
  c10::cuda::CUDAGuard guard(x.device());
  const int parts = mt_sumsq_num_partials(x.numel(), num_sms());
  auto partials = torch::empty({parts}, x.options());
  check(mt_sumsq(x.data_ptr<float>(), x.numel(), partials.data_ptr<float>(), out.data_ptr<float>(), num_sms(), cur_stream()), "mt_sumsq", 2);
}

}  // namespace

int* mt_status_ptr() { return status_tensor().data_ptr<int>(); }
void mt_count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int mt_num_sms() { return num_sms(); }

void register_attention(pybind11::module_& m);
void register_moe(pybind11::module_& m);
void register_comm(pybind11::module_& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm_supported", &gemm_supported);
  m.def("gemm", &gemm);
  m.def("gemm_small_m_supported", &gemm_small_m_supported);
  m.def("gemm_small_m", &gemm_small_m);
  m.def("gemm_pair", &gemm_pair);
  m.def("gemm_use_pair", [](bool v) { g_use_pair = v; });
  m.def("gemm_set_raster", [](int64_t v) { mt_gemm_set_raster((int)v); });
  m.def("gemm_set_group_m", [](int64_t v) { TORCH_CHECK(mt_gemm_set_group_m((int)v) == 0, "bad group size"); });
  m.def("quantize_fp8", &quantize_fp8);
  m.def("quantize_fp8_with", &quantize_fp8_with);
  m.def("gemm_fp8", &gemm_fp8);
  m.def("kernel_status", &kernel_status);
  m.def("launch_count", &launch_count);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rope_inplace", &rope_inplace);
  m.def("gated_act_fwd", &gated_act_fwd);
  m.def("gated_act_bwd", &gated_act_bwd);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("xent_fwd_bwd", &xent_fwd_bwd);
  m.def("adamw", &adamw);
  m.def("sumsq", &sumsq);
  register_attention(m);
  register_moe(m);
  register_comm(m);
}
