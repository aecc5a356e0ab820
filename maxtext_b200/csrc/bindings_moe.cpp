// Bindings for the mixture-of-experts kernels (stable padded sort, row gather / combine, grouped GEMM).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>

extern "C" {
int mt_quant_fp8_rows(const void* x, long R, int C, long ldx, void* q, float* scales_t, cudaStream_t st);
int mt_quant_fp8_blocks(const void* w, int G, int R, int C, void* q, void* qt, float* scales, cudaStream_t st);
int mt_gemm_fp8_block(const void* aq, const void* bq, void* c, int M, int N, int K, long lda, long ldb, long ldc, const float* sa, const float* sb,
                      long sb_e, long sb_n, long sb_k, int experts, const int* x_offs, const int* blk_expert, int* status, int num_sms,
                      cudaStream_t st);
int mt_router_topk(const void* logits, int is_bf16, const float* bias, long tokens, int E, int k, int mode, int sigmoid_scores, int raw_weights,
                   float scaling, int* idx, float* wts, float* probs, int* counts, cudaStream_t st);
int mt_moe_sort(const int* idx, int n, int E, int rows_max, int* sizes, int* offs, int* blk_expert, int* dest, int* row_pair, cudaStream_t st);
int mt_moe_gather(const void* x, const int* row_pair, const int* offs, int E, int k, int D, int rows_max, void* rows, int sms, cudaStream_t st);
int mt_moe_combine(const void* y, const int* dest, const float* w, int T, int k, int D, void* out, int sms, cudaStream_t st);
int mt_moe_combine_bwd(const void* dout, const void* y, const int* row_pair, const int* offs, int E, const float* w, int k, int D,
                       int rows_max, void* dy, float* dw, int sms, cudaStream_t st);
int mt_gemm_bf16_grouped(int mode, const void* a, const void* b, void* c, int rows_max, int n_out, int k_in, int experts, const int* offs,
                         const int* blk_expert, int accumulate, long lda, long ldb, long ldc, int* status, int num_sms, cudaStream_t stream);
int mt_ep_put_counts(const int* sizes, int E, int my_rank, int ep, int* const* counts_peer, cudaStream_t st);
int mt_ep_index(const int* counts, int ep, int E, int my_rank, int cap, int* offs, int* blk_expert, int* valid_rows, int* send_base,
                int* status, cudaStream_t st);
int mt_ep_push(const void* src, int src_div, const int* idx, const int* dest_local, const int* offs_local, const int* send_base, int n,
               int el, int cap, int D, void* const* peer_buf, int* pair_owner, int* pair_row, int sms, cudaStream_t st);
int mt_ep_pull(void* const* peer_buf, const int* pair_owner, const int* pair_row, int n, int cap, int D, void* out, int sms, cudaStream_t st);
int mt_ep_zero_pads(void* buf, const int* offs, const int* valid_rows, int el, int D, cudaStream_t st);
}

int* mt_status_ptr();          // defined in bindings.cpp
void mt_count_launches(int n); // defined in bindings.cpp
int mt_num_sms();              // defined in bindings.cpp

namespace {

cudaStream_t cur() { return at::cuda::getCurrentCUDAStream().stream(); }

bool i32(const torch::Tensor& t) { return t.is_cuda() && t.is_contiguous() && t.scalar_type() == torch::kInt32; }
bool bf16_rows(const torch::Tensor& t) {
  return t.is_cuda() && t.dim() == 2 && t.scalar_type() == torch::kBFloat16 && t.stride(1) == 1 && t.stride(0) % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(t.data_ptr()) % 16) == 0;
}

// idx [n] int32 -> fills sizes [E], offs [E+1], blk_expert [rows_max/128], dest [n], row_pair [rows_max]
// ---- block-scaled FP8 (gemm_fp8_block_sm100.cu)
// x [R, C] bf16 -> (q [R, C] uint8 holding e4m3, scales_t [ceil(C/128), R] fp32)
std::vector<torch::Tensor> quant_fp8_rows(const torch::Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 && x.stride(0) % 4 == 0 && x.scalar_type() == torch::kBFloat16 && x.size(1) % 16 == 0 &&
              (reinterpret_cast<uintptr_t>(x.data_ptr()) % 8) == 0);
  c10::cuda::CUDAGuard guard(x.device());
  auto q = torch::empty({x.size(0), x.size(1)}, torch::dtype(torch::kUInt8).device(x.device()));
  auto s = torch::empty({(x.size(1) + 127) / 128, x.size(0)}, torch::dtype(torch::kFloat32).device(x.device()));
  int rc = mt_quant_fp8_rows(x.data_ptr(), x.size(0), (int)x.size(1), x.stride(0), q.data_ptr(), s.data_ptr<float>(), cur());
  TORCH_CHECK(rc == 0, "mt_quant_fp8_rows failed with code ", rc);
  mt_count_launches(1);
  return {q, s};
}

// w [R, C] or [G, R, C] bf16 -> (q or None, qt [.., C, R] or None, scales [G, ceil(R/128), ceil(C/128)])
std::vector<c10::optional<torch::Tensor>> quant_fp8_blocks(const torch::Tensor& w, bool want_q, bool want_t) {
  TORCH_CHECK(w.is_cuda() && (w.dim() == 2 || w.dim() == 3) && w.is_contiguous() && w.scalar_type() == torch::kBFloat16);
  const int64_t G = w.dim() == 3 ? w.size(0) : 1, R = w.size(w.dim() - 2), C = w.size(w.dim() - 1);
  TORCH_CHECK(R % 16 == 0 && C % 16 == 0, "quant_fp8_blocks: dims must be multiples of 16");
  c10::cuda::CUDAGuard guard(w.device());
  auto o8 = torch::dtype(torch::kUInt8).device(w.device());
  c10::optional<torch::Tensor> q, qt;
  if (want_q) q = torch::empty({G, R, C}, o8);
  if (want_t) qt = torch::empty({G, C, R}, o8);
  auto s = torch::empty({G, (R + 127) / 128, (C + 127) / 128}, torch::dtype(torch::kFloat32).device(w.device()));
  int rc = mt_quant_fp8_blocks(w.data_ptr(), (int)G, (int)R, (int)C, q ? q->data_ptr() : nullptr, qt ? qt->data_ptr() : nullptr,
                               s.data_ptr<float>(), cur());
  TORCH_CHECK(rc == 0, "mt_quant_fp8_blocks failed with code ", rc);
  mt_count_launches(1);
  return {q, qt, s};
}

// out [M, N] bf16 = aq [M, K] (e4m3, scales sa [KB, M]) x bq [G, N, K]^T (e4m3, scales sb [G, NB', KB'] read as element
// (e, nb, kb) = sb[e][nb][kb], or with `sb_transposed` as sb[e][kb][nb]: the table of the un-transposed weight). Grouped when
// offs / blk_expert are given (rows grouped by expert, padded to 128 per group).
void gemm_fp8_block(const torch::Tensor& aq, const torch::Tensor& sa, const torch::Tensor& bq, const torch::Tensor& sb, bool sb_transposed,
                    torch::Tensor& out, const c10::optional<torch::Tensor>& offs, const c10::optional<torch::Tensor>& blk_expert) {
  TORCH_CHECK(aq.is_cuda() && aq.dim() == 2 && aq.scalar_type() == torch::kUInt8 && aq.stride(1) == 1 && bq.dim() == 3 && bq.is_contiguous() &&
              bq.scalar_type() == torch::kUInt8 && sb.dim() == 3 && sb.is_contiguous() && sa.is_contiguous() && sa.scalar_type() == torch::kFloat32 &&
              sb.scalar_type() == torch::kFloat32 && out.dim() == 2 && out.stride(1) == 1 && out.scalar_type() == torch::kBFloat16);
  const int64_t M = aq.size(0), K = aq.size(1), G = bq.size(0), N = bq.size(1);
  TORCH_CHECK(bq.size(2) == K && out.size(0) == M && out.size(1) == N && sa.size(0) == (K + 127) / 128 && sa.size(1) == M);
  const bool grouped = offs.has_value();
  if (grouped) {
    TORCH_CHECK(i32(*offs) && blk_expert && i32(*blk_expert) && offs->numel() == G + 1 && blk_expert->numel() * 128 == M);
  } else {
    TORCH_CHECK(G == 1);
  }
  const int64_t NB = (N + 127) / 128, KB = (K + 127) / 128;
  TORCH_CHECK(sb.size(0) == G && sb.size(1) == (sb_transposed ? KB : NB) && sb.size(2) == (sb_transposed ? NB : KB));
  c10::cuda::CUDAGuard guard(aq.device());
  int rc = mt_gemm_fp8_block(aq.data_ptr(), bq.data_ptr(), out.data_ptr(), (int)M, (int)N, (int)K, aq.stride(0), K, out.stride(0),
                             sa.data_ptr<float>(), sb.data_ptr<float>(), sb.stride(0), sb_transposed ? 1 : sb.stride(1),
                             sb_transposed ? sb.stride(1) : 1, grouped ? (int)G : 0, grouped ? offs->data_ptr<int>() : nullptr,
                             grouped ? blk_expert->data_ptr<int>() : nullptr, mt_status_ptr(), mt_num_sms(), cur());
  TORCH_CHECK(rc == 0, "mt_gemm_fp8_block failed with code ", rc);
  mt_count_launches(1);
}

// logits [T,E] fp32 / bf16 -> (idx [T,k] int32, wts [T,k] fp32, probs [T,E] fp32, counts [E] int32), see router_sm100.cu
std::vector<torch::Tensor> router_topk(const torch::Tensor& logits, const c10::optional<torch::Tensor>& bias, int64_t k, int64_t mode,
                                       bool sigmoid_scores, bool raw_weights, double scaling) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous() &&
              (logits.scalar_type() == torch::kFloat32 || logits.scalar_type() == torch::kBFloat16));
  const int64_t T = logits.size(0), E = logits.size(1);
  if (bias) TORCH_CHECK(bias->is_cuda() && bias->is_contiguous() && bias->scalar_type() == torch::kFloat32 && bias->numel() == E);
  c10::cuda::CUDAGuard guard(logits.device());
  auto oi = torch::TensorOptions().dtype(torch::kInt32).device(logits.device());
  auto of = torch::TensorOptions().dtype(torch::kFloat32).device(logits.device());
  auto idx = torch::empty({T, k}, oi), counts = torch::zeros({E}, oi);
  auto wts = torch::empty({T, k}, of), probs = torch::empty({T, E}, of);
  int rc = mt_router_topk(logits.data_ptr(), logits.scalar_type() == torch::kBFloat16 ? 1 : 0, bias ? bias->data_ptr<float>() : nullptr, T, (int)E,
                          (int)k, (int)mode, sigmoid_scores ? 1 : 0, raw_weights ? 1 : 0, (float)scaling, idx.data_ptr<int>(),
                          wts.data_ptr<float>(), probs.data_ptr<float>(), counts.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "mt_router_topk failed with code ", rc);
  mt_count_launches(1);
  return {idx, wts, probs, counts};
}

void moe_sort(const torch::Tensor& idx, int64_t E, torch::Tensor& sizes, torch::Tensor& offs, torch::Tensor& blk_expert, torch::Tensor& dest,
              torch::Tensor& row_pair) {
  TORCH_CHECK(i32(idx) && i32(sizes) && i32(offs) && i32(blk_expert) && i32(dest) && i32(row_pair));
  const int64_t n = idx.numel(), rows_max = row_pair.numel();
  TORCH_CHECK(sizes.numel() == E && offs.numel() == E + 1 && dest.numel() == n && blk_expert.numel() * 128 == rows_max);
  TORCH_CHECK(rows_max >= n + E * 127 || rows_max >= (n + 127) / 128 * 128 + E * 128 - 128, "rows_max too small for the padded layout");
  c10::cuda::CUDAGuard guard(idx.device());
  int rc = mt_moe_sort(idx.data_ptr<int>(), (int)n, (int)E, (int)rows_max, sizes.data_ptr<int>(), offs.data_ptr<int>(),
                       blk_expert.data_ptr<int>(), dest.data_ptr<int>(), row_pair.data_ptr<int>(), cur());
  TORCH_CHECK(rc == 0, "mt_moe_sort failed with code ", rc);
  mt_count_launches(1);
}

void moe_gather(const torch::Tensor& x, const torch::Tensor& row_pair, const torch::Tensor& offs, int64_t k, torch::Tensor& rows) {
  TORCH_CHECK(x.is_contiguous() && rows.is_contiguous() && bf16_rows(x) && bf16_rows(rows) && x.size(1) == rows.size(1));
  TORCH_CHECK(i32(row_pair) && i32(offs) && row_pair.numel() == rows.size(0));
  c10::cuda::CUDAGuard guard(x.device());
  int rc = mt_moe_gather(x.data_ptr(), row_pair.data_ptr<int>(), offs.data_ptr<int>(), (int)offs.numel() - 1, (int)k, (int)x.size(1),
                         (int)rows.size(0), rows.data_ptr(), mt_num_sms(), cur());
  TORCH_CHECK(rc == 0, "mt_moe_gather failed with code ", rc);
  mt_count_launches(1);
}

// out[t] = sum_c w[t,c] * y[dest[t*k+c]]; w undefined -> plain sum
void moe_combine(const torch::Tensor& y, const torch::Tensor& dest, const c10::optional<torch::Tensor>& w, int64_t k, torch::Tensor& out) {
  TORCH_CHECK(y.is_contiguous() && out.is_contiguous() && bf16_rows(y) && bf16_rows(out) && y.size(1) == out.size(1) && i32(dest));
  TORCH_CHECK(dest.numel() == out.size(0) * k);
  if (w) TORCH_CHECK(w->is_contiguous() && w->scalar_type() == torch::kFloat32 && w->numel() == dest.numel());
  c10::cuda::CUDAGuard guard(y.device());
  int rc = mt_moe_combine(y.data_ptr(), dest.data_ptr<int>(), w ? w->data_ptr<float>() : nullptr, (int)out.size(0), (int)k, (int)y.size(1),
                          out.data_ptr(), mt_num_sms(), cur());
  TORCH_CHECK(rc == 0, "mt_moe_combine failed with code ", rc);
  mt_count_launches(1);
}

void moe_combine_bwd(const torch::Tensor& dout, const torch::Tensor& y, const torch::Tensor& row_pair, const torch::Tensor& offs,
                     const torch::Tensor& w, int64_t k, torch::Tensor& dy, torch::Tensor& dw) {
  TORCH_CHECK(dout.is_contiguous() && y.is_contiguous() && dy.is_contiguous() && bf16_rows(dout) && bf16_rows(y) && bf16_rows(dy));
  TORCH_CHECK(i32(row_pair) && i32(offs) && w.scalar_type() == torch::kFloat32 && dw.scalar_type() == torch::kFloat32 && w.is_contiguous() &&
              dw.is_contiguous() && dw.numel() == w.numel() && row_pair.numel() == y.size(0) && dy.size(0) == y.size(0));
  c10::cuda::CUDAGuard guard(y.device());
  int rc = mt_moe_combine_bwd(dout.data_ptr(), y.data_ptr(), row_pair.data_ptr<int>(), offs.data_ptr<int>(), (int)offs.numel() - 1,
                              w.data_ptr<float>(), (int)k, (int)y.size(1), (int)y.size(0), dy.data_ptr(), dw.data_ptr<float>(), mt_num_sms(),
                              cur());
  TORCH_CHECK(rc == 0, "mt_moe_combine_bwd failed with code ", rc);
  mt_count_launches(1);
}

bool grouped_gemm_supported(int64_t rows_max, int64_t n_out, int64_t k_in) {
  return rows_max % 128 == 0 && n_out % 128 == 0 && k_in % 128 == 0;
}

// mode 1: c = a W^T; mode 2: c = a W; mode 3: c (+)= a^T b per expert (see gemm_sm100.cu). w / c are [E, n_out, k_in] where a weight.
void grouped_gemm(int64_t mode, const torch::Tensor& a, const torch::Tensor& b, torch::Tensor& c, const torch::Tensor& offs,
                  const torch::Tensor& blk_expert, bool accumulate) {
  TORCH_CHECK(bf16_rows(a) && i32(offs) && i32(blk_expert));
  const int64_t E = offs.numel() - 1, rows_max = a.size(0);
  int64_t n_out, k_in;
  long lda = a.stride(0), ldb = 0, ldc = 0;
  if (mode == 1 || mode == 2) {
    TORCH_CHECK(b.dim() == 3 && b.is_contiguous() && b.scalar_type() == torch::kBFloat16 && b.size(0) == E && bf16_rows(c));
    n_out = b.size(1); k_in = b.size(2);
    TORCH_CHECK(a.size(1) == (mode == 1 ? k_in : n_out) && c.size(0) == rows_max && c.size(1) == (mode == 1 ? n_out : k_in));
    ldc = c.stride(0);
  } else {
    TORCH_CHECK(mode == 3 && bf16_rows(b) && b.size(0) == rows_max && c.dim() == 3 && c.is_contiguous() && c.scalar_type() == torch::kFloat32);
    n_out = c.size(1); k_in = c.size(2);
    TORCH_CHECK(c.size(0) == E && a.size(1) == n_out && b.size(1) == k_in);
    ldb = b.stride(0);
  }
  TORCH_CHECK(grouped_gemm_supported(rows_max, n_out, k_in) && blk_expert.numel() * 128 == rows_max, "grouped_gemm: unsupported shape");
  c10::cuda::CUDAGuard guard(a.device());
  int rc = mt_gemm_bf16_grouped((int)mode, a.data_ptr(), b.data_ptr(), c.data_ptr(), (int)rows_max, (int)n_out, (int)k_in, (int)E,
                                offs.data_ptr<int>(), blk_expert.data_ptr<int>(), accumulate ? 1 : 0, lda, ldb, ldc, mt_status_ptr(),
                                mt_num_sms(), cur());
  TORCH_CHECK(rc == 0, "mt_gemm_bf16_grouped failed with code ", rc);
  mt_count_launches(1);
}

// ---- expert-parallel dispatch over peer memory. `*_table` tensors are int64 device arrays of per-rank base addresses.
void ep_put_counts(const torch::Tensor& sizes, int64_t my_rank, const torch::Tensor& counts_table) {
  TORCH_CHECK(i32(sizes) && counts_table.is_cuda() && counts_table.scalar_type() == torch::kInt64);
  c10::cuda::CUDAGuard guard(sizes.device());
  int rc = mt_ep_put_counts(sizes.data_ptr<int>(), (int)sizes.numel(), (int)my_rank, (int)counts_table.numel(),
                            reinterpret_cast<int* const*>(counts_table.data_ptr<int64_t>()), cur());
  TORCH_CHECK(rc == 0, "mt_ep_put_counts failed with code ", rc);
  mt_count_launches(1);
}

void ep_index(const torch::Tensor& counts, int64_t ep, int64_t my_rank, torch::Tensor& offs, torch::Tensor& blk_expert,
              torch::Tensor& valid_rows, torch::Tensor& send_base) {
  TORCH_CHECK(i32(counts) && i32(offs) && i32(blk_expert) && i32(valid_rows) && i32(send_base));
  const int64_t E = send_base.numel(), el = E / ep;
  TORCH_CHECK(counts.numel() == ep * E && offs.numel() == el + 1 && valid_rows.numel() == el);
  c10::cuda::CUDAGuard guard(counts.device());
  int rc = mt_ep_index(counts.data_ptr<int>(), (int)ep, (int)E, (int)my_rank, (int)blk_expert.numel() * 128, offs.data_ptr<int>(),
                       blk_expert.data_ptr<int>(), valid_rows.data_ptr<int>(), send_base.data_ptr<int>(), mt_status_ptr(), cur());
  TORCH_CHECK(rc == 0, "mt_ep_index failed with code ", rc);
  mt_count_launches(1);
}

void ep_push(const torch::Tensor& src, int64_t src_div, const torch::Tensor& idx, const torch::Tensor& dest_local, const torch::Tensor& offs_local,
             const torch::Tensor& send_base, int64_t el, int64_t cap, const torch::Tensor& buf_table, torch::Tensor& pair_owner,
             torch::Tensor& pair_row) {
  TORCH_CHECK(src.is_contiguous() && bf16_rows(src) && i32(idx) && i32(dest_local) && i32(offs_local) && i32(send_base) && i32(pair_owner) &&
              i32(pair_row) && buf_table.scalar_type() == torch::kInt64);
  const int64_t n = idx.numel();
  TORCH_CHECK(pair_owner.numel() == n && pair_row.numel() == n && src.size(0) * src_div >= n);
  c10::cuda::CUDAGuard guard(src.device());
  int rc = mt_ep_push(src.data_ptr(), (int)src_div, idx.data_ptr<int>(), dest_local.data_ptr<int>(), offs_local.data_ptr<int>(),
                      send_base.data_ptr<int>(), (int)n, (int)el, (int)cap, (int)src.size(1),
                      reinterpret_cast<void* const*>(buf_table.data_ptr<int64_t>()), pair_owner.data_ptr<int>(), pair_row.data_ptr<int>(),
                      mt_num_sms(), cur());
  TORCH_CHECK(rc == 0, "mt_ep_push failed with code ", rc);
  mt_count_launches(1);
}

void ep_pull(const torch::Tensor& buf_table, const torch::Tensor& pair_owner, const torch::Tensor& pair_row, int64_t cap, torch::Tensor& out) {
  TORCH_CHECK(out.is_contiguous() && bf16_rows(out) && i32(pair_owner) && i32(pair_row) && buf_table.scalar_type() == torch::kInt64);
  TORCH_CHECK(pair_owner.numel() == out.size(0) && pair_row.numel() == out.size(0));
  c10::cuda::CUDAGuard guard(out.device());
  int rc = mt_ep_pull(reinterpret_cast<void* const*>(buf_table.data_ptr<int64_t>()), pair_owner.data_ptr<int>(), pair_row.data_ptr<int>(),
                      (int)out.size(0), (int)cap, (int)out.size(1), out.data_ptr(), mt_num_sms(), cur());
  TORCH_CHECK(rc == 0, "mt_ep_pull failed with code ", rc);
  mt_count_launches(1);
}

void ep_zero_pads(torch::Tensor& buf, const torch::Tensor& offs, const torch::Tensor& valid_rows) {
  TORCH_CHECK(buf.is_contiguous() && bf16_rows(buf) && i32(offs) && i32(valid_rows) && offs.numel() == valid_rows.numel() + 1);
  c10::cuda::CUDAGuard guard(buf.device());
  int rc = mt_ep_zero_pads(buf.data_ptr(), offs.data_ptr<int>(), valid_rows.data_ptr<int>(), (int)valid_rows.numel(), (int)buf.size(1), cur());
  TORCH_CHECK(rc == 0, "mt_ep_zero_pads failed with code ", rc);
  mt_count_launches(1);
}

}  // namespace

void register_moe(pybind11::module_& m) {
  m.def("ep_put_counts", &ep_put_counts);
  m.def("ep_index", &ep_index);
  m.def("ep_push", &ep_push);
  m.def("ep_pull", &ep_pull);
  m.def("ep_zero_pads", &ep_zero_pads);
  m.def("router_topk", &router_topk);
  m.def("quant_fp8_rows", &quant_fp8_rows);
  m.def("quant_fp8_blocks", &quant_fp8_blocks);
  m.def("gemm_fp8_block", &gemm_fp8_block);
  m.def("moe_sort", &moe_sort);
  m.def("moe_gather", &moe_gather);
  m.def("moe_combine", &moe_combine);
  m.def("moe_combine_bwd", &moe_combine_bwd);
  m.def("grouped_gemm", &grouped_gemm);
  m.def("grouped_gemm_supported", &grouped_gemm_supported);
}
