// Bindings for the peer-memory communication kernels (flags, fused reduce-scatter, gather, all-gather GEMM).
// Pointer tables are int64 CUDA tensors holding one device pointer per rank (built from symmetric-memory handles).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>

extern "C" {
int mt_comm_signal(int* const* peer_flags, int slot, int my_rank, int world, int epoch, cudaStream_t st);
int mt_comm_wait(const int* my_flags, int slot, int world, int epoch, int* status, unsigned long long limit_ns, cudaStream_t st);
int mt_rs_num_partials(long n, int ctas);
int mt_rs_sumsq(const float* const* peer, long offset, long n, float* dst, int accumulate, float scale, int world, float* partials,
                float* sumsq_out, int ctas, cudaStream_t st);
int mt_rs_sumsq_mc(const float* mc, long offset, long n, float* dst, int accumulate, float scale, float* partials, float* sumsq_out, int ctas,
                   cudaStream_t st);
int mt_gather_dma(const long long* peer_ptrs, void* full, long chunk_bytes, int world, int first, cudaStream_t st);
int mt_gather_segments(const void* const* peer_shards, void* full, long chunk_bytes, long seg_bytes, int world, int* seg_flags, int ctas,
                       cudaStream_t st);
int mt_gemm_bf16_ag(const void* a, void* c, int M, int N, int K, int64_t lda, int64_t ldc, const void* const* peer_shards, void* full,
                    long chunk_elems, long seg_elems, long b_offset, int world, int* seg_flags, int comm_ctas, int* status, int num_sms,
                    cudaStream_t stream);
int mt_gemm_rs_encode_maps(void* out_maps, const void* const* bufs, int world, int rows, int N, int bf16);
int mt_reduce_staged(const void* staged, long chunk_elems, int world, void* out, int ctas, cudaStream_t st);
int mt_tensor_map_bytes();
int mt_gemm_bf16_rs(const void* a, const void* b, int M, int N, int K, int64_t lda, int64_t ldb, int b_mn, const void* dev_maps, int world,
                    int out_bf16, int* status, int num_sms, cudaStream_t stream);
int mt_gather_cvt(const float* const* peer_acc, long chunk_elems, int world, void* out, int ctas, cudaStream_t st);
}

int* mt_status_ptr();
void mt_count_launches(int n);

namespace {

cudaStream_t cur() { return at::cuda::getCurrentCUDAStream().stream(); }

int sm_count() {
  int dev = 0, n = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

void ptr_table_ok(const torch::Tensor& t, int64_t world) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == torch::kInt64 && t.is_contiguous() && t.numel() >= world, "bad pointer table");
}

void comm_signal(const torch::Tensor& peer_flags, int64_t slot, int64_t my_rank, int64_t world, int64_t epoch) {
  ptr_table_ok(peer_flags, world);
  c10::cuda::CUDAGuard g(peer_flags.device());
  TORCH_CHECK(mt_comm_signal(reinterpret_cast<int* const*>(peer_flags.data_ptr<int64_t>()), (int)slot, (int)my_rank, (int)world, (int)epoch,
                             cur()) == 0, "mt_comm_signal failed");
  mt_count_launches(1);
}

void comm_wait(const torch::Tensor& my_flags, int64_t slot, int64_t world, int64_t epoch, double limit_ms) {
  TORCH_CHECK(my_flags.is_cuda() && my_flags.scalar_type() == torch::kInt32);
  c10::cuda::CUDAGuard g(my_flags.device());
  TORCH_CHECK(mt_comm_wait(my_flags.data_ptr<int>(), (int)slot, (int)world, (int)epoch, mt_status_ptr(),
                           (unsigned long long)(limit_ms * 1e6), cur()) == 0, "mt_comm_wait failed");
  mt_count_launches(1);
}

void rs_sumsq(const torch::Tensor& peer_bufs, int64_t offset, int64_t n, torch::Tensor& dst, bool accumulate, double scale, int64_t world,
              const c10::optional<torch::Tensor>& sumsq_out, int64_t ctas) {
  ptr_table_ok(peer_bufs, world);
  TORCH_CHECK(dst.is_cuda() && dst.scalar_type() == torch::kFloat32 && dst.is_contiguous() && dst.numel() >= n);
  c10::cuda::CUDAGuard g(dst.device());
  const int parts = mt_rs_num_partials(n, (int)ctas);
  auto partials = torch::empty({parts}, dst.options());
  TORCH_CHECK(mt_rs_sumsq(reinterpret_cast<const float* const*>(peer_bufs.data_ptr<int64_t>()), offset, n, dst.data_ptr<float>(),
                          accumulate ? 1 : 0, (float)scale, (int)world, partials.data_ptr<float>(),
                          sumsq_out ? sumsq_out->data_ptr<float>() : nullptr, (int)ctas, cur()) == 0, "mt_rs_sumsq failed");
  mt_count_launches(sumsq_out ? 2 : 1);
}

// reduce-scatter through the switch: mc_ptr is the multicast address of the symmetric gradient buffer
void rs_sumsq_mc(int64_t mc_ptr, int64_t offset, int64_t n, torch::Tensor& dst, bool accumulate, double scale,
                 const c10::optional<torch::Tensor>& sumsq_out, int64_t ctas) {
  TORCH_CHECK(mc_ptr != 0 && dst.is_cuda() && dst.scalar_type() == torch::kFloat32 && dst.is_contiguous() && dst.numel() >= n);
  c10::cuda::CUDAGuard g(dst.device());
  const int parts = mt_rs_num_partials(n, (int)ctas);
  auto partials = torch::empty({parts}, dst.options());
  TORCH_CHECK(mt_rs_sumsq_mc(reinterpret_cast<const float*>(mc_ptr), offset, n, dst.data_ptr<float>(), accumulate ? 1 : 0, (float)scale,
                             partials.data_ptr<float>(), sumsq_out ? sumsq_out->data_ptr<float>() : nullptr, (int)ctas, cur()) == 0,
              "mt_rs_sumsq_mc failed");
  mt_count_launches(sumsq_out ? 2 : 1);
}

void gather_dma(const std::vector<int64_t>& peer_ptrs, torch::Tensor& full, int64_t chunk_bytes, int64_t first) {
  std::vector<long long> p(peer_ptrs.begin(), peer_ptrs.end());
  TORCH_CHECK((int64_t)p.size() * chunk_bytes <= (int64_t)full.numel() * full.element_size(), "gather_dma: destination too small");
  TORCH_CHECK(mt_gather_dma(p.data(), full.data_ptr(), chunk_bytes, (int)p.size(), (int)first, cur()) == 0, "mt_gather_dma failed");
}

void gather_segments(const torch::Tensor& peer_shards, torch::Tensor& full, int64_t chunk_bytes, int64_t seg_bytes, int64_t world,
                     int64_t ctas) {
  ptr_table_ok(peer_shards, world);
  TORCH_CHECK(full.is_cuda() && full.is_contiguous() && full.numel() * full.element_size() >= chunk_bytes * world);
  c10::cuda::CUDAGuard g(full.device());
  TORCH_CHECK(mt_gather_segments(reinterpret_cast<const void* const*>(peer_shards.data_ptr<int64_t>()), full.data_ptr(), chunk_bytes,
                                 seg_bytes, (int)world, nullptr, (int)ctas, cur()) == 0, "mt_gather_segments failed");
  mt_count_launches(1);
}

// out[M,N] = a[M,K] . W^T with W = full[b_offset : b_offset + N*K] viewed [N,K]; gathers the whole unit on the way.
void gemm_ag(const torch::Tensor& a, torch::Tensor& out, const torch::Tensor& peer_shards, torch::Tensor& full, int64_t N, int64_t K,
             int64_t chunk_elems, int64_t seg_elems, int64_t b_offset, int64_t world, torch::Tensor& seg_flags, int64_t comm_ctas) {
  ptr_table_ok(peer_shards, world);
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == torch::kBFloat16 && a.dim() == 2 && a.stride(1) == 1 && a.size(1) == K);
  TORCH_CHECK(out.scalar_type() == torch::kBFloat16 && out.dim() == 2 && out.stride(1) == 1 && out.size(0) == a.size(0) && out.size(1) == N);
  TORCH_CHECK(full.scalar_type() == torch::kBFloat16 && full.is_contiguous() && full.numel() >= chunk_elems * world);
  TORCH_CHECK(seg_flags.scalar_type() == torch::kInt32 && seg_flags.numel() >= world * ((chunk_elems + seg_elems - 1) / seg_elems));
  TORCH_CHECK(a.size(0) >= 128 && N >= 256 && K >= 64 && K % 8 == 0 && b_offset + N * K <= chunk_elems * world);
  c10::cuda::CUDAGuard g(a.device());
  int rc = mt_gemm_bf16_ag(a.data_ptr(), out.data_ptr(), (int)a.size(0), (int)N, (int)K, a.stride(0), out.stride(0),
                           reinterpret_cast<const void* const*>(peer_shards.data_ptr<int64_t>()), full.data_ptr(), chunk_elems, seg_elems,
                           b_offset, (int)world, seg_flags.data_ptr<int>(), (int)comm_ctas, mt_status_ptr(), sm_count(), cur());
  TORCH_CHECK(rc == 0, "mt_gemm_bf16_ag failed with code ", rc);
  mt_count_launches(1);
}

}  // namespace

// Device tensor holding one tensor map per rank over that rank's fp32 accumulation buffer [rows, N] (addresses from `ptrs`).
torch::Tensor gemm_rs_maps(const std::vector<int64_t>& ptrs, int64_t rows, int64_t N, const torch::Device& device, bool bf16) {
  const int world = (int)ptrs.size();
  const int mb = mt_tensor_map_bytes();
  std::vector<const void*> bufs(world);
  for (int r = 0; r < world; ++r) bufs[r] = reinterpret_cast<const void*>(ptrs[r]);
  auto host = torch::empty({world * mb}, torch::dtype(torch::kUInt8).pinned_memory(false));
  TORCH_CHECK(reinterpret_cast<uintptr_t>(host.data_ptr()) % 64 == 0, "tensor map staging buffer is not 64-byte aligned");
  int rc = mt_gemm_rs_encode_maps(host.data_ptr(), bufs.data(), world, (int)rows, (int)N, bf16 ? 1 : 0);
  TORCH_CHECK(rc == 0, "mt_gemm_rs_encode_maps failed with code ", rc);
  auto dev = host.to(device);
  TORCH_CHECK(reinterpret_cast<uintptr_t>(dev.data_ptr()) % 64 == 0);
  return dev;
}

// Partial product a . op(w) reduce-scattered over the group: every rank's fp32 buffer (zeroed beforehand) receives the sum
// of the rows it owns. tb: w stored [N, K] (y = a w^T); else [K, N].
void gemm_rs(const torch::Tensor& a, const torch::Tensor& w, bool tb, const torch::Tensor& dev_maps, int64_t world, bool out_bf16) {
  TORCH_CHECK(a.is_cuda() && a.dim() == 2 && w.dim() == 2 && a.scalar_type() == torch::kBFloat16 && w.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(a.stride(1) == 1 && w.stride(1) == 1 && a.stride(0) % 8 == 0 && w.stride(0) % 8 == 0);
  const int64_t M = a.size(0), K = a.size(1), N = tb ? w.size(0) : w.size(1);
  TORCH_CHECK((tb ? w.size(1) : w.size(0)) == K && K % 64 == 0 && N % 128 == 0, "gemm_rs: unsupported shape");
  c10::cuda::CUDAGuard guard(a.device());
  int rc = mt_gemm_bf16_rs(a.data_ptr(), w.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), w.stride(0), tb ? 0 : 1, dev_maps.data_ptr(),
                           (int)world, out_bf16 ? 1 : 0, mt_status_ptr(), sm_count(), cur());
  TORCH_CHECK(rc == 0, "mt_gemm_bf16_rs failed with code ", rc);
  mt_count_launches(1);
}

void gather_cvt(const torch::Tensor& acc_table, int64_t chunk_elems, int64_t world, torch::Tensor& out) {
  ptr_table_ok(acc_table, world);
  TORCH_CHECK(out.is_contiguous() && out.scalar_type() == torch::kBFloat16 && out.numel() == chunk_elems * world);
  c10::cuda::CUDAGuard guard(out.device());
  int rc = mt_gather_cvt(reinterpret_cast<const float* const*>(acc_table.data_ptr<int64_t>()), chunk_elems, (int)world, out.data_ptr(),
                         sm_count() * 4, cur());
  TORCH_CHECK(rc == 0, "mt_gather_cvt failed with code ", rc);
  mt_count_launches(1);
}

// out [chunk] bf16 = sum over the `world` staged copies (consecutive chunks of `staged`), fixed order
void reduce_staged(const torch::Tensor& staged, int64_t world, torch::Tensor& out) {
  TORCH_CHECK(staged.is_cuda() && staged.is_contiguous() && out.is_contiguous() && staged.scalar_type() == torch::kBFloat16 &&
              out.scalar_type() == torch::kBFloat16 && staged.numel() == out.numel() * world);
  c10::cuda::CUDAGuard guard(out.device());
  int rc = mt_reduce_staged(staged.data_ptr(), out.numel(), (int)world, out.data_ptr(), sm_count() * 4, cur());
  TORCH_CHECK(rc == 0, "mt_reduce_staged failed with code ", rc);
  mt_count_launches(1);
}

void register_comm(pybind11::module_& m) {
  m.def("reduce_staged", &reduce_staged);
  m.def("rs_sumsq_mc", &rs_sumsq_mc);
  m.def("gemm_rs_maps", &gemm_rs_maps);
  m.def("gemm_rs", &gemm_rs);
  m.def("gather_cvt", &gather_cvt);
  m.def("comm_signal", &comm_signal);
  m.def("comm_wait", &comm_wait);
  m.def("rs_sumsq", &rs_sumsq);
  m.def("gather_segments", &gather_segments);
  m.def("gather_dma", &gather_dma);
  m.def("gemm_ag", &gemm_ag);
}
