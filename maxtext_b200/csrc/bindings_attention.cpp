// Bindings for the attention kernels (flash attention forward / backward).
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime.h>

extern "C" {
int mt_flash_fwd_supported(int Dqk, int Dv);
long mt_attn_tile_ints(int B, int Sq, int Skv);
int mt_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* seg_q, const int* seg_k, const int* pos_q,
                 const int* pos_k, int* tiles, const float* sinks, int B, int Sq, int Skv, int Hq, int Hkv, int Dqk, int Dv, long ldq, long bsq,
                 long ldk, long bsk, long ldv, long bsv, long ldo, long bso, float scale, float softcap, int causal, int window, int chunk,
                 int q_off, int* status, cudaStream_t st);
int mt_flash_bwd_supported(int Dqk, int Dv);
int mt_flash_bwd(const void* dout, const void* q, const void* k, const void* v, const void* out, const float* lse, float* delta, void* dq,
                 void* dk, void* dv, const int* seg_q, const int* seg_k, const int* pos_q, const int* pos_k, int* tiles, int B, int Sq, int Skv,
                 int Hq, int Hkv, int D, int Dv, long ldq, long bsq, long ldk, long bsk, long ldv, long bsv, long lddq, long bsdq, long lddk, long bsdk,
                 long lddv, long bsdv, float scale, float softcap, int causal, int window, int chunk, int q_off, int* status, cudaStream_t st);
}

extern "C" int mt_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int* slot_ids, const int* lengths, int B,
                                   int max_len, int Hq, int Hkv, int D, int window, float scale, float soft_cap, int splits, float* part,
                                   void* out, cudaStream_t st);


extern "C" int mt_sample(const void* logits, int is_bf16, const float* uniform, long rows, long V, int topk, float nucleus_p, float temperature,
                         int greedy, long long* out, cudaStream_t st);

int* mt_status_ptr();          // defined in bindings.cpp
void mt_count_launches(int n); // defined in bindings.cpp

namespace {

// [B,S,H,D] view usable as a {H*D, S, B} TMA tensor: unit inner stride, heads adjacent, 16-byte aligned row / batch strides
bool tma_view(const torch::Tensor& t) {
  return t.dim() == 4 && t.stride(3) == 1 && t.stride(2) == t.size(3) && t.stride(1) % 8 == 0 && t.stride(0) % 8 == 0 &&
         (reinterpret_cast<uintptr_t>(t.data_ptr()) % 16) == 0 && t.scalar_type() == torch::kBFloat16;
}

// forward-only shape check: q [B,Sq,Hq,Dqk], k [B,Skv,Hkv,Dqk], v [B,Skv,Hkv,Dv]; any Sq / Skv
bool flash_fwd_supported(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v) {
  if (!q.is_cuda() || !tma_view(q) || !tma_view(k) || !tma_view(v)) return false;
  if (!mt_flash_fwd_supported((int)q.size(3), (int)v.size(3)) || k.size(3) != q.size(3)) return false;
  if (k.size(0) != q.size(0) || v.size(0) != q.size(0) || k.size(1) != v.size(1)) return false;
  return k.size(2) == v.size(2) && q.size(2) % k.size(2) == 0;
}

const int* opt_int(const c10::optional<torch::Tensor>& t, int64_t numel, const char* what) {
  if (!t) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->is_contiguous() && t->scalar_type() == torch::kInt32 && t->numel() == numel, what, ": int32 contiguous tensor of ",
              numel, " elements expected");
  return t->data_ptr<int>();
}

void flash_fwd(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v, torch::Tensor& out, torch::Tensor& lse,
               const c10::optional<torch::Tensor>& seg_q, const c10::optional<torch::Tensor>& seg_k, const c10::optional<torch::Tensor>& pos_q,
               const c10::optional<torch::Tensor>& pos_k, const c10::optional<torch::Tensor>& sinks, double scale, double softcap, bool causal,
               int64_t window, int64_t chunk, int64_t q_off) {
  TORCH_CHECK(flash_fwd_supported(q, k, v) && tma_view(out) && lse.is_contiguous() && lse.scalar_type() == torch::kFloat32);
  const int B = (int)q.size(0), Sq = (int)q.size(1), Skv = (int)k.size(1), Hq = (int)q.size(2);
  TORCH_CHECK(out.size(0) == B && out.size(1) == Sq && out.size(2) == Hq && out.size(3) == v.size(3) && lse.numel() == (int64_t)B * Hq * Sq);
  TORCH_CHECK(bool(seg_q) == bool(seg_k) && bool(pos_q) == bool(pos_k), "segment ids / positions must be given for queries and keys together");
  if (sinks) TORCH_CHECK(sinks->is_cuda() && sinks->is_contiguous() && sinks->scalar_type() == torch::kFloat32 && sinks->numel() == Hq);
  c10::cuda::CUDAGuard guard(q.device());
  torch::Tensor tiles;
  if (pos_q) tiles = torch::empty({mt_attn_tile_ints(B, Sq, Skv)}, torch::dtype(torch::kInt32).device(q.device()));
  int rc = mt_flash_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr<float>(), opt_int(seg_q, (int64_t)B * Sq, "seg_q"),
                        opt_int(seg_k, (int64_t)B * Skv, "seg_k"), opt_int(pos_q, (int64_t)B * Sq, "pos_q"), opt_int(pos_k, (int64_t)B * Skv, "pos_k"),
                        pos_q ? tiles.data_ptr<int>() : nullptr, sinks ? sinks->data_ptr<float>() : nullptr, B, Sq, Skv, Hq, (int)k.size(2),
                        (int)q.size(3), (int)v.size(3), q.stride(1), q.stride(0), k.stride(1), k.stride(0), v.stride(1), v.stride(0),
                        out.stride(1), out.stride(0), (float)scale, (float)softcap, causal ? 1 : 0, (int)window, (int)chunk, (int)q_off,
                        mt_status_ptr(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "mt_flash_fwd failed with code ", rc);
  mt_count_launches(pos_q ? 3 : 1);
}

bool flash_bwd_supported(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v) {
  return flash_fwd_supported(q, k, v) && mt_flash_bwd_supported((int)q.size(3), (int)v.size(3));
}

void flash_bwd(const torch::Tensor& dout, const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v, const torch::Tensor& out,
               const torch::Tensor& lse, torch::Tensor& dq, torch::Tensor& dk, torch::Tensor& dv, const c10::optional<torch::Tensor>& seg_q,
               const c10::optional<torch::Tensor>& seg_k, const c10::optional<torch::Tensor>& pos_q, const c10::optional<torch::Tensor>& pos_k,
               double scale, double softcap, bool causal, int64_t window, int64_t chunk, int64_t q_off) {
  TORCH_CHECK(flash_bwd_supported(q, k, v) && tma_view(dq) && tma_view(dk) && tma_view(dv));
  TORCH_CHECK(dq.sizes() == q.sizes() && dk.sizes() == k.sizes() && dv.sizes() == v.sizes());
  TORCH_CHECK(dout.is_contiguous() && out.is_contiguous() && lse.is_contiguous() && dout.sizes() == out.sizes() &&
              dout.scalar_type() == torch::kBFloat16 && out.scalar_type() == torch::kBFloat16 && lse.scalar_type() == torch::kFloat32);
  TORCH_CHECK(bool(seg_q) == bool(seg_k) && bool(pos_q) == bool(pos_k), "segment ids / positions must be given for queries and keys together");
  const int B = (int)q.size(0), Sq = (int)q.size(1), Skv = (int)k.size(1), Hq = (int)q.size(2);
  TORCH_CHECK(lse.numel() == (int64_t)B * Hq * Sq && out.size(0) == B && out.size(1) == Sq && out.size(2) == Hq && out.size(3) == v.size(3));
  c10::cuda::CUDAGuard guard(q.device());
  auto delta = torch::empty({B, Hq, Sq}, lse.options());
  torch::Tensor tiles;
  if (pos_q) tiles = torch::empty({mt_attn_tile_ints(B, Sq, Skv)}, torch::dtype(torch::kInt32).device(q.device()));
  int rc = mt_flash_bwd(dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr<float>(), delta.data_ptr<float>(),
                        dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), opt_int(seg_q, (int64_t)B * Sq, "seg_q"), opt_int(seg_k, (int64_t)B * Skv, "seg_k"),
                        opt_int(pos_q, (int64_t)B * Sq, "pos_q"), opt_int(pos_k, (int64_t)B * Skv, "pos_k"), pos_q ? tiles.data_ptr<int>() : nullptr,
                        B, Sq, Skv, Hq, (int)k.size(2), (int)q.size(3), (int)v.size(3), q.stride(1), q.stride(0), k.stride(1), k.stride(0), v.stride(1), v.stride(0),
                        dq.stride(1), dq.stride(0), dk.stride(1), dk.stride(0), dv.stride(1), dv.stride(0), (float)scale, (float)softcap,
                        causal ? 1 : 0, (int)window, (int)chunk, (int)q_off, mt_status_ptr(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "mt_flash_bwd failed with code ", rc);
  mt_count_launches(pos_q ? 5 : 3);
}

// q [B, Hq, D], caches [slots, max_len, Hkv, D] (bf16), slot_ids / lengths int32 [B] (lengths include the new token); out [B, Hq, D].
void decode_attention(const torch::Tensor& q, const torch::Tensor& k_cache, const torch::Tensor& v_cache, const torch::Tensor& slot_ids,
                      const torch::Tensor& lengths, torch::Tensor& out, double scale, double soft_cap, int64_t window, int64_t splits) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 3 && q.is_contiguous() && out.is_contiguous() && q.scalar_type() == torch::kBFloat16);
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous() && k_cache.scalar_type() == torch::kBFloat16 &&
              v_cache.sizes() == k_cache.sizes() && k_cache.size(3) == q.size(2));
  TORCH_CHECK(slot_ids.scalar_type() == torch::kInt32 && lengths.scalar_type() == torch::kInt32 && slot_ids.numel() == q.size(0) &&
              lengths.numel() == q.size(0) && slot_ids.is_contiguous() && lengths.is_contiguous());
  const int B = (int)q.size(0), Hq = (int)q.size(1), D = (int)q.size(2), Hkv = (int)k_cache.size(2);
  c10::cuda::CUDAGuard guard(q.device());
  auto part = torch::empty({(int64_t)B * Hkv * splits * (Hq / Hkv) * (D + 2)}, torch::dtype(torch::kFloat32).device(q.device()));
  int rc = mt_decode_attention(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), slot_ids.data_ptr<int>(), lengths.data_ptr<int>(), B,
                               (int)k_cache.size(1), Hq, Hkv, D, (int)window, (float)scale, (float)soft_cap, (int)splits, part.data_ptr<float>(),
                               out.data_ptr(), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "mt_decode_attention failed with code ", rc);
  mt_count_launches(2);
}

// logits [rows, V] fp32 / bf16 -> token ids [rows] int64; `uniform` [rows] fp32 in [0,1) drives the draw (unused when greedy)
torch::Tensor sample_tokens(const torch::Tensor& logits, const c10::optional<torch::Tensor>& uniform, int64_t topk, double nucleus_p,
                            double temperature, bool greedy) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous() &&
              (logits.scalar_type() == torch::kFloat32 || logits.scalar_type() == torch::kBFloat16));
  if (!greedy) TORCH_CHECK(uniform && uniform->is_cuda() && uniform->is_contiguous() && uniform->scalar_type() == torch::kFloat32 &&
                           uniform->numel() == logits.size(0), "one uniform number per row is needed");
  c10::cuda::CUDAGuard guard(logits.device());
  auto out = torch::empty({logits.size(0)}, torch::dtype(torch::kInt64).device(logits.device()));
  int rc = mt_sample(logits.data_ptr(), logits.scalar_type() == torch::kBFloat16 ? 1 : 0, greedy ? nullptr : uniform->data_ptr<float>(),
                     logits.size(0), logits.size(1), (int)topk, (float)nucleus_p, (float)temperature, greedy ? 1 : 0,
                     reinterpret_cast<long long*>(out.data_ptr<int64_t>()), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "mt_sample failed with code ", rc);
  mt_count_launches(1);
  return out;
}

}  // namespace

void register_attention(pybind11::module_& m) {
  m.def("sample_tokens", &sample_tokens);
  m.def("decode_attention", &decode_attention);
  m.def("flash_fwd_supported", &flash_fwd_supported);
  m.def("flash_bwd_supported", &flash_bwd_supported);
  m.def("flash_fwd", &flash_fwd);
  m.def("flash_bwd", &flash_bwd);
}
