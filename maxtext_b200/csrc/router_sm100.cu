// MoE router: softmax / sigmoid scores, top-k selection, routing weights and the per-expert histogram in one launch.
//
// One warp per token; lane l holds experts l, l+32, ... (up to 16 per lane, so E <= 512). The k winners are found by k rounds
// of a warp-wide arg-max over the not yet selected scores (ties go to the lower expert index), which for k <= 8 is cheaper
// than any sort. Two forms:
//   mode 0  selection on the logits (plus an optional per-expert bias); weights = softmax over the k selected logits, or
//           the raw logits (`raw_weights`, Llama-4 style); probs = softmax over all experts (for the load-balance loss)
//   mode 1  DeepSeek style: scores = softmax or sigmoid of the logits, selection on scores + bias, weights = the selected
//           scores (renormalised over the k for sigmoid scores) times a scaling factor; probs = scores
// The gradient of these few small tensors is taken in PyTorch from the saved outputs.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mt {

constexpr int ROUTER_MAX_PER_LANE = 16;

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T>
__global__ void router_topk_kernel(const T* __restrict__ logits, const float* __restrict__ bias, long tokens, int E, int k, int mode,
                                   int sigmoid_scores, int raw_weights, float scaling, int* __restrict__ idx_out, float* __restrict__ wts_out,
                                   float* __restrict__ probs_out, int* __restrict__ counts) {
  const long tok = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (tok >= tokens) return;
  const int per = (E + 31) / 32;
  float x[ROUTER_MAX_PER_LANE], sc[ROUTER_MAX_PER_LANE], sel[ROUTER_MAX_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
    const int e = lane + 32 * j;
    x[j] = (j < per && e < E) ? to_f<T>(logits[tok * E + e]) + ((mode == 0 && bias) ? bias[e] : 0.f) : -INFINITY;      // mode 0: the bias is part of the logits
    mx = fmaxf(mx, x[j]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
    const int e = lane + 32 * j;
    const bool live = j < per && e < E;
    float s;
    if (mode == 1 && sigmoid_scores) s = live ? 1.f / (1.f + expf(-x[j])) : 0.f;
    else s = live ? expf(x[j] - mx) : 0.f;
    sc[j] = s;
    sum += s;
  }
  if (!(mode == 1 && sigmoid_scores)) {
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) sc[j] *= inv;
  }
#pragma unroll
  for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
    const int e = lane + 32 * j;
    const bool live = j < per && e < E;
    if (live && probs_out) probs_out[tok * E + e] = sc[j];
    const float b = (mode == 1 && bias && live) ? bias[e] : 0.f;              // mode 1: the bias only steers the selection
    sel[j] = !live ? -INFINITY : (mode == 1 ? sc[j] + b : x[j]);
  }
  // k rounds of arg-max; the winner's lane keeps its value for the weight computation
  float wsel = 0.f;      // lane r (r < k) ends up holding the r-th winner: its selection value, score and expert
  float wscore = 0.f;
  int wexp = 0;
  for (int r = 0; r < k; ++r) {
    float best = -INFINITY;
    int bj = 0;
#pragma unroll
    for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j)
      if (sel[j] > best) { best = sel[j]; bj = j; }
    int be = lane + 32 * bj;
    float v = best;
    int e = be;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oe = __shfl_xor_sync(0xffffffffu, e, o);
      if (ov > v || (ov == v && oe < e)) { v = ov; e = oe; }
    }
    // the owner of expert e retires it and publishes its score
    float s_owner = 0.f;
    if ((e & 31) == lane) {
      const int j = e >> 5;
#pragma unroll
      for (int jj = 0; jj < ROUTER_MAX_PER_LANE; ++jj)
        if (jj == j) { s_owner = (mode == 1) ? sc[jj] : x[jj]; sel[jj] = -INFINITY; }
    }
    s_owner = __shfl_sync(0xffffffffu, s_owner, e & 31);
    if (lane == r) { wsel = v; wscore = s_owner; wexp = e; }
  }
  // weights over the k winners (lanes 0..k-1)
  float w;
  if (mode == 1) {
    w = lane < k ? wscore : 0.f;
    if (sigmoid_scores) { const float tot = warp_sum(w); w = w / (tot + 1e-20f); }
    w *= scaling;
  } else if (raw_weights) {
    w = lane < k ? wscore : 0.f;
  } else {
    const float v = lane < k ? wscore : -INFINITY;
    const float m2 = warp_max(v);
    const float ex = lane < k ? expf(v - m2) : 0.f;
    w = ex / warp_sum(ex);
  }
  (void)wsel;
  if (lane < k) {
    idx_out[tok * k + lane] = wexp;
    wts_out[tok * k + lane] = w;
    if (counts) atomicAdd(counts + wexp, 1);
  }
}

}  // namespace mt

// logits [tokens, E] fp32 (is_bf16 = 0) or bf16; bias [E] fp32 or null; outputs idx [tokens,k] int32, wts [tokens,k] fp32,
// probs [tokens,E] fp32 (may be null), counts [E] int32 (may be null; must be zeroed by the caller).
extern "C" int mt_router_topk(const void* logits, int is_bf16, const float* bias, long tokens, int E, int k, int mode, int sigmoid_scores,
                              int raw_weights, float scaling, int* idx, float* wts, float* probs, int* counts, cudaStream_t st) {
  if (E < 1 || E > 32 * mt::ROUTER_MAX_PER_LANE || k < 1 || k > 32 || k > E) return -1;
  const int threads = 256;
  const long blocks = (tokens * 32 + threads - 1) / threads;
  if (blocks == 0) return 0;
  if (is_bf16)
    mt::router_topk_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, st>>>((const __nv_bfloat16*)logits, bias, tokens, E, k, mode,
                                                                                sigmoid_scores, raw_weights, scaling, idx, wts, probs, counts);
  else
    mt::router_topk_kernel<float><<<(unsigned)blocks, threads, 0, st>>>((const float*)logits, bias, tokens, E, k, mode, sigmoid_scores,
                                                                        raw_weights, scaling, idx, wts, probs, counts);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
