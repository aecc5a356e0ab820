// Token sampling for decode: greedy, temperature, top-k, nucleus (top-p) and their composition, one CTA per row of logits.
//
// Nothing is sorted. The k-th largest logit is found by a radix select over the order-preserving integer image of the floats
// (four passes of 8-bit histograms in shared memory); the nucleus cut is found by the same walk over histograms of probability
// MASS instead of counts; the token is drawn by inverting the cumulative distribution of the kept entries against one uniform
// number per row supplied by the caller. All masses are fixed-point integers (2^-40 of the largest probability), so every sum
// is exact and order independent: the same logits and the same uniform number give the same token on every run.
// Order of operations as in the reference: top-k mask, then nucleus mask on the softmax (temperature 1) of what is left, then a
// draw from softmax(kept logits / temperature).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mt {

constexpr int SAMPLE_THREADS = 512;
constexpr float SAMPLE_FIX = 1099511627776.f;      // 2^40

template <typename T>
__device__ __forceinline__ float ld_logit(const T* p, long i);
template <>
__device__ __forceinline__ float ld_logit<float>(const float* p, long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, long i) { return __bfloat162float(p[i]); }

// larger float <-> larger unsigned key
__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  unsigned long long t = 0;
  for (int i = 0; i < SAMPLE_THREADS / 32; ++i) t += sh[i];
  return t;
}

template <typename T>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const T* __restrict__ logits, const float* __restrict__ uniform, long V, int topk, float nucleus_p, float inv_temp, int greedy,
              long long* __restrict__ out) {
  __shared__ unsigned long long hist[256];
  __shared__ unsigned long long red[SAMPLE_THREADS / 32];
  __shared__ unsigned long long scan[SAMPLE_THREADS];
  __shared__ float s_max;
  __shared__ uint32_t s_prefix;
  __shared__ unsigned long long s_remaining;
  __shared__ long long s_pick;
  const T* row = logits + (long)blockIdx.x * V;
  const int tid = threadIdx.x;

  // ---- row maximum (and its first index, which is the greedy answer)
  float mx = -INFINITY;
  long arg = 0;
  for (long i = tid; i < V; i += SAMPLE_THREADS) {
    const float x = ld_logit<T>(row, i);
    if (x > mx) { mx = x; arg = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ox = __shfl_xor_sync(0xffffffffu, mx, o);
    const long oa = __shfl_xor_sync(0xffffffffu, arg, o);
    if (ox > mx || (ox == mx && oa < arg)) { mx = ox; arg = oa; }
  }
  __shared__ float w_max[SAMPLE_THREADS / 32];
  __shared__ long w_arg[SAMPLE_THREADS / 32];
  if ((tid & 31) == 0) { w_max[tid >> 5] = mx; w_arg[tid >> 5] = arg; }
  __syncthreads();
  if (tid == 0) {
    for (int i = 1; i < SAMPLE_THREADS / 32; ++i)
      if (w_max[i] > mx || (w_max[i] == mx && w_arg[i] < arg)) { mx = w_max[i]; arg = w_arg[i]; }
    s_max = mx;
    s_pick = arg;
  }
  __syncthreads();
  if (greedy) {
    if (tid == 0) out[blockIdx.x] = s_pick;
    return;
  }
  const float M = s_max;

  // ---- top-k: key of the k-th largest logit (everything >= it is kept)
  uint32_t lo_key = 0;                       // keep keys >= lo_key
  if (topk > 0 && topk < V) {
    if (tid == 0) { s_prefix = 0; s_remaining = (unsigned long long)topk; }
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t mask = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
      for (long i = tid; i < V; i += SAMPLE_THREADS) {
        const uint32_t k = order_key(ld_logit<T>(row, i));
        if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255], 1ull);
      }
      __syncthreads();
      if (tid == 0) {
        unsigned long long need = s_remaining, acc = 0;
        int b = 255;
        for (; b > 0; --b) {
          if (acc + hist[b] >= need) break;
          acc += hist[b];
        }
        s_remaining = need - acc;
        s_prefix = prefix | ((uint32_t)b << shift);
      }
      __syncthreads();
    }
    lo_key = s_prefix;
  }

  // ---- nucleus: smallest set of the largest kept entries whose probability mass reaches p
  if (nucleus_p > 0.f && nucleus_p < 1.f) {
    unsigned long long z = 0;
    for (long i = tid; i < V; i += SAMPLE_THREADS) {
      const float x = ld_logit<T>(row, i);
      if (order_key(x) >= lo_key) z += (unsigned long long)(__expf(x - M) * SAMPLE_FIX);
    }
    z = block_sum_u64(z, red);
    if (tid == 0) { s_prefix = 0; s_remaining = (unsigned long long)((double)nucleus_p * (double)z); }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t mask = shift == 24 ? 0u : (0xFFFFFFFFu << (shift + 8));
      for (long i = tid; i < V; i += SAMPLE_THREADS) {
        const float x = ld_logit<T>(row, i);
        const uint32_t k = order_key(x);
        if (k >= lo_key && (k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255], (unsigned long long)(__expf(x - M) * SAMPLE_FIX));
      }
      __syncthreads();
      if (tid == 0) {
        // walk from the largest bucket: an entry is kept while the mass before it is below the target
        unsigned long long need = s_remaining, acc = 0;
        int b = 255;
        for (; b > 0; --b) {
          if (acc + hist[b] >= need) break;
          acc += hist[b];
        }
        s_remaining = need - acc;
        s_prefix = prefix | ((uint32_t)b << shift);
      }
      __syncthreads();
    }
    if (s_prefix > lo_key) lo_key = s_prefix;
  }

  // ---- draw: invert the cumulative distribution of softmax(kept / temperature), entries in index order
  const long per = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const long i0 = (long)tid * per, i1 = i0 + per < V ? i0 + per : V;
  unsigned long long mine = 0;
  for (long i = i0; i < i1; ++i) {
    const float x = ld_logit<T>(row, i);
    if (order_key(x) >= lo_key) mine += (unsigned long long)(__expf((x - M) * inv_temp) * SAMPLE_FIX);
  }
  scan[tid] = mine;
  __syncthreads();
  if (tid == 0) {
    unsigned long long tot = 0;
    for (int i = 0; i < SAMPLE_THREADS; ++i) { const unsigned long long v = scan[i]; scan[i] = tot; tot += v; }
    double u = (double)uniform[blockIdx.x];
    u = u < 0.0 ? 0.0 : (u >= 1.0 ? 0.99999994 : u);
    s_remaining = (unsigned long long)(u * (double)tot);         // target in [0, tot)
    s_pick = -1;
  }
  __syncthreads();
  const unsigned long long target = s_remaining, before = scan[tid];
  if (mine > 0 && target >= before && target < before + mine) {
    unsigned long long acc = before;
    long pick = i0;
    for (long i = i0; i < i1; ++i) {
      const float x = ld_logit<T>(row, i);
      if (order_key(x) < lo_key) continue;
      const unsigned long long w = (unsigned long long)(__expf((x - M) * inv_temp) * SAMPLE_FIX);
      pick = i;
      if (target < acc + w) break;
      acc += w;
    }
    s_pick = pick;
  }
  __syncthreads();
  if (tid == 0) out[blockIdx.x] = s_pick >= 0 ? s_pick : arg;       // no mass at all (cannot happen: the maximum weighs 2^40)
}

}  // namespace mt

// logits [rows, V] fp32 (is_bf16 = 0) or bf16, contiguous; uniform [rows] fp32 in [0, 1) (unused when greedy); out [rows] int64.
// topk <= 0 and nucleus_p outside (0, 1) switch the respective mask off.
extern "C" int mt_sample(const void* logits, int is_bf16, const float* uniform, long rows, long V, int topk, float nucleus_p, float temperature,
                         int greedy, long long* out, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (V < 1 || (!greedy && !uniform)) return -1;
  const float inv_t = 1.f / (temperature > 1e-6f ? temperature : 1e-6f);
  if (is_bf16)
    mt::sample_kernel<__nv_bfloat16><<<(unsigned)rows, mt::SAMPLE_THREADS, 0, st>>>((const __nv_bfloat16*)logits, uniform, V, topk, nucleus_p, inv_t,
                                                                                   greedy, out);
  else
    mt::sample_kernel<float><<<(unsigned)rows, mt::SAMPLE_THREADS, 0, st>>>((const float*)logits, uniform, V, topk, nucleus_p, inv_t, greedy, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
