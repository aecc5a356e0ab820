// Mixture-of-experts data movement for the dropless path: a stable counting sort of the (token, choice) pairs by expert
// into a row layout in which every expert's group is padded to a multiple of 128 rows (so that each 128-row GEMM tile
// belongs to one expert), the row gather with its deterministic backward, and the weighted combine with its backward.
// What the reference gets from jnp.argsort / take / ragged_dot preprocessing (src/maxtext/layers/moe.py:872-1063).
// Group sizes never visit the host: the grouped GEMM reads the offsets from device memory.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mt {

constexpr int SORT_THREADS = 1024;
constexpr int SORT_WARPS = SORT_THREADS / 32;
constexpr int PAD = 128;
constexpr int MAX_EXPERTS = 512;

// One CTA. idx[n] expert of pair j (pair j = token j / k, choice j % k).
//   sizes[E]      rows per expert
//   offs[E + 1]   first padded row of each expert; offs[E] = padded rows in use
//   blk_expert[]  expert of each 128-row block below offs[E]; blocks above it are set to 0
//   dest[n]       padded row of pair j (stable: pairs of one expert keep their order)
//   row_pair[rows_max]  pair stored in each padded row, -1 for padding rows
__global__ void __launch_bounds__(SORT_THREADS)
moe_sort_kernel(const int* __restrict__ idx, int n, int E, int rows_max, int* __restrict__ sizes, int* __restrict__ offs,
                int* __restrict__ blk_expert, int* __restrict__ dest, int* __restrict__ row_pair) {
  __shared__ int hist[MAX_EXPERTS];
  __shared__ int start[MAX_EXPERTS + 1];
  __shared__ int running[MAX_EXPERTS];
  extern __shared__ int warp_cnt[];          // [SORT_WARPS][E]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int e = tid; e < E; e += SORT_THREADS) { hist[e] = 0; running[e] = 0; }
  for (int r = tid; r < rows_max; r += SORT_THREADS) row_pair[r] = -1;
  __syncthreads();
  for (int j = tid; j < n; j += SORT_THREADS) atomicAdd(&hist[idx[j]], 1);
  __syncthreads();
  if (tid == 0) {
    int o = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = o;
      sizes[e] = hist[e];
      offs[e] = o;
      o += (hist[e] + PAD - 1) / PAD * PAD;
    }
    start[E] = o;
    offs[E] = o;
  }
  __syncthreads();
  for (int b = tid; b < rows_max / PAD; b += SORT_THREADS) {
    const int r = b * PAD;
    int e = 0;
    if (r < start[E]) {
      int lo = 0, hi = E - 1;                 // last expert whose start <= r
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (start[mid] <= r) lo = mid; else hi = mid - 1;
      }
      e = lo;
    }
    blk_expert[b] = e;
  }
  // stable placement, 1024 pairs per round
  for (int base = 0; base < n; base += SORT_THREADS) {
    for (int i = tid; i < SORT_WARPS * E; i += SORT_THREADS) warp_cnt[i] = 0;
    __syncthreads();
    const int j = base + tid;
    const bool live = j < n;
    const int e = live ? idx[j] : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (live && rank_in_warp == 0) warp_cnt[warp * E + e] = __popc(peers);
    __syncthreads();
    for (int x = tid; x < E; x += SORT_THREADS) {          // exclusive scan over the warps, per expert
      int acc = running[x];
      for (int w = 0; w < SORT_WARPS; ++w) {
        const int c = warp_cnt[w * E + x];
        warp_cnt[w * E + x] = acc;
        acc += c;
      }
      running[x] = acc;
    }
    __syncthreads();
    if (live) {
      const int d = start[e] + warp_cnt[warp * E + e] + rank_in_warp;
      dest[j] = d;
      row_pair[d] = j;
    }
    __syncthreads();
  }
}

// rows[r, :] = x[row_pair[r] / k, :] (zeros for padding rows), r < offs[E]; 16-byte vectors.
__global__ void __launch_bounds__(256)
moe_gather_kernel(const uint4* __restrict__ x, const int* __restrict__ row_pair, const int* __restrict__ offs, int E, int k, int vec_per_row,
                  uint4* __restrict__ rows) {
  const int used = offs[E];
  for (int r = blockIdx.x; r < used; r += gridDim.x) {
    const int pair = row_pair[r];
    uint4* dst = rows + (long)r * vec_per_row;
    if (pair < 0) {
      for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    } else {
      const uint4* src = x + (long)(pair / k) * vec_per_row;
      for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = src[i];
    }
  }
}

__device__ __forceinline__ void acc8(float* a, const uint4& v, float w) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    a[2 * i] += w * f.x;
    a[2 * i + 1] += w * f.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float* a) {
  uint4 o;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
  return o;
}

// out[t, :] = sum_c w[t, c] * y[dest[t*k + c], :]   (w == nullptr: plain sum, the backward of the gather). fp32 accumulation.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const uint4* __restrict__ y, const int* __restrict__ dest, const float* __restrict__ w, int T, int k, int vec_per_row,
                   uint4* __restrict__ out) {
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) {
      float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int c = 0; c < k; ++c) {
        const int r = dest[t * k + c];
        acc8(a, y[(long)r * vec_per_row + i], w ? w[t * k + c] : 1.f);
      }
      out[(long)t * vec_per_row + i] = pack8(a);
    }
  }
}

// Backward of the combine: dy[dest[t*k+c], :] = w[t,c] * dout[t, :];  dw[t,c] = <dout[t, :], y[dest[t*k+c], :]>;
// padding rows of dy are zeroed (they feed the weight-gradient product).
__global__ void __launch_bounds__(256)
moe_combine_bwd_kernel(const uint4* __restrict__ dout, const uint4* __restrict__ y, const int* __restrict__ row_pair,
                       const int* __restrict__ offs, int E, const float* __restrict__ w, int k, int vec_per_row, uint4* __restrict__ dy,
                       float* __restrict__ dw) {
  __shared__ float red[8];
  const int used = offs[E];
  for (int r = blockIdx.x; r < used; r += gridDim.x) {
    const int pair = row_pair[r];
    uint4* drow = dy + (long)r * vec_per_row;
    if (pair < 0) {
      for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) drow[i] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const float wt = w[pair];
    const uint4* g = dout + (long)(pair / k) * vec_per_row;
    const uint4* yr = y + (long)r * vec_per_row;
    float dot = 0.f;
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) {
      const uint4 gv = g[i];
      float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      acc8(a, gv, wt);
      drow[i] = pack8(a);
      const uint4 yv = yr[i];
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
      const __nv_bfloat162* yh = reinterpret_cast<const __nv_bfloat162*>(&yv);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 gf = __bfloat1622float2(gh[q]), yf = __bfloat1622float2(yh[q]);
        dot += gf.x * yf.x + gf.y * yf.y;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dot;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
      for (int q = 0; q < 8; ++q) s += red[q];
      dw[pair] = s;
    }
    __syncthreads();
  }
}

}  // namespace mt

using namespace mt;

extern "C" int mt_moe_sort(const int* idx, int n, int E, int rows_max, int* sizes, int* offs, int* blk_expert, int* dest, int* row_pair,
                           cudaStream_t st) {
  if (E > MAX_EXPERTS || rows_max % PAD || rows_max < n + 0) return -1;
  const size_t dyn = sizeof(int) * SORT_WARPS * E;
  static bool configured = false;
  if (!configured && dyn > 48 * 1024) {
    if (cudaFuncSetAttribute(moe_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn) != cudaSuccess) return -2;
    configured = true;
  }
  moe_sort_kernel<<<1, SORT_THREADS, dyn, st>>>(idx, n, E, rows_max, sizes, offs, blk_expert, dest, row_pair);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int mt_moe_gather(const void* x, const int* row_pair, const int* offs, int E, int k, int D, int rows_max, void* rows, int sms,
                             cudaStream_t st) {
  if (D % 8) return -1;
  const int grid = rows_max < sms * 8 ? rows_max : sms * 8;
  moe_gather_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint4*>(x), row_pair, offs, E, k, D / 8, reinterpret_cast<uint4*>(rows));
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int mt_moe_combine(const void* y, const int* dest, const float* w, int T, int k, int D, void* out, int sms, cudaStream_t st) {
  if (D % 8) return -1;
  const int grid = T < sms * 8 ? T : sms * 8;
  moe_combine_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint4*>(y), dest, w, T, k, D / 8, reinterpret_cast<uint4*>(out));
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int mt_moe_combine_bwd(const void* dout, const void* y, const int* row_pair, const int* offs, int E, const float* w, int k, int D,
                                  int rows_max, void* dy, float* dw, int sms, cudaStream_t st) {
  if (D % 8) return -1;
  const int grid = rows_max < sms * 8 ? rows_max : sms * 8;
  moe_combine_bwd_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint4*>(dout), reinterpret_cast<const uint4*>(y), row_pair, offs, E, w,
                                               k, D / 8, reinterpret_cast<uint4*>(dy), dw);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
