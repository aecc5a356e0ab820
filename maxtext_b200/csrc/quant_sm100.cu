// Per-tensor FP8 quantisation for the 8-bit GEMM path: absolute maximum, then scale-and-convert to E4M3 / E5M2, writing the
// row-major copy and / or the transposed copy in one pass (the three products of a linear layer need both layouts because
// the 8-bit tensor-core path takes K-major operands only). The role of the scaling + cast fusions that the reference gets from
// its quantisation providers (src/maxtext/layers/quantizations.py: Fp8 / NANOOFp8 dot_general wrappers).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mt {

// amax[0] = max(amax[0], max |x|); amax must hold a non-negative value (0 to start a fresh maximum).
__global__ void __launch_bounds__(256) amax_kernel(const uint4* __restrict__ x, long n_vec, float* __restrict__ amax) {
  float m = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n_vec; i += (long)gridDim.x * blockDim.x) {
    const uint4 v = x[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float sh[8];
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int j = 1; j < 8; ++j) m = fmaxf(m, sh[j]);
    atomicMax(reinterpret_cast<int*>(amax), __float_as_int(m));     // non-negative floats order like their bit patterns
  }
}

template <bool E5M2>
__device__ __forceinline__ uint8_t to_fp8(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
}

// x [R, C] bf16 -> q [R, C] and / or qt [C, R] (8-bit), values multiplied by fmax / amax first; dequant[0] = amax / fmax.
// One 64 x 64 tile per block of 256 threads; R and C are multiples of 64.
template <bool E5M2>
__global__ void __launch_bounds__(256)
quantize_kernel(const __nv_bfloat16* __restrict__ x, int R, int C, const float* __restrict__ amax, float fmax, uint8_t* __restrict__ q,
                uint8_t* __restrict__ qt, float* __restrict__ dequant) {
  __shared__ uint8_t tile[64][80];              // padded rows: the transposed read walks a column
  const float am = *amax;
  const float scale = am > 0.f ? fmax / am : 1.f;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) *dequant = am > 0.f ? am / fmax : 1.f;
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tr = threadIdx.x >> 2, tc = (threadIdx.x & 3) * 16;
  const uint4* src = reinterpret_cast<const uint4*>(x + (long)(r0 + tr) * C + c0 + tc);
  uint8_t out[16];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint4 v = src[h];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(p[j]);
      out[h * 8 + 2 * j] = to_fp8<E5M2>(f.x * scale);
      out[h * 8 + 2 * j + 1] = to_fp8<E5M2>(f.y * scale);
    }
  }
  if (q) *reinterpret_cast<uint4*>(q + (long)(r0 + tr) * C + c0 + tc) = *reinterpret_cast<uint4*>(out);
  if (qt) {
    *reinterpret_cast<uint4*>(&tile[tr][tc]) = *reinterpret_cast<uint4*>(out);
    __syncthreads();
    uint8_t col[16];                             // thread (tr, tc): column tr of the tile, rows tc .. tc + 15
#pragma unroll
    for (int j = 0; j < 16; ++j) col[j] = tile[tc + j][tr];
    *reinterpret_cast<uint4*>(qt + (long)(c0 + tr) * R + r0 + tc) = *reinterpret_cast<uint4*>(col);
  }
}

}  // namespace mt

using namespace mt;

extern "C" int mt_amax(const void* x, long n, float* amax, int sms, cudaStream_t st) {
  if (n % 8) return -1;
  long blocks = (n / 8 + 255) / 256;
  const int grid = (int)(blocks < sms * 8 ? blocks : sms * 8);
  amax_kernel<<<grid > 0 ? grid : 1, 256, 0, st>>>(reinterpret_cast<const uint4*>(x), n / 8, amax);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// fmt: 0 = E4M3 (max 448), 1 = E5M2 (max 57344). q and qt may each be null.
extern "C" int mt_quantize_fp8(const void* x, int R, int C, const float* amax, int fmt, void* q, void* qt, float* dequant, cudaStream_t st) {
  if (R % 64 || C % 64) return -1;
  const dim3 grid(C / 64, R / 64);
  if (fmt == 0)
    quantize_kernel<false><<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), R, C, amax, 448.f, reinterpret_cast<uint8_t*>(q),
                                                 reinterpret_cast<uint8_t*>(qt), dequant);
  else
    quantize_kernel<true><<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), R, C, amax, 57344.f, reinterpret_cast<uint8_t*>(q),
                                                reinterpret_cast<uint8_t*>(qt), dequant);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
