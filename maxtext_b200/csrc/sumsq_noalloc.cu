// Allocation-free variant of the two-stage sum of squares (see no_alloc.h for who needs it and why).
// Stage 1 writes one partial per block into a scratch array that is part of the library image; stage 2 adds
// them up in a fixed order and accumulates into the caller's output. Grid sizes and arithmetic are those of
// mt_sumsq in loss_optim.cu, so both entry points return the same value on the same device.
#include "no_alloc.h"
#include <stdint.h>
#include <atomic>
#include <mutex>

extern "C" int mt_sumsq_num_partials(long n, int sms);   // loss_optim.cu: grid size of stage 1

namespace {

constexpr int NA_THREADS = 512;

// The scratch itself. In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float g_noalloc_partials[MT_SUMSQ_NOALLOC_MAX_PARTIALS];

__device__ __forceinline__ float na_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float na_block_sum(float v, float* sh) {
  v = na_warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (NA_THREADS >> 5)) ? sh[threadIdx.x] : 0.f;
  if (w == 0) t = na_warp_sum(t);
  return t;   // valid in thread 0
}

__global__ void __launch_bounds__(NA_THREADS) na_stage1(const float* __restrict__ x, long long n, float* __restrict__ partials) {
  __shared__ float sh[32];
  float acc = 0.f;
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 t = reinterpret_cast<const float4*>(x)[i];
    acc += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
  }
  if (blockIdx.x == 0) {
    for (long long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) acc += x[i] * x[i];
  }
  const float s = na_block_sum(acc, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

__global__ void __launch_bounds__(NA_THREADS) na_stage2(const float* __restrict__ partials, int nparts, float* __restrict__ out) {
  __shared__ float sh[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) acc += partials[i];
  const float s = na_block_sum(acc, sh);
  if (threadIdx.x == 0) *out += s;
}

constexpr int NA_MAX_DEVICES = 64;

// Per-device set-up result, published once: `ready` is stored with release order after the other two fields, and
// read with acquire order, so a host thread that sees ready != 0 also sees the pointer and the SM count.
struct NaDevice {
  std::atomic<int> ready{0};
  float* scratch = nullptr;
  int sms = 0;
  std::mutex init;
};
NaDevice g_dev[NA_MAX_DEVICES];

}  // namespace

extern "C" const char* mt_sumsq_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "success";
    case -1: return "bad argument: null pointer, negative length or misaligned input";
    case -2: return "input longer than MT_SUMSQ_NOALLOC_MAX_ELEMS";
    case -3: return "this device needs more stage-1 partials than the built-in scratch (MT_SUMSQ_NOALLOC_MAX_PARTIALS) holds";
    case -4: return "could not obtain the device address of the built-in scratch (cudaGetSymbolAddress failed)";
    case -5: return "kernel launch failed";
    case -6: return "device ordinal beyond the 64 devices this entry point keeps set-up state for (or no current device)";
    default: return "unknown error code";
  }
}

extern "C" int mt_sumsq_noalloc(const float* x, long long n, float* out, cudaStream_t stream) {
  if (!x || !out || n < 0 || (reinterpret_cast<uintptr_t>(x) & 15u)) return -1;
  if (n > MT_SUMSQ_NOALLOC_MAX_ELEMS) return -2;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NA_MAX_DEVICES) return -6;
  NaDevice& d = g_dev[dev];
  if (!d.ready.load(std::memory_order_acquire)) {
    // one-time set-up for this device (it is current): resolve the device address of the scratch symbol
    std::lock_guard<std::mutex> lock(d.init);
    if (!d.ready.load(std::memory_order_relaxed)) {
      float* ptr = nullptr;
      if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_partials) != cudaSuccess || !ptr) return -4;
      int sms = 0;
      if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return -4;
      d.sms = sms;
      d.scratch = ptr;
      d.ready.store(1, std::memory_order_release);
    }
  }
  if (n == 0) return 0;
  const int parts = mt_sumsq_num_partials((long)n, d.sms);
  if (parts > MT_SUMSQ_NOALLOC_MAX_PARTIALS) return -3;
  float* scratch = d.scratch;
  // each launch's own return code is read (cudaLaunchKernel), so an earlier, unrelated error of the caller is neither
  // reported as ours nor cleared
  long long n_arg = n;
  int parts_arg = parts;
  const float* x_arg = x;
  void* a1[] = {(void*)&x_arg, (void*)&n_arg, (void*)&scratch};
  if (cudaLaunchKernel((const void*)na_stage1, dim3(parts), dim3(NA_THREADS), a1, 0, stream) != cudaSuccess) return -5;
  const float* sc = scratch;
  void* a2[] = {(void*)&sc, (void*)&parts_arg, (void*)&out};
  if (cudaLaunchKernel((const void*)na_stage2, dim3(1), dim3(NA_THREADS), a2, 0, stream) != cudaSuccess) return -5;
  return 0;
}
