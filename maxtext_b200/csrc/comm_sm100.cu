// Communication kernels over NVLink peer memory (symmetric buffers mapped into every rank of a node).
//
//   * signal / wait: per-peer epoch flags with release / acquire at system scope. Every wait is bounded: when the
//     limit passes the kernel records ST_TIMEOUT_FLAG in the status word and returns, it never spins forever.
//   * rs_sumsq: fused gradient reduce-scatter. Each rank reads ITS chunk of every peer's full gradient buffer
//     with plain peer loads, adds the copies in rank order (bitwise reproducible), applies the bucket scale,
//     writes (or accumulates into) its fp32 gradient shard and emits the sum-of-squares partials of the
//     global gradient norm in the same pass. What the reference gets from an NCCL reduce-scatter followed by
//     separate cast / norm fusions.
//   * gather_segments: pulls the peers' parameter shards into the local full buffer, segment by segment, and
//     publishes one flag per segment; the GEMM in gemm_sm100.cu runs the same loop in spare CTAs of its own
//     launch so that tiles start as soon as their rows have arrived.
// No kernel here uses bulk-tensor copies from peer memory: remote data is read with ld.global by the copying CTA.
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mt {

enum : int { COMM_ST_TIMEOUT_FLAG = 4 };

__device__ __forceinline__ uint64_t comm_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Thread r tells rank r that this rank reached `epoch` on slot `slot`: flags[r][slot * world + my_rank] = epoch.
__global__ void signal_kernel(int* const* __restrict__ peer_flags, int slot, int my_rank, int world, int epoch) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    st_release_sys(peer_flags[r] + slot * world + my_rank, epoch);
  }
}

// Wait until every peer's flag on `slot` reached `epoch`, at most limit_ns.
__global__ void wait_kernel(const int* __restrict__ my_flags, int slot, int world, int epoch, int* status, unsigned long long limit_ns) {
  const int r = threadIdx.x;
  if (r >= world) return;
  const int* f = my_flags + slot * world + r;
  const uint64_t t0 = comm_timer_ns();
  while (ld_acquire_sys(f) < epoch) {
    if (comm_timer_ns() - t0 > limit_ns) {
      atomicCAS(status, 0, COMM_ST_TIMEOUT_FLAG);
      return;
    }
    __nanosleep(200);
  }
}

constexpr int RS_THREADS = 512;

__device__ __forceinline__ float rs_block_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (RS_THREADS >> 5)) ? sh[threadIdx.x] : 0.f;
  if (w == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  return t;
}

// dst[i] (+)= scale * sum_r peer[r][offset + i];  partials[block] = sum of squares of what was written this call.
// A thread keeps RS_UNROLL independent 16-byte loads in flight per peer: with one load per thread the kernel is bound by the
// NVLink round trip (measured 183 GB/s at two ranks), not by the links. Ranks are added in rank order for every element, so the
// result does not depend on the unrolling.
constexpr int RS_UNROLL = 8;

__device__ __forceinline__ void rs_finish(float4& s, float scale, int accumulate, float4* dst, long i, float& acc) {
  s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
  if (accumulate) {
    const float4 o = dst[i];
    s.x += o.x; s.y += o.y; s.z += o.z; s.w += o.w;
  }
  dst[i] = s;
  acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
}

__global__ void __launch_bounds__(RS_THREADS)
rs_sumsq_kernel(const float* const* __restrict__ peer, long offset, long n, float* __restrict__ dst, int accumulate, float scale,
                int world, float* __restrict__ partials) {
  __shared__ float sh[32];
  float acc = 0.f;
  const long n4 = n / 4;
  const long stride = (long)gridDim.x * blockDim.x;
  float4* dst4 = reinterpret_cast<float4*>(dst);
  long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
  for (; i + (RS_UNROLL - 1) * stride < n4; i += RS_UNROLL * stride) {
    float4 s[RS_UNROLL];
#pragma unroll
    for (int u = 0; u < RS_UNROLL; ++u) s[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4* src = reinterpret_cast<const float4*>(peer[r] + offset);
      float4 v[RS_UNROLL];
#pragma unroll
      for (int u = 0; u < RS_UNROLL; ++u) v[u] = src[i + u * stride];
#pragma unroll
      for (int u = 0; u < RS_UNROLL; ++u) { s[u].x += v[u].x; s[u].y += v[u].y; s[u].z += v[u].z; s[u].w += v[u].w; }
    }
#pragma unroll
    for (int u = 0; u < RS_UNROLL; ++u) rs_finish(s[u], scale, accumulate, dst4, i + u * stride, acc);
  }
  for (; i < n4; i += stride) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 v = reinterpret_cast<const float4*>(peer[r] + offset)[i];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    rs_finish(s, scale, accumulate, dst4, i, acc);
  }
  const float t = rs_block_sum(acc, sh);
  if (threadIdx.x == 0 && partials) partials[blockIdx.x] = t;
}

// The same reduce-scatter with the sum done inside the NVSwitch: `mc` is the multicast address of the symmetric gradient
// buffer, and one multimem.ld_reduce returns the element-wise sum of every rank's copy, so each element costs this SM one
// load instead of `world` loads (and the reduction traffic never enters the GPU). U of them are in flight per thread.
__device__ __forceinline__ float4 mc_ld_reduce(const float* p) {
  float4 s;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(s.x), "=f"(s.y), "=f"(s.z), "=f"(s.w)
               : "l"(p)
               : "memory");
  return s;
}

template <int U>
__global__ void __launch_bounds__(RS_THREADS)
rs_sumsq_mc_kernel(const float* __restrict__ mc, long offset, long n, float* __restrict__ dst, int accumulate, float scale,
                   float* __restrict__ partials) {
  __shared__ float sh[32];
  float acc = 0.f;
  const long n4 = n / 4;
  const long stride = (long)gridDim.x * blockDim.x;
  const float* base = mc + offset;
  float4* dst4 = reinterpret_cast<float4*>(dst);
  long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
  for (; i + (U - 1) * stride < n4; i += U * stride) {
    float4 s[U];
#pragma unroll
    for (int u = 0; u < U; ++u) s[u] = mc_ld_reduce(base + 4 * (i + u * stride));
#pragma unroll
    for (int u = 0; u < U; ++u) rs_finish(s[u], scale, accumulate, dst4, i + u * stride, acc);
  }
  for (; i < n4; i += stride) {
    float4 s = mc_ld_reduce(base + 4 * i);
    rs_finish(s, scale, accumulate, dst4, i, acc);
  }
  const float t = rs_block_sum(acc, sh);
  if (threadIdx.x == 0 && partials) partials[blockIdx.x] = t;
}

__global__ void __launch_bounds__(RS_THREADS) rs_stage2_kernel(const float* __restrict__ partials, int nparts, float* __restrict__ out) {
  __shared__ float sh[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) acc += partials[i];
  const float t = rs_block_sum(acc, sh);
  if (threadIdx.x == 0) *out += t;
}

// Segment s of the gathered buffer = rank (s / segs_per_chunk), piece (s % segs_per_chunk) of its chunk.
__global__ void __launch_bounds__(256)
gather_segments_kernel(const uint4* const* __restrict__ peer_shards, uint4* __restrict__ full, long chunk_vec, long seg_vec, int segs_per_chunk,
                       int n_segs, int first_seg, int* __restrict__ seg_flags) {
  for (int k = blockIdx.x; k < n_segs; k += gridDim.x) {
    const int s = (first_seg + k) % n_segs;
    const int r = s / segs_per_chunk;
    const long lo = (long)(s % segs_per_chunk) * seg_vec;
    const long hi = lo + seg_vec < chunk_vec ? lo + seg_vec : chunk_vec;
    const uint4* src = peer_shards[r];
    uint4* dst = full + (long)r * chunk_vec;
    long i = lo + threadIdx.x;
    for (; i + 7 * (long)blockDim.x < hi; i += 8 * (long)blockDim.x) {     // eight independent peer loads in flight per thread
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = src[i + u * (long)blockDim.x];
#pragma unroll
      for (int u = 0; u < 8; ++u) dst[i + u * (long)blockDim.x] = v[u];
    }
    for (; i < hi; i += blockDim.x) dst[i] = src[i];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0 && seg_flags) atomicExch(seg_flags + s, 1);
  }
}

// out[r * rows + i, :] = bf16(acc_r[i, :]) for every rank r: the all-gather half of an all-reduce whose reduce-scatter half was
// done by the GEMM epilogue (gemm_sm100.cu, mt_gemm_bf16_rs). Peer chunks are read with plain loads.
__global__ void __launch_bounds__(256)
gather_cvt_kernel(const float4* const* __restrict__ peer_acc, long chunk_vec4, int world, uint2* __restrict__ out) {
  const long total = chunk_vec4 * world;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int r = (int)(i / chunk_vec4);
    const float4 v = peer_acc[r][i - (long)r * chunk_vec4];
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&lo);
    o.y = *reinterpret_cast<uint32_t*>(&hi);
    out[i] = o;
  }
}

// out[i] = sum over sources s (in order) of staged[s * chunk + i], fp32 accumulation, bf16 in and out: the owner's half of a
// reduce-scatter whose partial tiles were stored into `staged` by the peers' GEMM epilogues.
__global__ void __launch_bounds__(256)
reduce_staged_kernel(const uint4* __restrict__ staged, long chunk_vec, int world, uint4* __restrict__ out) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < chunk_vec; i += (long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < world; ++s) {
      const uint4 v = staged[(long)s * chunk_vec + i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    out[i] = o;
  }
}

}  // namespace mt

using namespace mt;

extern "C" int mt_reduce_staged(const void* staged, long chunk_elems, int world, void* out, int ctas, cudaStream_t st) {
  if (chunk_elems % 8) return -1;
  reduce_staged_kernel<<<ctas, 256, 0, st>>>(reinterpret_cast<const uint4*>(staged), chunk_elems / 8, world, reinterpret_cast<uint4*>(out));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int mt_gather_cvt(const float* const* peer_acc, long chunk_elems, int world, void* out, int ctas, cudaStream_t st) {
  if (chunk_elems % 4) return -1;
  gather_cvt_kernel<<<ctas, 256, 0, st>>>(reinterpret_cast<const float4* const*>(peer_acc), chunk_elems / 4, world,
                                          reinterpret_cast<uint2*>(out));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int mt_comm_signal(int* const* peer_flags, int slot, int my_rank, int world, int epoch, cudaStream_t st) {
  if (world > 32) return -1;
  signal_kernel<<<1, 32, 0, st>>>(peer_flags, slot, my_rank, world, epoch);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int mt_comm_wait(const int* my_flags, int slot, int world, int epoch, int* status, unsigned long long limit_ns, cudaStream_t st) {
  if (world > 32) return -1;
  wait_kernel<<<1, 32, 0, st>>>(my_flags, slot, world, epoch, status, limit_ns);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int mt_rs_num_partials(long n, int ctas) {
  long blocks = (n / 4 + RS_THREADS - 1) / RS_THREADS;
  if (blocks < 1) blocks = 1;
  return (int)(blocks < ctas ? blocks : ctas);
}

// partials: scratch of mt_rs_num_partials(n, ctas) floats; sumsq_out[0] += sum of squares (pass nullptr to skip).
extern "C" int mt_rs_sumsq(const float* const* peer, long offset, long n, float* dst, int accumulate, float scale, int world, float* partials,
                           float* sumsq_out, int ctas, cudaStream_t st) {
  if (n % 4 || offset % 4) return -1;
  if (n == 0) return 0;
  const int parts = mt_rs_num_partials(n, ctas);
  rs_sumsq_kernel<<<parts, RS_THREADS, 0, st>>>(peer, offset, n, dst, accumulate, scale, world, partials);
  if (sumsq_out && partials) rs_stage2_kernel<<<1, RS_THREADS, 0, st>>>(partials, parts, sumsq_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// mc: multicast (NVLS) address of the symmetric buffer; otherwise as mt_rs_sumsq.
extern "C" int mt_rs_sumsq_mc(const float* mc, long offset, long n, float* dst, int accumulate, float scale, float* partials, float* sumsq_out,
                              int ctas, cudaStream_t st) {
  if (n % 4 || offset % 4 || !mc) return -1;
  if (n == 0) return 0;
  const int parts = mt_rs_num_partials(n, ctas);
  // In-switch loads in flight per thread: 1 is the form every multi-GPU step time of this repository was measured with; 8
  // (MAXTEXT_B200_RS_MC_UNROLL=8) is 2.9x faster in isolation at two ranks but has no same-box step measurement at 4 / 8 ranks.
  static const int unroll = [] { const char* e = getenv("MAXTEXT_B200_RS_MC_UNROLL"); return (e && atoi(e) == 8) ? 8 : 1; }();
  if (unroll == 8) rs_sumsq_mc_kernel<8><<<parts, RS_THREADS, 0, st>>>(mc, offset, n, dst, accumulate, scale, partials);
  else rs_sumsq_mc_kernel<1><<<parts, RS_THREADS, 0, st>>>(mc, offset, n, dst, accumulate, scale, partials);
  if (sumsq_out && partials) rs_stage2_kernel<<<1, RS_THREADS, 0, st>>>(partials, parts, sumsq_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Stand-alone all-gather by peer loads (the GEMM-fused form runs the same kernel body inside the GEMM launch).
extern "C" int mt_gather_segments(const void* const* peer_shards, void* full, long chunk_bytes, long seg_bytes, int world, int* seg_flags,
                                  int ctas, cudaStream_t st) {
  if (chunk_bytes % 16 || seg_bytes % 16) return -1;
  const long chunk_vec = chunk_bytes / 16, seg_vec = seg_bytes / 16;
  const int spc = (int)((chunk_vec + seg_vec - 1) / seg_vec);
  gather_segments_kernel<<<ctas, 256, 0, st>>>(reinterpret_cast<const uint4* const*>(peer_shards), reinterpret_cast<uint4*>(full), chunk_vec,
                                               seg_vec, spc, spc * world, 0, seg_flags);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// The same all-gather issued to the copy engines: one peer-to-local DMA per rank, no SM time. `peer_ptrs` are host values.
// The copies are spread over a few helper streams that fork from and join back into `st`, so several copy engines (and several
// NVLink peers) work at once; issued back to back on one stream they run one after another.
namespace {
constexpr int kDmaLanes = 4;
struct DmaLanes {
  cudaStream_t s[kDmaLanes];
  cudaEvent_t fork, join[kDmaLanes];
  bool ok = false;
};
DmaLanes* dma_lanes() {
  static DmaLanes lanes[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  DmaLanes& l = lanes[dev];
  if (!l.ok) {
    if (cudaEventCreateWithFlags(&l.fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    for (int i = 0; i < kDmaLanes; ++i)
      if (cudaStreamCreateWithFlags(&l.s[i], cudaStreamNonBlocking) != cudaSuccess ||
          cudaEventCreateWithFlags(&l.join[i], cudaEventDisableTiming) != cudaSuccess)
        return nullptr;
    l.ok = true;
  }
  return &l;
}
}  // namespace

extern "C" int mt_gather_dma(const long long* peer_ptrs, void* full, long chunk_bytes, int world, int first, cudaStream_t st) {
  DmaLanes* l = world > 2 ? dma_lanes() : nullptr;
  if (l && cudaEventRecord(l->fork, st) != cudaSuccess) return -2;
  const int lanes = l ? (world - 1 < kDmaLanes ? world - 1 : kDmaLanes) : 0;
  for (int i = 0; i < lanes; ++i)
    if (cudaStreamWaitEvent(l->s[i], l->fork, 0) != cudaSuccess) return -2;
  for (int k = 0; k < world; ++k) {
    const int r = (first + k) % world;               // start at a different peer on every rank so the links are used evenly
    cudaStream_t on = lanes ? l->s[k % lanes] : st;
    cudaError_t e = cudaMemcpyAsync(static_cast<char*>(full) + (long)r * chunk_bytes, reinterpret_cast<const void*>(peer_ptrs[r]), (size_t)chunk_bytes,
                                    cudaMemcpyDeviceToDevice, on);
    if (e != cudaSuccess) return -2;
  }
  for (int i = 0; i < lanes; ++i)
    if (cudaEventRecord(l->join[i], l->s[i]) != cudaSuccess || cudaStreamWaitEvent(st, l->join[i], 0) != cudaSuccess) return -2;
  return 0;
}
