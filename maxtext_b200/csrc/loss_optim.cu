// Cross-entropy (forward + in-place d(logits)), fused AdamW over a flat parameter shard, and the
// deterministic two-stage sum of squares used for the global gradient norm.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>

namespace mt {

struct alignas(16) bf16x8 { __nv_bfloat162 v[4]; };

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum2(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------------------------------------ cross entropy
// One block per token row of logits [rows, V] (bf16, leading stride ld). Pass 1: online (max, sum-exp)
// and the target logit. Pass 2 (optional): overwrite the row with
//   dlogits = w * ((1 + 2 z lse) * softmax - onehot(target))
// so the caller can feed it straight into the dX / dW GEMMs. loss = lse - logit[target] + z * lse^2.
__global__ void __launch_bounds__(1024) xent_kernel(__nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                                                    const float* __restrict__ weights, float z_loss, float* __restrict__ loss_out,
                                                    float* __restrict__ z_out, long ld, int V, int write_grad) {
  __shared__ float s_m[32], s_s[32];
  __shared__ float s_lse;
  const long row = blockIdx.x;
  __nv_bfloat16* lrow = logits + row * ld;
  const int tgt = targets[row];
  const int nvec = V / 8;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    bf16x8 p = *reinterpret_cast<const bf16x8*>(lrow + i * 8);
    float f[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 t = __bfloat1622float2(p.v[e]);
      f[2 * e] = t.x;
      f[2 * e + 1] = t.y;
    }
    float lm = f[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) lm = fmaxf(lm, f[e]);
    const float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += expf(f[e] - nm);
    s = s * expf(m - nm) + acc;
    m = nm;
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) {   // tail when V % 8 != 0
    const float f = __bfloat162float(lrow[i]);
    const float nm = fmaxf(m, f);
    s = s * expf(m - nm) + expf(f - nm);
    m = nm;
  }
  // block reduce (max, sum)
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  float wm = warp_max(m);
  float ws = warp_sum2(s * ((m == -INFINITY) ? 0.f : expf(m - wm)));
  if (l == 0) { s_m[w] = wm; s_s[w] = ws; }
  __syncthreads();
  if (w == 0) {
    const int nw = blockDim.x >> 5;
    float mm = (l < nw) ? s_m[l] : -INFINITY;
    float ss = (l < nw) ? s_s[l] : 0.f;
    const float gm = warp_max(mm);
    const float gs = warp_sum2(ss * ((mm == -INFINITY) ? 0.f : expf(mm - gm)));
    if (l == 0) {
      const float lse = gm + logf(gs);
      s_lse = lse;
      const float tl = (tgt >= 0 && tgt < V) ? __bfloat162float(lrow[tgt]) : 0.f;
      const float z = z_loss * lse * lse;
      loss_out[row] = lse - tl + z;
      if (z_out) z_out[row] = z;
    }
  }
  __syncthreads();
  if (!write_grad) return;
  const float lse = s_lse;
  const float wgt = weights ? weights[row] : 1.f;
  const float coef = wgt * (1.f + 2.f * z_loss * lse);
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    bf16x8 p = *reinterpret_cast<const bf16x8*>(lrow + i * 8);
    bf16x8 o;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 t = __bfloat1622float2(p.v[e]);
      float a = coef * expf(t.x - lse), b = coef * expf(t.y - lse);
      const int c0 = i * 8 + 2 * e;
      if (c0 == tgt) a -= wgt;
      if (c0 + 1 == tgt) b -= wgt;
      o.v[e] = __floats2bfloat162_rn(a, b);
    }
    *reinterpret_cast<bf16x8*>(lrow + i * 8) = o;
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) {
    float a = coef * expf(__bfloat162float(lrow[i]) - lse);
    if (i == tgt) a -= wgt;
    lrow[i] = __float2bfloat16_rn(a);
  }
}

// ------------------------------------------------------------------------------------------------ AdamW
// optax.adamw: m = b1 m + (1-b1) g; v = b2 v + (1-b2) g^2; u = (m/bc1) / (sqrt(v/bc2 + eps_root) + eps);
// p -= lr * (u + wd * p). g is pre-multiplied by *grad_scale (clip factor / total weights, device scalar).
// Writes the fp32 master and, when given, the bf16 compute copy in the same pass.
template <typename MT>
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, MT* __restrict__ m, float* __restrict__ v,
                             __nv_bfloat16* __restrict__ shadow, long n, float lr, float b1, float b2, float eps, float eps_root,
                             float wd, float inv_bc1, float inv_bc2, const float* __restrict__ grad_scale) {
  const float gs = *grad_scale;
  const long n4 = n / 4;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    const float4 gg = reinterpret_cast<const float4*>(g)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float mm[4];
    if (sizeof(MT) == 4) {
      float4 t = reinterpret_cast<float4*>(m)[i];
      mm[0] = t.x; mm[1] = t.y; mm[2] = t.z; mm[3] = t.w;
    } else {
      const __nv_bfloat162* mp = reinterpret_cast<const __nv_bfloat162*>(m) + 2 * i;
      float2 a = __bfloat1622float2(mp[0]), b = __bfloat1622float2(mp[1]);
      mm[0] = a.x; mm[1] = a.y; mm[2] = b.x; mm[3] = b.y;
    }
    float pa[4] = {pp.x, pp.y, pp.z, pp.w};
    const float ga[4] = {gg.x * gs, gg.y * gs, gg.z * gs, gg.w * gs};
    float va[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      mm[e] = b1 * mm[e] + (1.f - b1) * ga[e];
      va[e] = b2 * va[e] + (1.f - b2) * ga[e] * ga[e];
      const float u = (mm[e] * inv_bc1) / (sqrtf(va[e] * inv_bc2 + eps_root) + eps);
      pa[e] = pa[e] - lr * (u + wd * pa[e]);
    }
    reinterpret_cast<float4*>(p)[i] = make_float4(pa[0], pa[1], pa[2], pa[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(va[0], va[1], va[2], va[3]);
    if (sizeof(MT) == 4) {
      reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    } else {
      __nv_bfloat162* mp = reinterpret_cast<__nv_bfloat162*>(m) + 2 * i;
      mp[0] = __floats2bfloat162_rn(mm[0], mm[1]);
      mp[1] = __floats2bfloat162_rn(mm[2], mm[3]);
    }
    if (shadow) {
      __nv_bfloat162* sp = reinterpret_cast<__nv_bfloat162*>(shadow) + 2 * i;
      sp[0] = __floats2bfloat162_rn(pa[0], pa[1]);
      sp[1] = __floats2bfloat162_rn(pa[2], pa[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ sum of squares
// Stage 1: each block writes one partial to `partials` (no atomics, fixed order); stage 2: one block sums the
// partials in a fixed order and ADDS the result to *out. Bitwise reproducible for a given size and grid.
constexpr int SUMSQ_THREADS = 512;

__device__ __forceinline__ float block_sum_512(float v, float* sh) {
  v = warp_sum2(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (SUMSQ_THREADS >> 5)) ? sh[threadIdx.x] : 0.f;
  if (w == 0) t = warp_sum2(t);
  return t;   // valid in thread 0
}

__global__ void __launch_bounds__(SUMSQ_THREADS) sumsq_stage1(const float* __restrict__ x, long n, float* __restrict__ partials) {
  __shared__ float sh[32];
  float acc = 0.f;
  const long n4 = n / 4;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) {
    const float4 t = reinterpret_cast<const float4*>(x)[i];
    acc += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
  }
  if (blockIdx.x == 0) {
    for (long i = n4 * 4 + threadIdx.x; i < n; i += blockDim.x) acc += x[i] * x[i];
  }
  const float s = block_sum_512(acc, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

__global__ void __launch_bounds__(SUMSQ_THREADS) sumsq_stage2(const float* __restrict__ partials, int nparts, float* __restrict__ out) {
  __shared__ float sh[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) acc += partials[i];
  const float s = block_sum_512(acc, sh);
  if (threadIdx.x == 0) *out += s;
}

}  // namespace mt

using namespace mt;

extern "C" int mt_xent(void* logits, const int* targets, const float* weights, float z_loss, float* loss_out, float* z_out, long rows,
                       long ld, int V, int write_grad, cudaStream_t st) {
  if (rows <= 0) return 0;
  if (ld % 8) return -1;
  xent_kernel<<<(unsigned)rows, 1024, 0, st>>>((__nv_bfloat16*)logits, targets, weights, z_loss, loss_out, z_out, ld, V, write_grad);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int mt_adamw(float* p, const float* g, void* m, int m_is_bf16, float* v, void* shadow, long n, float lr, float b1, float b2,
                        float eps, float eps_root, float wd, float bc1, float bc2, const float* grad_scale, int sms, cudaStream_t st) {
  if (n % 4) return -1;
  if (n == 0) return 0;
  long blocks = (n / 4 + 255) / 256;
  int grid = (int)(blocks < (long)sms * 16 ? blocks : (long)sms * 16);
  if (m_is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, g, (__nv_bfloat16*)m, v, (__nv_bfloat16*)shadow, n, lr, b1, b2, eps, eps_root,
                                                      wd, 1.f / bc1, 1.f / bc2, grad_scale);
  else
    adamw_kernel<float><<<grid, 256, 0, st>>>(p, g, (float*)m, v, (__nv_bfloat16*)shadow, n, lr, b1, b2, eps, eps_root, wd, 1.f / bc1,
                                              1.f / bc2, grad_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Number of stage-1 blocks (= floats of scratch needed) for an input of n floats on a device with `sms` SMs.
extern "C" int mt_sumsq_num_partials(long n, int sms) {
  long blocks = (n / 4 + SUMSQ_THREADS - 1) / SUMSQ_THREADS;
  long cap = (long)sms * 8;
  if (blocks < 1) blocks = 1;
  return (int)(blocks < cap ? blocks : cap);
}

// out[0] += sum(x^2). `partials` must hold mt_sumsq_num_partials(n, sms) floats of scratch.
extern "C" int mt_sumsq(const float* x, long n, float* partials, float* out, int sms, cudaStream_t st) {
  const int parts = mt_sumsq_num_partials(n, sms);
  sumsq_stage1<<<parts, SUMSQ_THREADS, 0, st>>>(x, n, partials);
  sumsq_stage2<<<1, SUMSQ_THREADS, 0, st>>>(partials, parts, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
