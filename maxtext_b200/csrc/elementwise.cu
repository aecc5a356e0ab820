// Memory-bound kernels of the decoder layer: RMSNorm (forward, backward), rotary embedding on a packed
// q|k|v tensor, gated activation (SwiGLU / GeGLU), embedding gather and its scatter-add backward.
// All are HBM-bandwidth bound: 16-byte vector accesses, one pass over the data where the row fits in
// registers, fp32 math.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mt {

struct alignas(16) bf16x8 { __nv_bfloat162 v[4]; };

__device__ __forceinline__ void unpack8(const bf16x8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float (&f)[8]) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over the TPR threads that share a row. TPR == 32: one warp per row; TPR == 256: one block per row.
template <int TPR>
__device__ __forceinline__ float row_sum(float v, float* smem) {
  v = warp_sum(v);
  if (TPR == 32) return v;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) smem[w] = v;
  __syncthreads();
  float t = (l < TPR / 32) ? smem[l] : 0.f;
  return warp_sum(t);
}

// ------------------------------------------------------------------------------------------------ RMSNorm forward
// y = bf16(x * rstd) * bf16(scale + offset), both roundings as in the reference layer.
template <int TPR, int VPT>
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ scale, float eps,
                                   float offset, __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int rows, int D) {
  __shared__ float red[8];
  const int rows_per_block = blockDim.x / TPR;
  const int r_in_block = threadIdx.x / TPR;
  const int tid = threadIdx.x % TPR;
  const long row = (long)blockIdx.x * rows_per_block + r_in_block;
  const bool active = row < rows;
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int col = (i * TPR + tid) * 8;
    if (active && col < D) {
      bf16x8 p = *reinterpret_cast<const bf16x8*>(x + row * D + col);
      unpack8(p, v[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  ss = row_sum<TPR>(ss, red);
  const float rstd = rsqrtf(ss / (float)D + eps);
  if (active && tid == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int col = (i * TPR + tid) * 8;
    if (active && col < D) {
      float o[8];
      if (scale) {
        float s[8];
        unpack8(*reinterpret_cast<const bf16x8*>(scale + col), s);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = bf16_round(v[i][e] * rstd) * bf16_round(s[e] + offset);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = v[i][e] * rstd;
      }
      *reinterpret_cast<bf16x8*>(y + row * D + col) = pack8(o);
    }
  }
}

// ------------------------------------------------------------------------------------------------ RMSNorm backward
// dx = rstd * (g - xhat * mean(g * xhat)), g = dy * (scale + offset);  dscale += sum_rows dy * xhat.
// Blocks stride over rows and keep per-column dscale partials in registers; each (block, row slot) writes its partial row
// into `partial`, and rms_dscale_reduce_kernel adds the rows up in index order: no atomics, so the result is bitwise
// reproducible.
template <int TPR, int VPT>
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ scale, const float* __restrict__ rstd_in, float offset,
                                   __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int D) {
  __shared__ float red[8];
  const int rows_per_block = blockDim.x / TPR;
  const int r_in_block = threadIdx.x / TPR;
  const int tid = threadIdx.x % TPR;
  float ds[VPT][8];
  float sc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int col = (i * TPR + tid) * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) { ds[i][e] = 0.f; sc[i][e] = 1.f; }
    if (scale && col < D) {
      float s[8];
      unpack8(*reinterpret_cast<const bf16x8*>(scale + col), s);
#pragma unroll
      for (int e = 0; e < 8; ++e) sc[i][e] = s[e] + offset;
    }
  }
  const long n_groups = ((long)rows + rows_per_block - 1) / rows_per_block;
  for (long grp = blockIdx.x; grp < n_groups; grp += gridDim.x) {
    const long row = grp * rows_per_block + r_in_block;
    const bool active = row < rows;
    const float rstd = active ? rstd_in[row] : 0.f;
    float g[VPT][8], xh[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int col = (i * TPR + tid) * 8;
      if (active && col < D) {
        float a[8], b[8];
        unpack8(*reinterpret_cast<const bf16x8*>(dy + row * D + col), a);
        unpack8(*reinterpret_cast<const bf16x8*>(x + row * D + col), b);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[i][e] = b[e] * rstd;
          g[i][e] = a[e] * sc[i][e];
          dot += g[i][e] * xh[i][e];
          ds[i][e] += a[e] * xh[i][e];
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) { xh[i][e] = 0.f; g[i][e] = 0.f; }
      }
    }
    dot = row_sum<TPR>(dot, red) / (float)D;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int col = (i * TPR + tid) * 8;
      if (active && col < D) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rstd * (g[i][e] - xh[i][e] * dot);
        *reinterpret_cast<bf16x8*>(dx + row * D + col) = pack8(o);
      }
    }
  }
  if (partial) {
    float* prow = partial + ((long)blockIdx.x * rows_per_block + r_in_block) * D;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int col = (i * TPR + tid) * 8;
      if (col < D) {
        *reinterpret_cast<float4*>(prow + col) = make_float4(ds[i][0], ds[i][1], ds[i][2], ds[i][3]);
        *reinterpret_cast<float4*>(prow + col + 4) = make_float4(ds[i][4], ds[i][5], ds[i][6], ds[i][7]);
      }
    }
  }
}

// dscale[c] += sum over partial rows (fixed order); four independent accumulators keep the loads in flight
__global__ void rms_dscale_reduce_kernel(const float* __restrict__ partial, int nrows, int D, float* __restrict__ dscale) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  int r = 0;
  for (; r + 3 < nrows; r += 4) {
    a0 += partial[(long)r * D + c];
    a1 += partial[(long)(r + 1) * D + c];
    a2 += partial[(long)(r + 2) * D + c];
    a3 += partial[(long)(r + 3) * D + c];
  }
  for (; r < nrows; ++r) a0 += partial[(long)r * D + c];
  dscale[c] += (a0 + a1) + (a2 + a3);
}

// ------------------------------------------------------------------------------------------------ rotary embedding
// In-place rotation of the first n_rot heads of x [tokens, heads, dh]; one block per token, thread per
// rotated pair (sin/cos evaluated once per pair and reused across heads).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos, const float* __restrict__ inv_ts,
                            int heads, int dh, int n_rot, int rot_dim, int interleaved, int inverse) {
  const long tok = blockIdx.x;
  const int half = rot_dim / 2;
  const float p = (float)pos[tok];
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float s, c;
    sincosf(p * inv_ts[j], &s, &c);
    if (inverse) s = -s;
    const int i0 = interleaved ? 2 * j : j;
    const int i1 = interleaved ? 2 * j + 1 : j + half;
    __nv_bfloat16* base = x + tok * (long)heads * dh;
    for (int h = 0; h < n_rot; ++h) {
      const float a = __bfloat162float(base[h * dh + i0]);
      const float b = __bfloat162float(base[h * dh + i1]);
      base[h * dh + i0] = __float2bfloat16_rn(a * c - b * s);
      base[h * dh + i1] = __float2bfloat16_rn(b * c + a * s);
    }
  }
}

// ------------------------------------------------------------------------------------------------ gated activation
__device__ __forceinline__ float act_apply(float g, int code) {
  switch (code) {
    case 0: return g / (1.f + __expf(-g));                                                         // silu
    case 1: { const float k = 0.7978845608028654f; return 0.5f * g * (1.f + tanhf(k * (g + 0.044715f * g * g * g))); }  // gelu (tanh)
    case 2: return g > 0.f ? g : 0.f;                                                              // relu
    default: return g;                                                                             // linear
  }
}
__device__ __forceinline__ float act_grad(float g, int code) {
  switch (code) {
    case 0: { const float s = 1.f / (1.f + __expf(-g)); return s * (1.f + g * (1.f - s)); }
    case 1: {
      const float k = 0.7978845608028654f;
      const float u = k * (g + 0.044715f * g * g * g);
      const float t = tanhf(u);
      return 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * g * g);
    }
    case 2: return g > 0.f ? 1.f : 0.f;
    default: return 1.f;
  }
}

// gu [rows, 2F] = [gate | up] -> out [rows, F]
__global__ void gated_act_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long rows, int F, int code) {
  const long vec_per_row = F / 8;
  const long total = rows * vec_per_row;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / vec_per_row;
    const int c = (int)(i % vec_per_row) * 8;
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const bf16x8*>(gu + r * 2 * F + c), g);
    unpack8(*reinterpret_cast<const bf16x8*>(gu + r * 2 * F + F + c), u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = act_apply(g[e], code) * u[e];
    *reinterpret_cast<bf16x8*>(out + r * F + c) = pack8(o);
  }
}

__global__ void gated_act_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ gu,
                                     __nv_bfloat16* __restrict__ dgu, long rows, int F, int code) {
  const long vec_per_row = F / 8;
  const long total = rows * vec_per_row;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / vec_per_row;
    const int c = (int)(i % vec_per_row) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const bf16x8*>(gu + r * 2 * F + c), g);
    unpack8(*reinterpret_cast<const bf16x8*>(gu + r * 2 * F + F + c), u);
    unpack8(*reinterpret_cast<const bf16x8*>(dy + r * F + c), d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      dg[e] = d[e] * u[e] * act_grad(g[e], code);
      du[e] = d[e] * act_apply(g[e], code);
    }
    *reinterpret_cast<bf16x8*>(dgu + r * 2 * F + c) = pack8(dg);
    *reinterpret_cast<bf16x8*>(dgu + r * 2 * F + F + c) = pack8(du);
  }
}

// ------------------------------------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const int* __restrict__ tok, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, int D, int V) {
  const long t = blockIdx.x;
  int id = tok[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const uint4* src = reinterpret_cast<const uint4*>(table + (long)id * D);
  uint4* dst = reinterpret_cast<uint4*>(out + t * D);
  for (int i = threadIdx.x; i < D / 8; i += blockDim.x) dst[i] = src[i];
}

__global__ void embedding_bwd_kernel(const int* __restrict__ tok, const __nv_bfloat16* __restrict__ dy, float* __restrict__ dtable,
                                     int D, int V) {
  const long t = blockIdx.x;
  int id = tok[t];
  if (id < 0 || id >= V) return;
  for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(dtable + (long)id * D + i, __bfloat162float(dy[t * D + i]));
}

}  // namespace mt

// ================================================================================================ launchers
using namespace mt;

template <int TPR>
static void launch_rms_fwd(const void* x, const void* scale, float eps, float offset, void* y, float* rstd, int rows, int D,
                           cudaStream_t st) {
  const int vpt = (D / 8 + TPR - 1) / TPR;
  const int threads = 256;
  const int rpb = threads / TPR;
  const int grid = (rows + rpb - 1) / rpb;
#define L(V) rmsnorm_fwd_kernel<TPR, V><<<grid, threads, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)scale, eps, offset, \
                                                                  (__nv_bfloat16*)y, rstd, rows, D)
  if (vpt <= 1) L(1); else if (vpt <= 2) L(2); else if (vpt <= 4) L(4); else L(8);
#undef L
}

extern "C" int mt_rmsnorm_fwd(const void* x, const void* scale, float eps, float offset, void* y, float* rstd, int rows, int D,
                              cudaStream_t st) {
  if (D % 8 || D > 8 * 256 * 8) return -1;
  if (D <= 512) launch_rms_fwd<32>(x, scale, eps, offset, y, rstd, rows, D, st);
  else launch_rms_fwd<256>(x, scale, eps, offset, y, rstd, rows, D, st);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

static int rms_bwd_grid(int rows, int tpr, int sms) {
  const int rpb = 256 / tpr;
  long groups = ((long)rows + rpb - 1) / rpb;
  int grid = (int)(groups < (long)sms * 4 ? groups : (long)sms * 4);
  return grid < 1 ? 1 : grid;
}

template <int TPR>
static void launch_rms_bwd(const void* dy, const void* x, const void* scale, const float* rstd, float offset, void* dx, float* dscale,
                           float* partial, int rows, int D, int sms, cudaStream_t st) {
  const int vpt = (D / 8 + TPR - 1) / TPR;
  const int threads = 256;
  const int grid = rms_bwd_grid(rows, TPR, sms);
  float* part = dscale ? partial : nullptr;
#define L(V) rmsnorm_bwd_kernel<TPR, V><<<grid, threads, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,                 \
                                                                  (const __nv_bfloat16*)scale, rstd, offset, (__nv_bfloat16*)dx,    \
                                                                  part, rows, D)
  if (vpt <= 1) L(1); else if (vpt <= 2) L(2); else if (vpt <= 4) L(4); else L(8);
#undef L
  if (part) rms_dscale_reduce_kernel<<<(D + 127) / 128, 128, 0, st>>>(part, grid * (threads / TPR), D, dscale);
}

// number of fp32 rows of length D that `partial` must hold for mt_rmsnorm_bwd with a scale gradient
extern "C" int mt_rmsnorm_bwd_partial_rows(int rows, int D, int sms) {
  const int tpr = D <= 512 ? 32 : 256;
  return rms_bwd_grid(rows, tpr, sms) * (256 / tpr);
}

// `partial`: scratch of mt_rmsnorm_bwd_partial_rows(rows, D, sms) x D floats (needed only when dscale is given); rows of a
// block that saw no input row are written as zeros by the kernel, so the scratch needs no clearing.
extern "C" int mt_rmsnorm_bwd(const void* dy, const void* x, const void* scale, const float* rstd, float offset, void* dx,
                              float* dscale, float* partial, int rows, int D, int sms, cudaStream_t st) {
  if (D % 8 || D > 8 * 256 * 8 || (dscale && !partial)) return -1;
  if (D <= 512) launch_rms_bwd<32>(dy, x, scale, rstd, offset, dx, dscale, partial, rows, D, sms, st);
  else launch_rms_bwd<256>(dy, x, scale, rstd, offset, dx, dscale, partial, rows, D, sms, st);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int mt_rope(void* x, const int* pos, const float* inv_ts, long tokens, int heads, int dh, int n_rot, int rot_dim,
                       int interleaved, int inverse, cudaStream_t st) {
  if (tokens <= 0) return 0;
  int threads = rot_dim / 2;
  threads = threads < 32 ? 32 : (threads > 256 ? 256 : threads);
  rope_kernel<<<(unsigned)tokens, threads, 0, st>>>((__nv_bfloat16*)x, pos, inv_ts, heads, dh, n_rot, rot_dim, interleaved, inverse);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int mt_gated_act_fwd(const void* gu, void* out, long rows, int F, int code, int sms, cudaStream_t st) {
  if (F % 8) return -1;
  long total = rows * (F / 8);
  long blocks = (total + 255) / 256;
  int grid = (int)(blocks < (long)sms * 16 ? blocks : (long)sms * 16);
  if (grid < 1) return 0;
  gated_act_fwd_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, F, code);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int mt_gated_act_bwd(const void* dy, const void* gu, void* dgu, long rows, int F, int code, int sms, cudaStream_t st) {
  if (F % 8) return -1;
  long total = rows * (F / 8);
  long blocks = (total + 255) / 256;
  int grid = (int)(blocks < (long)sms * 16 ? blocks : (long)sms * 16);
  if (grid < 1) return 0;
  gated_act_bwd_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, rows, F, code);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int mt_embedding_fwd(const int* tok, const void* table, void* out, long tokens, int D, int V, cudaStream_t st) {
  if (D % 8) return -1;
  if (tokens <= 0) return 0;
  embedding_fwd_kernel<<<(unsigned)tokens, 128, 0, st>>>(tok, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, D, V);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int mt_embedding_bwd(const int* tok, const void* dy, float* dtable, long tokens, int D, int V, cudaStream_t st) {
  if (tokens <= 0) return 0;
  embedding_bwd_kernel<<<(unsigned)tokens, 256, 0, st>>>(tok, (const __nv_bfloat16*)dy, dtable, D, V);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
