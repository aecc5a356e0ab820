// Autoregressive decode attention over a slot-indexed KV cache: one new query token per sequence attends to everything
// cached for its slot. Memory-bound by design (every cached key and value is read once), so the kernel is organised around
// coalesced 16-byte loads of K/V tiles into shared memory and fp32 math on the CUDA cores; the KV range of each sequence is
// split over several CTAs (flash-decoding) so that small batches still fill 148 SMs, and a second kernel merges the partial
// (max, sum, output) triples. Lengths and slot ids are read from device memory: nothing here synchronises with the host,
// which lets a whole decode step be captured in a CUDA graph.
// The reference uses a Pallas ragged-attention kernel on TPU and a Triton kernel with a k_end mask on GPU
// (src/maxtext/kernels/ragged_attention.py; src/maxtext/layers/attention_op.py:1528-1587).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mt {

constexpr int DEC_THREADS = 128;
constexpr int DEC_TILE = 64;      // keys per shared-memory tile
constexpr int DEC_MAX_G = 16;     // query heads per kv head

// q [B, Hq, D]; k_cache / v_cache [slots, max_len, Hkv, D]; lengths[b] = tokens cached for row b INCLUDING the new one.
// part [B, Hkv, splits, G, D + 2] fp32: (acc[D], m, l) per query head of the group.
template <int D>
__global__ void __launch_bounds__(DEC_THREADS)
decode_attn_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                   const int* __restrict__ slot_ids, const int* __restrict__ lengths, int max_len, int Hq, int Hkv, int window, float scale,
                   float soft_cap, int splits, float* __restrict__ part) {
  constexpr int PAD = 8;                                   // bf16 elements of row padding: rows start in different banks
  __shared__ __align__(16) __nv_bfloat16 ks[DEC_TILE][D + PAD];
  __shared__ __align__(16) __nv_bfloat16 vs[DEC_TILE][D + PAD];
  __shared__ float qs[DEC_MAX_G][D];
  __shared__ float ps[DEC_MAX_G][DEC_TILE];
  __shared__ float red[DEC_MAX_G][2];
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int G = Hq / Hkv;
  const int tid = threadIdx.x;
  const int len = lengths[b];
  const int first = (window > 0 && len > window) ? len - window : 0;
  const int span = len - first;
  const int per = (span + splits - 1) / splits;
  const int lo = first + split * per;
  const int hi = min(len, lo + per);
  float* out = part + (((long)b * Hkv + h) * splits + split) * G * (D + 2);
  for (int i = tid; i < G * D; i += DEC_THREADS) qs[i / D][i % D] = __bfloat162float(q[((long)b * Hq + h * G + i / D) * D + i % D]) * scale;
  float acc[DEC_MAX_G];
  float m_run[DEC_MAX_G], l_run[DEC_MAX_G];
#pragma unroll
  for (int g = 0; g < DEC_MAX_G; ++g) { acc[g] = 0.f; m_run[g] = -1e30f; l_run[g] = 0.f; }
  const long slot = slot_ids[b];
  const long row_stride = (long)Hkv * D;
  const __nv_bfloat16* kb = k_cache + (slot * max_len) * row_stride + (long)h * D;
  const __nv_bfloat16* vb = v_cache + (slot * max_len) * row_stride + (long)h * D;
  constexpr int VEC_PER_ROW = D / 8;
  __syncthreads();
  for (int t0 = lo; t0 < hi; t0 += DEC_TILE) {
    const int n = min(DEC_TILE, hi - t0);
    for (int i = tid; i < n * VEC_PER_ROW; i += DEC_THREADS) {
      const int r = i / VEC_PER_ROW, c = (i % VEC_PER_ROW) * 8;
      *reinterpret_cast<uint4*>(&ks[r][c]) = *reinterpret_cast<const uint4*>(kb + (long)(t0 + r) * row_stride + c);
      *reinterpret_cast<uint4*>(&vs[r][c]) = *reinterpret_cast<const uint4*>(vb + (long)(t0 + r) * row_stride + c);
    }
    __syncthreads();
    // scores: (key j, head g) pairs spread over the threads
    for (int i = tid; i < n * G; i += DEC_THREADS) {
      const int j = i % n, g = i / n;
      float s = 0.f;
#pragma unroll 8
      for (int d = 0; d < D; d += 2) {
        const float2 kv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ks[j][d]));
        s += qs[g][d] * kv.x + qs[g][d + 1] * kv.y;
      }
      if (soft_cap > 0.f) s = tanhf(s / soft_cap) * soft_cap;
      ps[g][j] = s;
    }
    __syncthreads();
    // per head: tile max and the rescale of the running state (one warp per head, round robin)
    const int warp = tid >> 5, lane = tid & 31;
    for (int g = warp; g < G; g += DEC_THREADS / 32) {
      float mx = -1e30f;
      for (int j = lane; j < n; j += 32) mx = fmaxf(mx, ps[g][j]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float sum = 0.f;
      for (int j = lane; j < n; j += 32) {
        const float p = __expf(ps[g][j] - mx);
        ps[g][j] = p;
        sum += p;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane == 0) { red[g][0] = mx; red[g][1] = sum; }
    }
    __syncthreads();
    // output: thread d accumulates column d for every head of the group
    if (tid < D) {
#pragma unroll
      for (int g = 0; g < DEC_MAX_G; ++g) {
        if (g < G) {
          const float mt = red[g][0];
          const float m_new = fmaxf(m_run[g], mt);
          const float a = __expf(m_run[g] - m_new), bscale = __expf(mt - m_new);
          float o = 0.f;
          for (int j = 0; j < n; ++j) o += ps[g][j] * __bfloat162float(vs[j][tid]);
          acc[g] = acc[g] * a + o * bscale;
          l_run[g] = l_run[g] * a + red[g][1] * bscale;
          m_run[g] = m_new;
        }
      }
    }
    __syncthreads();
  }
  if (tid < D) {
#pragma unroll
    for (int g = 0; g < DEC_MAX_G; ++g) {
      if (g < G) {
        out[g * (D + 2) + tid] = acc[g];
        if (tid == 0) { out[g * (D + 2) + D] = m_run[g]; out[g * (D + 2) + D + 1] = l_run[g]; }
      }
    }
  }
}

// out [B, Hq, D] bf16 = merge of the `splits` partials.
template <int D>
__global__ void __launch_bounds__(D)
decode_merge_kernel(const float* __restrict__ part, int Hq, int Hkv, int splits, __nv_bfloat16* __restrict__ out) {
  const int hq = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int G = Hq / Hkv, h = hq / G, g = hq % G;
  const float* base = part + (((long)b * Hkv + h) * splits) * G * (D + 2) + (long)g * (D + 2);
  const long stride = (long)G * (D + 2);
  float m = -1e30f;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, base[s * stride + D]);
  float num = 0.f, den = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float w = __expf(base[s * stride + D] - m);
    num += base[s * stride + d] * w;
    den += base[s * stride + D + 1] * w;
  }
  out[((long)b * Hq + hq) * D + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
}

}  // namespace mt

using namespace mt;

extern "C" int mt_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int* slot_ids, const int* lengths, int B,
                                   int max_len, int Hq, int Hkv, int D, int window, float scale, float soft_cap, int splits, float* part,
                                   void* out, cudaStream_t st) {
  if (Hq % Hkv || Hq / Hkv > DEC_MAX_G || (D != 128 && D != 64) || splits < 1) return -1;
  const dim3 grid(splits, Hkv, B);
  const __nv_bfloat16 *qp = reinterpret_cast<const __nv_bfloat16*>(q), *kp = reinterpret_cast<const __nv_bfloat16*>(k_cache),
                      *vp = reinterpret_cast<const __nv_bfloat16*>(v_cache);
  __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(out);
  if (D == 128) {
    decode_attn_kernel<128><<<grid, DEC_THREADS, 0, st>>>(qp, kp, vp, slot_ids, lengths, max_len, Hq, Hkv, window, scale, soft_cap, splits, part);
    decode_merge_kernel<128><<<dim3(Hq, B), 128, 0, st>>>(part, Hq, Hkv, splits, op);
  } else {
    decode_attn_kernel<64><<<grid, DEC_THREADS, 0, st>>>(qp, kp, vp, slot_ids, lengths, max_len, Hq, Hkv, window, scale, soft_cap, splits, part);
    decode_merge_kernel<64><<<dim3(Hq, B), 64, 0, st>>>(part, Hq, Hkv, splits, op);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
