// Block-scaled FP8 (E4M3) products for sm_100a: activations carry one fp32 scale per 1 x 128 block of the contraction
// dimension, weights one per 128 x 128 block, products accumulate in fp32.
//
//   C[m, n] = sum_kb  sa[kb, m] * sb[n / 128, kb] * sum_{k in block kb} Aq[m, k] * Bq[n, k]
//
// The tensor core (tcgen05 kind::f8f6f4) forms the inner sum of one 128-wide K block in tensor memory; sixteen epilogue warps
// read that partial product, multiply it by the two scales of the block and add it to fp32 accumulators that live in their
// registers for the whole K loop (a thread owns 32 columns of one row of the 128 x 128 output tile; four warps per scheduler hide
// the latency of the tensor-memory loads). Four TMEM buffers rotate, so
// the tensor core runs up to three K blocks ahead of the promotion. The same kernel serves mixture-of-experts layers: rows
// grouped by expert and padded to 128 per group, one weight matrix (and one scale table) per expert.
//
// Measured limit of this tile shape: with 8-bit operands a 128 x 128 x 128 block moves 32 KB into shared memory and the tensor
// core reads 32 KB back out of it, 64 KB per 4.2 MFLOP, which at 128 B per clock is about 512 clocks: the kernel runs at that
// rate (1.25-1.4 PFLOP/s) with or without the promotion work. A 256-wide tile (or a CTA pair that shares B) halves the bytes
// per FLOP; it needs 64 accumulators per thread at 512 epilogue threads.
//
// The two quantisation kernels that produce the operands are here as well: 1 x 128 for activations / gradients (scales stored
// [K blocks, rows] so that an epilogue warp reads them coalesced) and 128 x 128 for weights (optionally also the transposed
// 8-bit copy, which is the operand of the input-gradient product).
#include "sm100_ptx.cuh"
#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace mt {
namespace f8b {

constexpr int BM = 128, BN = 128, BKB = 128;       // tile; BKB = bytes = elements of one K block
constexpr int STAGES = 5;
constexpr int A_BYTES = BM * BKB, B_BYTES = BN * BKB, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_BYTES = 2 * BM * 128;            // two 64-column bf16 staging buffers
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 256 + 1024;
constexpr int THREADS = 576;                       // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2..17: promotion / epilogue
constexpr int EPI_THREADS = 512;
constexpr int NACC = 4;
constexpr uint32_t TMEM_COLS = NACC * BN;

struct Params {
  int M, N, K;
  const float* sa;         // [KB, M] activation scales (de-quantisation factors)
  const float* sb;         // weight scales, element (e, nb, kb) at e * sb_e + nb * sb_n + kb * sb_k
  long sb_e, sb_n, sb_k;
  // grouped mode (experts != 0): x_offs[e] = first padded row of expert e, x_offs[experts] = rows in use; blk_expert[mb] = expert
  // of row block mb; the weights of expert e are rows [e * N, (e + 1) * N) of the B tensor
  int experts;
  const int* x_offs;
  const int* blk_expert;
  int* status;
};

template <int DUMMY = 0>
__global__ void __launch_bounds__(THREADS, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
            const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA = base, sB = base + STAGES * A_BYTES, sEpi = base + STAGES * STAGE_BYTES, bars = sEpi + EPI_BYTES;
  auto full = [&](int s) { return bars + 8u * s; };
  auto empty = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto tempty = [&](int a) { return bars + 8u * (2 * STAGES + NACC + a); };
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + (bars - base) + 8 * (2 * STAGES + 2 * NACC));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_blocks = p.experts ? p.x_offs[p.experts] / BM : (p.M + BM - 1) / BM;
  const int n_blocks = (p.N + BN - 1) / BN;
  const int num_kb = (p.K + BKB - 1) / BKB;
  const int num_tiles = m_blocks * n_blocks;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
    for (int a = 0; a < NACC; ++a) { mbar_init(tfull(a), 1); mbar_init(tempty(a), EPI_THREADS); }
    fence_barrier_init();
    prefetch_tensormap(&map_a); prefetch_tensormap(&map_b); prefetch_tensormap(&map_c);
  }
  if (warp == 1) { tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // tiles are walked n-fastest inside groups of 8 row blocks: concurrently running CTAs share the A rows and sweep B
  auto coords = [&](int t, int& mb, int& nb) {
    const int per_group = 8 * n_blocks, g = t / per_group, first = g * 8;
    const int gsz = min(8, m_blocks - first), r = t - g * per_group;
    mb = first + r % gsz;
    nb = r / gsz;
  };

  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mb, nb;
        coords(t, mb, nb);
        const int e = p.experts ? p.blk_expert[mb] : 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty(s), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
          mbar_arrive_expect_tx(full(s), STAGE_BYTES);
          tma_load_2d(sA + s * A_BYTES, &map_a, full(s), kb * BKB, mb * BM);
          tma_load_3d(sB + s * B_BYTES, &map_b, full(s), kb * BKB, nb * BN, e);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_fp8(BM, BN, 0, 0);
      int s = 0, acc = 0;
      uint32_t ph = 0, aph = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(tempty(acc), aph ^ 1, abort_flag, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
          if (!mbar_wait(full(s), ph, abort_flag, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint64_t da = make_smem_desc(sA + s * A_BYTES, 16, 1024), db = make_smem_desc(sB + s * B_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f8_ss(tmem + acc * BN, da + (uint64_t)((k * 32) >> 4), db + (uint64_t)((k * 32) >> 4), idesc, k != 0);
          umma_commit(empty(s));
          umma_commit(tfull(acc));
          if (++s == STAGES) { s = 0; ph ^= 1; }
          if (++acc == NACC) { acc = 0; aph ^= 1; }
        }
      }
    }
  } else {
    // A thread owns columns [cg * 32, cg * 32 + 32) of row `row` of the tile. Every thread waits on the barriers itself; one
    // that gave up (ok = false) keeps meeting the others at the named barriers of the output stage but touches no tensor memory.
    const int q = warp & 3, cg = (warp - 2) >> 2, row = q * 32 + lane, et = threadIdx.x - 64;
    int acc = 0;
    uint32_t aph = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int mb, nb;
      coords(t, mb, nb);
      const int e = p.experts ? p.blk_expert[mb] : 0;
      const long m = (long)mb * BM + row;
      const bool row_ok = m < p.M;
      const float* sap = p.sa + (row_ok ? m : 0);
      const float* sbp = p.sb + e * p.sb_e + nb * p.sb_n;
      float c[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) c[j] = 0.f;
      float s_next = row_ok ? sap[0] * sbp[0] : 0.f;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const float sc = s_next;
        if (kb + 1 < num_kb) s_next = row_ok ? sap[(long)(kb + 1) * p.M] * sbp[(long)(kb + 1) * p.sb_k] : 0.f;   // in flight during the wait
        if (!mbar_wait(tfull(acc), aph, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
        tc_fence_after();
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem + acc * BN + cg * 32 + ((uint32_t)(q * 32) << 16), r);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(tempty(acc));                       // the values are in registers: the tensor core may reuse the buffer
#pragma unroll
        for (int j = 0; j < 32; ++j) c[j] = fmaf(__uint_as_float(r[j]), sc, c[j]);
        if (++acc == NACC) { acc = 0; aph ^= 1; }
      }
      // bf16 output: two 64-column staging boxes, each filled by two column groups; one thread stores both (rows beyond M are
      // clipped by the map)
      if (et == 0) tma_wait_group_read<0>();
      named_bar_sync(1, EPI_THREADS);
      const uint32_t sbuf = sEpi + (cg >> 1) * (BM * 128);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t pk[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) pk[x] = pack_bf16(c[8 * j + 2 * x], c[8 * j + 2 * x + 1]);
        const uint32_t dst = sbuf + row * 128 + ((((cg & 1) * 4 + j) ^ (row & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]) : "memory");
      }
      if (!ok) *abort_flag = 1;
      fence_proxy_async_smem();
      named_bar_sync(2, EPI_THREADS);
      if (et == 0 && *abort_flag == 0) {
#pragma unroll
        for (int h = 0; h < BN / 64; ++h)
          if (nb * BN + h * 64 < p.N) tma_store_2d(&map_c, sEpi + h * (BM * 128), nb * BN + h * 64, mb * BM);
        tma_commit_group();
      }
    }
    if (et == 0) tma_wait_group<0>();
  }
  if (*abort_flag) { const uint64_t t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 200000ull) { } }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// ---------------------------------------------------------------------------------------------- quantisation
__device__ __forceinline__ uint8_t e4m3(float v) { return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3); }

// x [R, C] bf16 (row stride ldx elements) -> q [R, C] e4m3 and scales_t [ceil(C/128), R]: one warp per (row, 128-column block)
__global__ void __launch_bounds__(256) quant_rows_kernel(const __nv_bfloat16* __restrict__ x, long R, int C, long ldx, uint8_t* __restrict__ q,
                                                         float* __restrict__ scales_t) {
  const int kbs = (C + 127) / 128;
  const long w = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= R * kbs) return;
  const long r = w / kbs;
  const int kb = (int)(w % kbs);
  const int c0 = kb * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (c0 + 3 < C) {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + r * ldx + c0);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else {
    for (int j = 0; j < 4; ++j)
      if (c0 + j < C) v[j] = __bfloat162float(x[r * ldx + c0 + j]);
  }
  float am = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
  const float inv = am > 0.f ? 448.f / am : 1.f;
  if (lane == 0) scales_t[(long)kb * R + r] = am > 0.f ? am / 448.f : 1.f;
  if (c0 + 3 < C) {
    const uint32_t pk = e4m3(v[0] * inv) | (e4m3(v[1] * inv) << 8) | (e4m3(v[2] * inv) << 16) | ((uint32_t)e4m3(v[3] * inv) << 24);
    *reinterpret_cast<uint32_t*>(q + r * C + c0) = pk;
  } else {
    for (int j = 0; j < 4; ++j)
      if (c0 + j < C) q[r * C + c0 + j] = e4m3(v[j] * inv);
  }
}

// w [G, R, C] bf16 -> q [G, R, C] (and qt [G, C, R]) e4m3 and scales [G, ceil(R/128), ceil(C/128)]: one CTA per 128 x 128 block
__global__ void __launch_bounds__(256) quant_blocks_kernel(const __nv_bfloat16* __restrict__ w, int R, int C, uint8_t* __restrict__ q,
                                                           uint8_t* __restrict__ qt, float* __restrict__ scales) {
  __shared__ float red[8];
  __shared__ float s_inv;
  __shared__ uint8_t tile[128][132];
  const int cb = blockIdx.x, rb = blockIdx.y, g = blockIdx.z;
  const int nrb = (R + 127) / 128, ncb = (C + 127) / 128;
  const __nv_bfloat16* src = w + (long)g * R * C;
  float am = 0.f;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = rb * 128 + i / 128, c = cb * 128 + i % 128;
    if (r < R && c < C) am = fmaxf(am, fabsf(__bfloat162float(src[(long)r * C + c])));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = am;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int j = 1; j < 8; ++j) am = fmaxf(am, red[j]);
    scales[((long)g * nrb + rb) * ncb + cb] = am > 0.f ? am / 448.f : 1.f;
    s_inv = am > 0.f ? 448.f / am : 1.f;
  }
  __syncthreads();
  const float inv = s_inv;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int lr = i / 128, lc = i % 128, r = rb * 128 + lr, c = cb * 128 + lc;
    uint8_t v = 0;
    if (r < R && c < C) {
      v = e4m3(__bfloat162float(src[(long)r * C + c]) * inv);
      if (q) q[((long)g * R + r) * C + c] = v;
    }
    tile[lr][lc] = v;
  }
  if (qt) {
    __syncthreads();
    for (int i = threadIdx.x; i < 128 * 128; i += 256) {
      const int lc = i / 128, lr = i % 128, r = rb * 128 + lr, c = cb * 128 + lc;      // consecutive threads walk r: coalesced in qt
      if (r < R && c < C) qt[((long)g * C + c) * R + r] = tile[lr][lc];
    }
  }
}

// ---------------------------------------------------------------------------------------------- host
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                             const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || !ptr) return nullptr;
    fn = reinterpret_cast<EncodeFn>(ptr);
  }
  return fn;
}

static int make_map(CUtensorMap* m, CUtensorMapDataType dt, int esize, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                    const cuuint32_t* box) {
  EncodeFn enc = encode_fn();
  if (!enc) return -1;
  cuuint32_t es[3] = {1, 1, 1};
  (void)esize;
  CUresult r = enc(m, dt, rank, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

}  // namespace f8b
}  // namespace mt

extern "C" {

// x [R, C] bf16 (C a multiple of 4) -> q [R, C] e4m3, scales_t [ceil(C / 128), R] fp32
int mt_quant_fp8_rows(const void* x, long R, int C, long ldx, void* q, float* scales_t, cudaStream_t st) {
  if (C % 4 || ldx % 4 || R < 0) return -1;
  const long warps = R * ((C + 127) / 128);
  if (warps == 0) return 0;
  mt::f8b::quant_rows_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>((const __nv_bfloat16*)x, R, C, ldx, (uint8_t*)q, scales_t);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// w [G, R, C] bf16 -> q [G, R, C] and / or qt [G, C, R] e4m3, scales [G, ceil(R / 128), ceil(C / 128)] fp32
int mt_quant_fp8_blocks(const void* w, int G, int R, int C, void* q, void* qt, float* scales, cudaStream_t st) {
  if (G < 1 || R < 1 || C < 1) return -1;
  mt::f8b::quant_blocks_kernel<<<dim3((C + 127) / 128, (R + 127) / 128, G), 256, 0, st>>>((const __nv_bfloat16*)w, R, C, (uint8_t*)q, (uint8_t*)qt,
                                                                                          scales);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// C[M, N] bf16 = block-scaled product of aq [M, K] (row stride lda bytes) and bq [experts or 1, N, K] e4m3.
//   sa: [ceil(K/128), M] fp32; sb: element (e, nb, kb) at e * sb_e + nb * sb_n + kb * sb_k (so a transposed table can be passed)
//   grouped: experts > 0 with x_offs [experts + 1] and blk_expert [M / 128] on the device (M = padded row capacity, multiple of 128)
// K and the strides must be multiples of 16 bytes.
int mt_gemm_fp8_block(const void* aq, const void* bq, void* c, int M, int N, int K, long lda, long ldb, long ldc, const float* sa, const float* sb,
                      long sb_e, long sb_n, long sb_k, int experts, const int* x_offs, const int* blk_expert, int* status, int num_sms,
                      cudaStream_t st) {
  using namespace mt::f8b;
  if (M < 1 || N < 1 || K < 1 || K % 16 || lda % 16 || ldb % 16 || ldc % 8 || (experts && M % BM)) return -1;
  CUtensorMap ma, mb, mc;
  {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)lda};
    cuuint32_t box[2] = {BKB, BM};
    if (make_map(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, aq, 2, dims, strides, box)) return -3;
  }
  {
    const int G = experts ? experts : 1;
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)N, (cuuint64_t)G};
    cuuint64_t strides[2] = {(cuuint64_t)ldb, (cuuint64_t)ldb * N};
    cuuint32_t box[3] = {BKB, BN, 1};
    if (make_map(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, bq, 3, dims, strides, box)) return -3;
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)ldc * 2};
    cuuint32_t box[2] = {64, BM};
    if (make_map(&mc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, c, 2, dims, strides, box)) return -3;
  }
  Params p{};
  p.M = M; p.N = N; p.K = K; p.sa = sa; p.sb = sb; p.sb_e = sb_e; p.sb_n = sb_n; p.sb_k = sb_k;
  p.experts = experts; p.x_offs = x_offs; p.blk_expert = blk_expert; p.status = status;
  static bool cfg = false;
  if (!cfg) {
    if (cudaFuncSetAttribute(gemm_fp8_block_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -2;
    cfg = true;
  }
  const int tiles = (M / BM + (M % BM != 0)) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  gemm_fp8_block_kernel<0><<<grid, THREADS, SMEM_BYTES, st>>>(ma, mb, mc, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // extern "C"
