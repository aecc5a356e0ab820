// Flash attention backward for sm_100a: deterministic (no atomics), two software-pipelined kernels.
//
//   delta = rowsum(dO * O)                                  (small pre-pass)
//   kernel A, CTA = 128 keys of one kv head, K and V resident in shared memory. It walks the query heads
//     of its GQA group and the 128-query tiles at or after its keys (Q / dO tiles double buffered):
//        S^T = K Q^T, dP^T = V dO^T  (128 x 128 fp32 in TMEM)
//        P^T = exp(S^T - lse), dS^T = scale * P^T * (dP^T - delta)  -> bf16, written back into TMEM
//        dV += P^T dO, dK += dS^T Q  (TMEM operands, accumulators stay in TMEM until the end)
//     The MMA warp interleaves the next tile's S^T / dP^T between dV and dK, so the 256 softmax threads and the
//     tensor core work at the same time.
//   kernel B, CTA = 128 queries of one head, Q and dO resident, K / V tiles double buffered:
//        S = Q K^T, dP = dO V^T, dS = scale * P * (dP - delta) -> TMEM, dQ += dS K.
// P is recomputed from the saved log-sum-exp in both kernels. Masks follow the forward kernel (causal by
// token index, sliding window, segment ids). All waits are bounded; a timeout sets the status word.
#include "sm100_ptx.cuh"
#include <cuda_bf16.h>

namespace mt {
namespace bwd {

constexpr int THREADS = 320;        // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2..9: softmax / epilogue
constexpr int SM_THREADS = 256;
constexpr float LOG2E = 1.4426950408889634f;

struct Params {
  int B, S, Hq, Hkv, D;
  int window;
  float scale;
  const int* seg;
  const float* lse;
  const float* delta;
  int* status;
};

__device__ __forceinline__ bool valid(int qg, int kg, int window, bool has_seg, int sq, int sk) {
  bool v = kg <= qg;
  if (window > 0) v = v && (qg - kg < window);
  if (has_seg) v = v && (sq == sk) && (sk != 0);
  return v;
}

// [128 x D] tile held as D/64 boxes {64 cols, 128 rows} (16 KB each)
__device__ __forceinline__ uint64_t big_kmajor(uint32_t tile, int k) { return make_smem_desc(tile + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024); }
// the same tile read with its 128 rows as the contraction index and d as N (MN-major): 16 rows = 2048 B per k-step
__device__ __forceinline__ uint64_t big_mnmajor(uint32_t tile, int k) { return make_smem_desc(tile + k * 2048, 16384, 1024); }
// TMEM column of k-step k of a bf16 operand whose two 64-row halves start 64 columns apart (32 packed columns each)
__device__ __forceinline__ uint32_t tmem_a_col(int k) { return (uint32_t)((k >> 2) * 64 + (k & 3) * 8); }

struct alignas(8) Ctl {
  uint64_t bars[16];
  uint32_t tmem_base;
  int abort_flag;
  int ok_flag;
  int pad;
};

__device__ __forceinline__ void stage_rows_bf16(uint32_t tmem_addr, uint32_t box, int row, int c) {
  // 32 fp32 columns of this thread's row -> 64 bytes of a 128-byte swizzled row in `box`
  uint32_t r[32];
  tmem_ld_32x32b_x32(tmem_addr, r);
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t pk[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) pk[e] = pack_bf16(__uint_as_float(r[8 * j + 2 * e]), __uint_as_float(r[8 * j + 2 * e + 1]));
    const int chunk = (c & 1) * 4 + j;
    const uint32_t dst = box + row * 128 + ((chunk ^ (row & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]) : "memory");
  }
}

// ================================================================================================ delta
__global__ void delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out, float* __restrict__ delta,
                             int B, int S, int H, int D) {
  const long w = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long)B * S * H) return;
  const int h = (int)(w % H);
  const long bs = w / H;
  const int s = (int)(bs % S), b = (int)(bs / S);
  const __nv_bfloat16* a = dout + w * D;
  const __nv_bfloat16* o = out + w * D;
  float acc = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + i));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + i));
    acc += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[((long)b * H + h) * S + s] = acc;
}

// ================================================================================================ kernel A: dK, dV
// Issue order of the MMA warp in steady state:  dV_i | S^T_{i+1} | dK_i | dP^T_{i+1}
// so the tensor core computes S^T of the next tile while the softmax threads turn dP^T_i into dS^T_i, and
// dP^T of the next tile while they turn S^T_{i+1} into P^T_{i+1}.
template <int D>
__global__ void __launch_bounds__(THREADS, 1)
dkv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
           const __grid_constant__ CUtensorMap map_do, const __grid_constant__ CUtensorMap map_dk, const __grid_constant__ CUtensorMap map_dv,
           Params p) {
  constexpr int BIG = 128 * D * 2;
  constexpr int NBOX = D / 64;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_ST = 0, COL_DPT = 128, COL_DV = 256, COL_DK = 384;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sK = base, sV = base + BIG, sStage = base + 2 * BIG;          // stage s: Q at +s*2*BIG, dO right after it
  Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + (base - smem_u32(smem_raw)) + 6 * BIG);
  float* s_lse = reinterpret_cast<float*>(ctl + 1);      // [2][128], pre-multiplied by log2(e)
  float* s_delta = s_lse + 256;                          // [2][128]
  int* s_seg = reinterpret_cast<int*>(s_delta + 256);    // [2][128]
  const uint32_t bar0 = smem_u32(&ctl->bars[0]);
  enum { KV_FULL = 0, Q_FULL0, Q_FULL1, Q_EMPTY0, Q_EMPTY1, ST_FULL, DP_FULL, P_READY, DS_READY, ACC_FULL };
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_t = p.S / 128;
  const int kt = blockIdx.x;
  const int hk = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int k0 = kt * 128;
  const int row_base = b * p.S;
  int qt_hi = n_t - 1;
  if (p.window > 0) { const int hi = (k0 + 127 + p.window - 1) / 128; qt_hi = hi < n_t - 1 ? hi : n_t - 1; }
  const int n_qt = qt_hi - kt + 1;
  const int n_iter = n_qt * G;

  if (threadIdx.x == 0) {
    ctl->abort_flag = 0;
    ctl->ok_flag = 1;
    mbar_init(bar(KV_FULL), 1);
    for (int s = 0; s < 2; ++s) { mbar_init(bar(Q_FULL0 + s), 1); mbar_init(bar(Q_EMPTY0 + s), 1); }
    mbar_init(bar(ST_FULL), 1); mbar_init(bar(DP_FULL), 1);
    mbar_init(bar(P_READY), SM_THREADS); mbar_init(bar(DS_READY), SM_THREADS);
    mbar_init(bar(ACC_FULL), 1);
    fence_barrier_init();
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_k); prefetch_tensormap(&map_v); prefetch_tensormap(&map_do);
  }
  if (warp == 1) { tmem_alloc(smem_u32(&ctl->tmem_base), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(bar(KV_FULL), 2 * BIG);
#pragma unroll
      for (int j = 0; j < NBOX; ++j) {
        tma_load_2d(sK + j * 16384, &map_k, bar(KV_FULL), hk * D + j * 64, row_base + k0);
        tma_load_2d(sV + j * 16384, &map_v, bar(KV_FULL), hk * D + j * 64, row_base + k0);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int h = hk * G + it / n_qt;
        const int q0 = (kt + it % n_qt) * 128;
        if (!mbar_wait(bar(Q_EMPTY0 + s), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_arrive_expect_tx(bar(Q_FULL0 + s), 2 * BIG);
        const uint32_t sq = sStage + s * 2 * BIG, sdo = sq + BIG;
#pragma unroll
        for (int j = 0; j < NBOX; ++j) {
          tma_load_2d(sq + j * 16384, &map_q, bar(Q_FULL0 + s), h * D + j * 64, row_base + q0);
          tma_load_2d(sdo + j * 16384, &map_do, bar(Q_FULL0 + s), h * D + j * 64, row_base + q0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_nt = make_idesc_bf16(128, 128, false, false);   // [128 kv x d] . [128 q x d]^T
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, false, true);     // TMEM [128 kv x 128 q] . [128 q x d]
      auto stage_q = [&](int it) { return sStage + (it & 1) * 2 * BIG; };
      auto issue_st = [&](int it) {
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16_ss(tmem + COL_ST, big_kmajor(sK, k), big_kmajor(stage_q(it), k), idesc_nt, k != 0);
        umma_commit(bar(ST_FULL));
      };
      auto issue_dpt = [&](int it) {
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16_ss(tmem + COL_DPT, big_kmajor(sV, k), big_kmajor(stage_q(it) + BIG, k), idesc_nt, k != 0);
        umma_commit(bar(DP_FULL));
      };
      bool ok = mbar_wait(bar(KV_FULL), 0, abort_flag, p.status, ST_TIMEOUT_MMA);
      if (ok && n_iter > 0) {
        ok = mbar_wait(bar(Q_FULL0), 0, abort_flag, p.status, ST_TIMEOUT_MMA);
        if (ok) { tc_fence_after(); issue_st(0); issue_dpt(0); }
      }
      for (int it = 0; it < n_iter && ok; ++it) {
        const uint32_t ph = it & 1;
        if (!mbar_wait(bar(P_READY), ph, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ts(tmem + COL_DV, tmem + COL_ST + tmem_a_col(k), big_mnmajor(stage_q(it) + BIG, k), idesc_acc, (it | k) != 0);
        if (it + 1 < n_iter) {
          if (!mbar_wait(bar(Q_FULL0 + ((it + 1) & 1)), ((it + 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
          tc_fence_after();
          issue_st(it + 1);        // overwrites P^T_it only after dV_it (issued above) has consumed it: MMAs retire in order
        }
        if (!mbar_wait(bar(DS_READY), ph, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ts(tmem + COL_DK, tmem + COL_DPT + tmem_a_col(k), big_mnmajor(stage_q(it), k), idesc_acc, (it | k) != 0);
        umma_commit(bar(Q_EMPTY0 + (it & 1)));
        if (it + 1 < n_iter) issue_dpt(it + 1);
        else umma_commit(bar(ACC_FULL));
      }
    }
  } else {
    // ---------------------------------------------------------------- 256 softmax threads: (key row, 64-query half)
    const int sw = warp - 2;                    // 0..7
    const int qd = warp & 3;                    // TMEM lane quarter this warp may touch
    const int half = sw >> 2;                   // which 64 of the 128 query columns
    const int row = qd * 32 + lane;             // key row
    const int et = threadIdx.x - 64;            // 0..255
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const float a = p.scale * LOG2E;
    const bool has_seg = p.seg != nullptr;
    const int kg = k0 + row;
    const int my_seg = has_seg ? p.seg[b * p.S + kg] : 0;
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int s = it & 1;
      const uint32_t ph = it & 1;
      const int h = hk * G + it / n_qt;
      const int q0 = (kt + it % n_qt) * 128;
      if (et < 128) {
        const long idx = ((long)b * p.Hq + h) * p.S + q0 + et;
        s_lse[s * 128 + et] = p.lse[idx] * LOG2E;
        s_delta[s * 128 + et] = p.delta[idx];
        if (has_seg) s_seg[s * 128 + et] = p.seg[b * p.S + q0 + et];
      }
      // One thread waits for the MMAs; its verdict is sticky. A failed CTA keeps meeting at the named barriers
      // (so nobody is left waiting there) but does no further tensor-memory work.
      if (et == 128 && !mbar_wait(bar(ST_FULL), ph, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ctl->ok_flag = 0;
      named_bar_sync(1, SM_THREADS);
      if (*reinterpret_cast<volatile int*>(&ctl->ok_flag) == 0) ok = false;
      const bool need_mask = (q0 == k0) || p.window > 0 || has_seg;
      const float* lse_s = s_lse + s * 128 + half * 64;
      const float* del_s = s_delta + s * 128 + half * 64;
      const int* seg_s = s_seg + s * 128 + half * 64;
      float pr[64];
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem + lane_off + COL_ST + half * 64 + c * 32, r);
          tmem_ld_wait();
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int col = c * 32 + e;
            float v = fast_exp2(fmaf(a, __uint_as_float(r[e]), -lse_s[col]));
            if (need_mask && !valid(q0 + half * 64 + col, kg, p.window, has_seg, has_seg ? seg_s[col] : 0, my_seg)) v = 0.f;
            pr[col] = v;
          }
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = pack_bf16(pr[c * 32 + 2 * e], pr[c * 32 + 2 * e + 1]);
          // P^T of this thread's 64 queries: 32 packed columns at the start of its own 64 score columns, so the two
          // halves never write over each other's unread scores
          tmem_st_32x32b_x16(tmem + lane_off + COL_ST + half * 64 + c * 16, pk);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      if (ok) mbar_arrive(bar(P_READY));
      if (et == 128 && ok && !mbar_wait(bar(DP_FULL), ph, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ctl->ok_flag = 0;
      named_bar_sync(2, SM_THREADS);
      if (*reinterpret_cast<volatile int*>(&ctl->ok_flag) == 0) ok = false;
      if (!ok) continue;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t d[32];
        tmem_ld_32x32b_x32(tmem + lane_off + COL_DPT + half * 64 + c * 32, d);
        tmem_ld_wait();
        uint32_t dk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int col = c * 32 + 2 * e;
          const float d0 = pr[col] * (__uint_as_float(d[2 * e]) - del_s[col]) * p.scale;
          const float d1 = pr[col + 1] * (__uint_as_float(d[2 * e + 1]) - del_s[col + 1]) * p.scale;
          dk[e] = pack_bf16(d0, d1);
        }
        tmem_st_32x32b_x16(tmem + lane_off + COL_DPT + half * 64 + c * 16, dk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar(DS_READY));
    }
    if (et == 0 && ok && !mbar_wait(bar(ACC_FULL), 0, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ctl->ok_flag = 0;
    named_bar_sync(1, SM_THREADS);
    ok = *reinterpret_cast<volatile int*>(&ctl->ok_flag) != 0;
    if (ok && n_iter > 0) {
      tc_fence_after();
      // all MMAs have retired: the Q/dO stages become the staging area, dV first then dK
      for (int c = half; c < D / 32; c += 2) {
        stage_rows_bf16(tmem + lane_off + COL_DV + c * 32, sStage + (c >> 1) * 16384, row, c);
        stage_rows_bf16(tmem + lane_off + COL_DK + c * 32, sStage + NBOX * 16384 + (c >> 1) * 16384, row, c);
      }
      fence_proxy_async_smem();
      named_bar_sync(2, SM_THREADS);
      if (et == 0) {
#pragma unroll
        for (int j = 0; j < NBOX; ++j) {
          tma_store_2d(&map_dv, sStage + j * 16384, hk * D + j * 64, row_base + k0);
          tma_store_2d(&map_dk, sStage + NBOX * 16384 + j * 16384, hk * D + j * 64, row_base + k0);
        }
        tma_commit_group();
        tma_wait_group<0>();
      }
    }
  }
  if (*abort_flag) { const uint64_t t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 200000ull) { } }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// ================================================================================================ kernel B: dQ
// Issue order of the MMA warp in steady state:  S_{i+1} | dQ_i | dP_{i+1}: the next tile's scores are computed while
// the softmax threads turn dP_i into dS_i.
template <int D>
__global__ void __launch_bounds__(THREADS, 1)
dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
          const __grid_constant__ CUtensorMap map_do, const __grid_constant__ CUtensorMap map_dq, Params p) {
  constexpr int BIG = 128 * D * 2;
  constexpr int NBOX = D / 64;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DQ = 256;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sDO = base + BIG, sStage = base + 2 * BIG;         // stage s: K at +s*2*BIG, V right after it
  Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + (base - smem_u32(smem_raw)) + 6 * BIG);
  int* s_seg = reinterpret_cast<int*>(ctl + 1);          // [2][128]
  const uint32_t bar0 = smem_u32(&ctl->bars[0]);
  enum { Q_FULL = 0, KV_FULL0, KV_FULL1, KV_EMPTY0, KV_EMPTY1, S_FULL, DP_FULL, S_DONE, DS_READY, ACC_FULL };
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_t = p.S / 128;
  const int qt = n_t - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qt * 128;
  const int row_base = b * p.S;
  int kt_lo = 0;
  if (p.window > 0) { const int lo = q0 - p.window + 1; kt_lo = lo > 0 ? lo / 128 : 0; }
  const int n_kt = qt - kt_lo + 1;

  if (threadIdx.x == 0) {
    ctl->abort_flag = 0;
    ctl->ok_flag = 1;
    mbar_init(bar(Q_FULL), 1);
    for (int s = 0; s < 2; ++s) { mbar_init(bar(KV_FULL0 + s), 1); mbar_init(bar(KV_EMPTY0 + s), 1); }
    mbar_init(bar(S_FULL), 1); mbar_init(bar(DP_FULL), 1);
    mbar_init(bar(S_DONE), SM_THREADS); mbar_init(bar(DS_READY), SM_THREADS);
    mbar_init(bar(ACC_FULL), 1);
    fence_barrier_init();
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_k); prefetch_tensormap(&map_v); prefetch_tensormap(&map_do);
  }
  if (warp == 1) { tmem_alloc(smem_u32(&ctl->tmem_base), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(bar(Q_FULL), 2 * BIG);
#pragma unroll
      for (int j = 0; j < NBOX; ++j) {
        tma_load_2d(sQ + j * 16384, &map_q, bar(Q_FULL), h * D + j * 64, row_base + q0);
        tma_load_2d(sDO + j * 16384, &map_do, bar(Q_FULL), h * D + j * 64, row_base + q0);
      }
      for (int it = 0; it < n_kt; ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int kk = (kt_lo + it) * 128;
        if (!mbar_wait(bar(KV_EMPTY0 + s), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_arrive_expect_tx(bar(KV_FULL0 + s), 2 * BIG);
        const uint32_t sk = sStage + s * 2 * BIG, sv = sk + BIG;
#pragma unroll
        for (int j = 0; j < NBOX; ++j) {
          tma_load_2d(sk + j * 16384, &map_k, bar(KV_FULL0 + s), hk * D + j * 64, row_base + kk);
          tma_load_2d(sv + j * 16384, &map_v, bar(KV_FULL0 + s), hk * D + j * 64, row_base + kk);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_nt = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, false, true);
      auto stage_k = [&](int it) { return sStage + (it & 1) * 2 * BIG; };
      auto issue_s = [&](int it) {
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16_ss(tmem + COL_S, big_kmajor(sQ, k), big_kmajor(stage_k(it), k), idesc_nt, k != 0);
        umma_commit(bar(S_FULL));
      };
      auto issue_dp = [&](int it) {
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16_ss(tmem + COL_DP, big_kmajor(sDO, k), big_kmajor(stage_k(it) + BIG, k), idesc_nt, k != 0);
        umma_commit(bar(DP_FULL));
      };
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag, p.status, ST_TIMEOUT_MMA);
      if (ok) {
        ok = mbar_wait(bar(KV_FULL0), 0, abort_flag, p.status, ST_TIMEOUT_MMA);
        if (ok) { tc_fence_after(); issue_s(0); issue_dp(0); }
      }
      for (int it = 0; it < n_kt && ok; ++it) {
        const uint32_t ph = it & 1;
        if (it + 1 < n_kt) {
          // the score buffer is free as soon as the softmax threads have read it
          if (!mbar_wait(bar(S_DONE), ph, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
          if (!mbar_wait(bar(KV_FULL0 + ((it + 1) & 1)), ((it + 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
          tc_fence_after();
          issue_s(it + 1);
        }
        if (!mbar_wait(bar(DS_READY), ph, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ts(tmem + COL_DQ, tmem + COL_DP + tmem_a_col(k), big_mnmajor(stage_k(it), k), idesc_acc, (it | k) != 0);
        umma_commit(bar(KV_EMPTY0 + (it & 1)));
        if (it + 1 < n_kt) issue_dp(it + 1);
        else umma_commit(bar(ACC_FULL));
      }
    }
  } else {
    const int sw = warp - 2;
    const int qd = warp & 3;
    const int half = sw >> 2;                   // which 64 of the 128 key columns
    const int row = qd * 32 + lane;             // query row
    const int et = threadIdx.x - 64;
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const float a = p.scale * LOG2E;
    const bool has_seg = p.seg != nullptr;
    const int qg = q0 + row;
    const int my_seg = has_seg ? p.seg[b * p.S + qg] : 0;
    const long sidx = ((long)b * p.Hq + h) * p.S + qg;
    const float my_lse = p.lse[sidx] * LOG2E;
    const float my_delta = p.delta[sidx];
    bool ok = true;
    for (int it = 0; it < n_kt; ++it) {
      const int s = it & 1;
      const uint32_t ph = it & 1;
      const int kk = (kt_lo + it) * 128;
      if (has_seg && et < 128) s_seg[s * 128 + et] = p.seg[b * p.S + kk + et];
      if (et == 128 && !mbar_wait(bar(S_FULL), ph, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ctl->ok_flag = 0;
      named_bar_sync(1, SM_THREADS);
      if (*reinterpret_cast<volatile int*>(&ctl->ok_flag) == 0) ok = false;
      const bool need_mask = (kk == q0) || p.window > 0 || has_seg;
      const int* seg_s = s_seg + s * 128 + half * 64;
      float pr[64];
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem + lane_off + COL_S + half * 64 + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int col = c * 32 + e;
            float v = fast_exp2(fmaf(a, __uint_as_float(r[e]), -my_lse));
            if (need_mask && !valid(qg, kk + half * 64 + col, p.window, has_seg, my_seg, has_seg ? seg_s[col] : 0)) v = 0.f;
            pr[col] = v;
          }
        }
        tc_fence_before();
        mbar_arrive(bar(S_DONE));
      }
      if (et == 128 && ok && !mbar_wait(bar(DP_FULL), ph, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ctl->ok_flag = 0;
      named_bar_sync(2, SM_THREADS);
      if (*reinterpret_cast<volatile int*>(&ctl->ok_flag) == 0) ok = false;
      if (!ok) continue;
      tc_fence_after();
      uint32_t dk[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t d[32];
        tmem_ld_32x32b_x32(tmem + lane_off + COL_DP + half * 64 + c * 32, d);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int col = c * 32 + 2 * e;
          dk[c * 16 + e] = pack_bf16(pr[col] * (__uint_as_float(d[2 * e]) - my_delta) * p.scale,
                                     pr[col + 1] * (__uint_as_float(d[2 * e + 1]) - my_delta) * p.scale);
        }
      }
      tmem_st_32x32b_x32(tmem + lane_off + COL_DP + half * 64, dk);   // dS over this thread's own (already read) dP columns
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar(DS_READY));
    }
    if (et == 0 && ok && !mbar_wait(bar(ACC_FULL), 0, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ctl->ok_flag = 0;
    named_bar_sync(1, SM_THREADS);
    ok = *reinterpret_cast<volatile int*>(&ctl->ok_flag) != 0;
    if (ok) {
      tc_fence_after();
      for (int c = half; c < D / 32; c += 2) stage_rows_bf16(tmem + lane_off + COL_DQ + c * 32, sStage + (c >> 1) * 16384, row, c);
      fence_proxy_async_smem();
      named_bar_sync(2, SM_THREADS);
      if (et == 0) {
#pragma unroll
        for (int j = 0; j < NBOX; ++j) tma_store_2d(&map_dq, sStage + j * 16384, h * D + j * 64, row_base + q0);
        tma_commit_group();
        tma_wait_group<0>();
      }
    }
  }
  if (*abort_flag) { const uint64_t t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 200000ull) { } }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// ================================================================================================ host
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

// tokens x (heads*D) view, row stride `ld` elements; box {64 columns, box_rows rows}
static int tok_map(CUtensorMap* m, const void* ptr, long rows, long cols, long ld, int box_rows) {
  EncodeFn enc = encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t es[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

template <typename K>
static int set_smem(K kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess ? 0 : -2;
}

template <int D>
static int run(const CUtensorMap& q64, const CUtensorMap& q128, const CUtensorMap& k64, const CUtensorMap& k128, const CUtensorMap& v64,
               const CUtensorMap& v128, const CUtensorMap& do64, const CUtensorMap& do128, const CUtensorMap& mdq, const CUtensorMap& mdk,
               const CUtensorMap& mdv, const Params& p, cudaStream_t st) {
  const int smem = 6 * 128 * D * 2 + (int)sizeof(Ctl) + 4096 + 1024;
  static bool cfg = false;
  if (!cfg) {
    if (set_smem(dkv_kernel<D>, smem) || set_smem(dq_kernel<D>, smem)) return -2;
    cfg = true;
  }
  dkv_kernel<D><<<dim3(p.S / 128, p.Hkv, p.B), THREADS, smem, st>>>(q128, k128, v128, do128, mdk, mdv, p);
  dq_kernel<D><<<dim3(p.S / 128, p.Hq, p.B), THREADS, smem, st>>>(q128, k128, v128, do128, mdq, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace bwd
}  // namespace mt

// dout/out: contiguous [B,S,Hq,D]; delta: scratch [B,Hq,S] fp32; dq/dk/dv: token-major views with their own row strides.
extern "C" int mt_flash_bwd(const void* dout, const void* q, const void* k, const void* v, const void* out, const float* lse, float* delta,
                            void* dq, void* dk, void* dv, const int* seg, int B, int S, int Hq, int Hkv, int D, long ldq, long ldk,
                            long ldv, long lddq, long lddk, long lddv, float scale, int window, int* status, cudaStream_t st) {
  using namespace mt::bwd;
  if ((D != 128 && D != 64) || S % 128 || Hq % Hkv) return -1;
  const long rows = (long)B * S;
  {
    const long warps = rows * Hq;
    const int threads = 256;
    const long blocks = (warps * 32 + threads - 1) / threads;
    delta_kernel<<<(unsigned)blocks, threads, 0, st>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, delta, B, S, Hq, D);
  }
  CUtensorMap q64, q128, k64, k128, v64, v128, do64, do128, mdq, mdk, mdv;
  const long cq = (long)Hq * D, ck = (long)Hkv * D;
  if (tok_map(&q64, q, rows, cq, ldq, 64) || tok_map(&q128, q, rows, cq, ldq, 128) || tok_map(&k64, k, rows, ck, ldk, 64) ||
      tok_map(&k128, k, rows, ck, ldk, 128) || tok_map(&v64, v, rows, ck, ldv, 64) || tok_map(&v128, v, rows, ck, ldv, 128) ||
      tok_map(&do64, dout, rows, cq, cq, 64) || tok_map(&do128, dout, rows, cq, cq, 128) || tok_map(&mdq, dq, rows, cq, lddq, 128) ||
      tok_map(&mdk, dk, rows, ck, lddk, 128) || tok_map(&mdv, dv, rows, ck, lddv, 128))
    return -3;
  Params p{B, S, Hq, Hkv, D, window, scale, seg, lse, delta, status};
  if (D == 128) return run<128>(q64, q128, k64, k128, v64, v128, do64, do128, mdq, mdk, mdv, p, st);
  return run<64>(q64, q128, k64, k128, v64, v128, do64, do128, mdq, mdk, mdv, p, st);
}
