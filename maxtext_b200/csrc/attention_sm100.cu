// Flash attention forward for sm_100a on tcgen05 / TMEM.
//
// Layout: q [B,S,Hq,D], k/v [B,S,Hkv,D] as (possibly strided) views of a packed projection; tokens are
// rows of a 2-D tensor [B*S, H*D] for TMA. D is 128 or 64, S a multiple of 128, bf16 in / out, fp32
// softmax statistics. Masking is by token index: causal, optional sliding window, optional segment ids.
//
// CTA = 128 queries of one head, 320 threads: warp 0 TMA producer, warp 1 MMA issuer / TMEM owner,
// warps 2..9 softmax (two threads per query row, 64 key columns each).
//   S_i = Q K_i^T goes to one of two TMEM score buffers, so the tensor core computes S_{i+1} while the
//   softmax threads turn S_i into P_i (bf16, written over their own score columns) and O += P_i V_i reads
//   P_i straight from TMEM. O lives in TMEM and is rescaled only when a row maximum moves, after the
//   previous P V product has retired. K / V tiles are double buffered in shared memory.
// The backward lives in attention_bwd_sm100.cu. Every wait is bounded; a timeout records a status code
// and the CTA drains and exits.
#include "sm100_ptx.cuh"
#include <cuda_bf16.h>

namespace mt {
namespace fwd {

constexpr int THREADS = 320;
constexpr int SM_THREADS = 256;
constexpr float LOG2E = 1.4426950408889634f;

struct Params {
  int B, S, Hq, Hkv, D;
  int window;            // 0 = unlimited
  float scale;           // logits = scale * q.k
  const int* seg;        // [B, S] segment ids or nullptr
  float* lse;            // [B, Hq, S]
  int* status;
};

__device__ __forceinline__ bool valid(int qg, int kg, int window) {
  bool v = kg <= qg;
  if (window > 0) v = v && (qg - kg < window);
  return v;
}

// [128 rows x D] bf16 tile stored as D/64 TMA boxes {64, 128} (16 KB each)
__device__ __forceinline__ uint64_t kmajor(uint32_t tile, int k) { return make_smem_desc(tile + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024); }
__device__ __forceinline__ uint64_t mnmajor(uint32_t tile, int k) { return make_smem_desc(tile + k * 2048, 16384, 1024); }
// TMEM column of k-step k of a bf16 operand whose two 64-row halves start 64 columns apart (32 packed columns each)
__device__ __forceinline__ uint32_t tmem_a_col(int k) { return (uint32_t)((k >> 2) * 64 + (k & 3) * 8); }

struct alignas(8) Ctl {
  uint64_t bars[16];
  uint32_t tmem_base;
  int abort_flag;
  int pad[2];
};

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o, Params p) {
  constexpr int TILE = 128 * D * 2;
  constexpr int NBOX = D / 64;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0, COL_O = 256;          // two score buffers of 128 columns, then O
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sKV = base + TILE;         // stage s: K at sKV + s*2*TILE, V right after it
  Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + (base - smem_u32(smem_raw)) + 5 * TILE);
  float* x_max = reinterpret_cast<float*>(ctl + 1);    // [2 parity][2 half][128]
  float* x_sum = x_max + 512;                          // [2 half][128]
  int* seg_k = reinterpret_cast<int*>(x_sum + 256);    // [2 parity][128]
  const uint32_t bar0 = smem_u32(&ctl->bars[0]);
  enum { Q_FULL = 0, KV_FULL0, KV_FULL1, K_EMPTY0, K_EMPTY1, V_EMPTY0, V_EMPTY1, S_FULL0, S_FULL1, P_READY, PV_DONE };
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = p.S / 128;
  const int qt = n_qt - 1 - blockIdx.x;                // heavy (late) query tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qt * 128;
  const int row_base = b * p.S;
  int kt_lo = 0;
  if (p.window > 0) { const int lo = q0 - p.window + 1; kt_lo = lo > 0 ? lo / 128 : 0; }
  const int n_kt = qt - kt_lo + 1;

  if (threadIdx.x == 0) {
    ctl->abort_flag = 0;
    mbar_init(bar(Q_FULL), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(KV_FULL0 + s), 1); mbar_init(bar(K_EMPTY0 + s), 1); mbar_init(bar(V_EMPTY0 + s), 1); mbar_init(bar(S_FULL0 + s), 1);
    }
    mbar_init(bar(P_READY), SM_THREADS);
    mbar_init(bar(PV_DONE), 1);
    fence_barrier_init();
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_k); prefetch_tensormap(&map_v); prefetch_tensormap(&map_o);
  }
  if (warp == 1) { tmem_alloc(smem_u32(&ctl->tmem_base), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(bar(Q_FULL), TILE);
#pragma unroll
      for (int j = 0; j < NBOX; ++j) tma_load_2d(sQ + j * 16384, &map_q, bar(Q_FULL), h * D + j * 64, row_base + q0);
      for (int i = 0; i < n_kt; ++i) {
        const int s = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        const int k0 = (kt_lo + i) * 128;
        if (!mbar_wait(bar(K_EMPTY0 + s), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_PRODUCER)) break;
        if (!mbar_wait(bar(V_EMPTY0 + s), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_arrive_expect_tx(bar(KV_FULL0 + s), 2 * TILE);
        const uint32_t sk = sKV + s * 2 * TILE, sv = sk + TILE;
#pragma unroll
        for (int j = 0; j < NBOX; ++j) {
          tma_load_2d(sk + j * 16384, &map_k, bar(KV_FULL0 + s), hk * D + j * 64, row_base + k0);
          tma_load_2d(sv + j * 16384, &map_v, bar(KV_FULL0 + s), hk * D + j * 64, row_base + k0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
      auto issue_s = [&](int i) {
        const int s = i & 1;
        const uint32_t sk = sKV + s * 2 * TILE;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16_ss(tmem + COL_S + s * 128, kmajor(sQ, k), kmajor(sk, k), idesc_qk, k != 0);
        umma_commit(bar(K_EMPTY0 + s));
        umma_commit(bar(S_FULL0 + s));
      };
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag, p.status, ST_TIMEOUT_MMA);
      if (ok) ok = mbar_wait(bar(KV_FULL0), 0, abort_flag, p.status, ST_TIMEOUT_MMA);
      if (ok) { tc_fence_after(); issue_s(0); }
      for (int i = 0; i < n_kt && ok; ++i) {
        const int s = i & 1;
        if (i + 1 < n_kt) {
          // score buffer (i+1)&1 last held P_{i-1}, consumed by the P V product issued one iteration ago
          if (!mbar_wait(bar(KV_FULL0 + (s ^ 1)), ((i + 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
          tc_fence_after();
          issue_s(i + 1);
        }
        if (!mbar_wait(bar(P_READY), i & 1, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t sv = sKV + s * 2 * TILE + TILE;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_f16_ts(tmem + COL_O, tmem + COL_S + s * 128 + tmem_a_col(k), mnmajor(sv, k), idesc_pv, (i | k) != 0);
        umma_commit(bar(V_EMPTY0 + s));
        umma_commit(bar(PV_DONE));
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax: thread = (query row, 64-key half)
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = qd * 32 + lane;
    const int et = threadIdx.x - 64;
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const float a = p.scale * LOG2E;
    const bool has_seg = p.seg != nullptr;
    const int qg = q0 + row;
    const int my_seg = has_seg ? p.seg[b * p.S + qg] : 0;
    float m = -INFINITY, l = 0.f;                      // l is this thread's partial row sum (its 64 columns)
    bool ok = true;
    for (int i = 0; i < n_kt; ++i) {
      const int s = i & 1;
      const int kt = kt_lo + i;
      const int k0 = kt * 128;
      if (has_seg && et < 128) seg_k[s * 128 + et] = p.seg[b * p.S + k0 + et];
      // A thread whose wait fails goes passive: it keeps meeting the others at the named barriers (nobody is
      // left waiting there) but does no further tensor-memory work and never arrives on P_READY.
      if (ok && !mbar_wait(bar(S_FULL0 + s), (i >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ok = false;
      const bool need_mask = (kt == qt) || p.window > 0;
      float sv[64];
      float tmax = -INFINITY;
      if (ok) {
        tc_fence_after();
        const uint32_t src = tmem + lane_off + COL_S + s * 128 + half * 64;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(src + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) sv[c * 32 + e] = __uint_as_float(r[e]);
        }
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < 64; ++e)
            if (!valid(qg, k0 + half * 64 + e, p.window)) sv[e] = -INFINITY;
        }
        if (!has_seg) {
#pragma unroll
          for (int e = 0; e < 64; ++e) tmax = fmaxf(tmax, sv[e]);
        }
      }
      if (!has_seg) x_max[(s * 2 + half) * 128 + row] = tmax;
      named_bar_sync(1, SM_THREADS);                  // publishes the partial maxima (or the key segment ids)
      if (has_seg) {
        if (ok) {
          const int* sk = seg_k + s * 128 + half * 64;
#pragma unroll
          for (int e = 0; e < 64; ++e) {
            if (!(sk[e] == my_seg && sk[e] != 0)) sv[e] = -INFINITY;
            tmax = fmaxf(tmax, sv[e]);
          }
        }
        x_max[(s * 2 + half) * 128 + row] = tmax;
        named_bar_sync(2, SM_THREADS);
      }
      if (!ok) continue;
      tmax = fmaxf(tmax, x_max[(s * 2 + (half ^ 1)) * 128 + row]);
      const float m_new = fmaxf(m, tmax);
      const float alpha = (m_new == -INFINITY) ? 1.f : fast_exp2(a * (m - m_new));
      const float neg = (m_new == -INFINITY) ? 0.f : -a * m_new;
      float rsum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        float p0 = fast_exp2(fmaf(a, sv[2 * e], neg));
        float p1 = fast_exp2(fmaf(a, sv[2 * e + 1], neg));
        if (m_new == -INFINITY) { p0 = 0.f; p1 = 0.f; }
        rsum += p0 + p1;
        pk[e] = pack_bf16(p0, p1);
      }
      // P over this thread's own (already read) score columns: 32 packed columns at the start of its 64
      tmem_st_32x32b_x32(tmem + lane_off + COL_S + s * 128 + half * 64, pk);
      l = l * alpha + rsum;
      m = m_new;
      if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        // O may only be touched once the previous P V product has retired
        if (!mbar_wait(bar(PV_DONE), (i - 1) & 1, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; continue; }
        tc_fence_after();
#pragma unroll 1
        for (int c = half; c < D / 32; c += 2) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem + lane_off + COL_O + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
          tmem_st_32x32b_x32(tmem + lane_off + COL_O + c * 32, r);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar(P_READY));
    }
    // ---------------------------------------------------------------- epilogue
    x_sum[half * 128 + row] = l;
    if (ok && n_kt > 0 && !mbar_wait(bar(PV_DONE), (n_kt - 1) & 1, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ok = false;
    named_bar_sync(1, SM_THREADS);
    if (ok) {
      tc_fence_after();
      const float lt = l + x_sum[(half ^ 1) * 128 + row];
      const float inv_l = lt > 0.f ? 1.f / lt : 0.f;
      // Q's shared memory is free (all Q K^T products retired): stage the output there, 128-byte swizzled rows
#pragma unroll 1
      for (int c = half; c < D / 32; c += 2) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem + lane_off + COL_O + c * 32, r);
        tmem_ld_wait();
        const uint32_t box = sQ + (c >> 1) * 16384;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t o4[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            o4[e] = pack_bf16(__uint_as_float(r[8 * j + 2 * e]) * inv_l, __uint_as_float(r[8 * j + 2 * e + 1]) * inv_l);
          const int chunk = (c & 1) * 4 + j;
          const uint32_t dst = box + row * 128 + ((chunk ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(o4[0]), "r"(o4[1]), "r"(o4[2]), "r"(o4[3]) : "memory");
        }
      }
      if (half == 0 && p.lse) p.lse[((long)b * p.Hq + h) * p.S + qg] = (lt > 0.f) ? (p.scale * m + logf(lt)) : -INFINITY;
      fence_proxy_async_smem();
    }
    named_bar_sync(2, SM_THREADS);
    if (et == 0 && *abort_flag == 0) {
#pragma unroll
      for (int j = 0; j < NBOX; ++j) tma_store_2d(&map_o, sQ + j * 16384, h * D + j * 64, row_base + q0);
      tma_commit_group();
      tma_wait_group<0>();
    }
  }
  if (*abort_flag) { const uint64_t t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 200000ull) { } }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// ================================================================================================ two CTAs per SM
// The same algorithm arranged so that TWO CTAs fit on an SM (256 tensor-memory columns and ~100 KB of shared memory each,
// at most 102 registers per thread): one score buffer, K and V single-buffered with separate barriers, and the softmax
// threads walk their 64 columns in two chunks of 32 (one pass for the row maximum, one for the exponentials) instead of
// holding all of them in registers. Inside one CTA the tensor core now idles while its softmax runs, but the co-resident
// CTA's products fill that time, which overlaps better than the single-CTA double buffering did.
template <int D>
__global__ void __launch_bounds__(THREADS, 2)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                  const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o, Params p) {
  constexpr int TILE = 128 * D * 2;
  constexpr int NBOX = D / 64;
  constexpr uint32_t TMEM_COLS = 256;
  constexpr uint32_t COL_S = 0, COL_O = 128;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sK = base + TILE, sV = base + 2 * TILE;
  Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + (base - smem_u32(smem_raw)) + 3 * TILE);
  float* x_max = reinterpret_cast<float*>(ctl + 1);    // [2 half][128]
  float* x_sum = x_max + 256;                          // [2 half][128]
  int* seg_k = reinterpret_cast<int*>(x_sum + 256);    // [128]
  const uint32_t bar0 = smem_u32(&ctl->bars[0]);
  enum { Q_FULL = 0, K_FULL, V_FULL, K_EMPTY, V_EMPTY, S_FULL, P_READY, PV_DONE };
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = p.S / 128;
  const int qt = n_qt - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qt * 128;
  const int row_base = b * p.S;
  int kt_lo = 0;
  if (p.window > 0) { const int lo = q0 - p.window + 1; kt_lo = lo > 0 ? lo / 128 : 0; }
  const int n_kt = qt - kt_lo + 1;

  if (threadIdx.x == 0) {
    ctl->abort_flag = 0;
    for (int i = Q_FULL; i <= S_FULL; ++i) mbar_init(bar(i), 1);
    mbar_init(bar(P_READY), SM_THREADS);
    mbar_init(bar(PV_DONE), 1);
    fence_barrier_init();
    prefetch_tensormap(&map_q); prefetch_tensormap(&map_k); prefetch_tensormap(&map_v); prefetch_tensormap(&map_o);
  }
  if (warp == 1) { tmem_alloc(smem_u32(&ctl->tmem_base), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&ctl->tmem_base);
  volatile int* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(bar(Q_FULL), TILE);
#pragma unroll
      for (int j = 0; j < NBOX; ++j) tma_load_2d(sQ + j * 16384, &map_q, bar(Q_FULL), h * D + j * 64, row_base + q0);
      for (int i = 0; i < n_kt; ++i) {
        const uint32_t ph = i & 1;
        const int k0 = (kt_lo + i) * 128;
        if (!mbar_wait(bar(K_EMPTY), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_arrive_expect_tx(bar(K_FULL), TILE);
#pragma unroll
        for (int j = 0; j < NBOX; ++j) tma_load_2d(sK + j * 16384, &map_k, bar(K_FULL), hk * D + j * 64, row_base + k0);
        if (!mbar_wait(bar(V_EMPTY), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_arrive_expect_tx(bar(V_FULL), TILE);
#pragma unroll
        for (int j = 0; j < NBOX; ++j) tma_load_2d(sV + j * 16384, &map_v, bar(V_FULL), hk * D + j * 64, row_base + k0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag, p.status, ST_TIMEOUT_MMA);
      for (int i = 0; i < n_kt && ok; ++i) {
        const uint32_t ph = i & 1;
        if (!mbar_wait(bar(K_FULL), ph, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
        // the score buffer held P_{i-1}; the P V product that reads it was issued by this thread before, and products
        // issued by one thread execute in order
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16_ss(tmem + COL_S, kmajor(sQ, k), kmajor(sK, k), idesc_qk, k != 0);
        umma_commit(bar(K_EMPTY));
        umma_commit(bar(S_FULL));
        if (!mbar_wait(bar(V_FULL), ph, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
        if (!mbar_wait(bar(P_READY), ph, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) umma_f16_ts(tmem + COL_O, tmem + COL_S + tmem_a_col(k), mnmajor(sV, k), idesc_pv, (i | k) != 0);
        umma_commit(bar(V_EMPTY));
        umma_commit(bar(PV_DONE));
      }
    }
  } else {
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = qd * 32 + lane;
    const int et = threadIdx.x - 64;
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const float a = p.scale * LOG2E;
    const bool has_seg = p.seg != nullptr;
    const int qg = q0 + row;
    const int my_seg = has_seg ? p.seg[b * p.S + qg] : 0;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int i = 0; i < n_kt; ++i) {
      const uint32_t ph = i & 1;
      const int kt = kt_lo + i;
      const int k0 = kt * 128;
      if (ok && !mbar_wait(bar(S_FULL), ph, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ok = false;
      // S_i exists only after P V_{i-1} was issued, i.e. after every thread arrived on P_READY at the end of tile i-1:
      // nobody still reads the previous tile's seg_k / x_max, so they can be overwritten without a further barrier
      if (has_seg) {
        if (et < 128) seg_k[et] = p.seg[b * p.S + k0 + et];
        named_bar_sync(2, SM_THREADS);                 // seg_k published
      }
      const bool need_mask = (kt == qt) || p.window > 0 || has_seg;
      const uint32_t src = tmem + lane_off + COL_S + half * 64;
      const int* sk = seg_k + half * 64;
      float tmax = -INFINITY;
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(src + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            float v = __uint_as_float(r[e]);
            if (need_mask) {
              const int kg = k0 + half * 64 + c * 32 + e;
              bool keep = valid(qg, kg, p.window);
              if (has_seg) keep = keep && sk[c * 32 + e] == my_seg && my_seg != 0;
              if (!keep) v = -INFINITY;
            }
            tmax = fmaxf(tmax, v);
          }
        }
      }
      x_max[half * 128 + row] = tmax;
      named_bar_sync(1, SM_THREADS);
      if (!ok) continue;
      tmax = fmaxf(tmax, x_max[(half ^ 1) * 128 + row]);
      const float m_new = fmaxf(m, tmax);
      const float alpha = (m_new == -INFINITY) ? 1.f : fast_exp2(a * (m - m_new));
      const float neg = (m_new == -INFINITY) ? 0.f : -a * m_new;
      float rsum = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(src + c * 32, r);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          float v0 = __uint_as_float(r[2 * e]), v1 = __uint_as_float(r[2 * e + 1]);
          if (need_mask) {
            const int kg = k0 + half * 64 + c * 32 + 2 * e;
            bool k0v = valid(qg, kg, p.window), k1v = valid(qg, kg + 1, p.window);
            if (has_seg) {
              k0v = k0v && sk[c * 32 + 2 * e] == my_seg && my_seg != 0;
              k1v = k1v && sk[c * 32 + 2 * e + 1] == my_seg && my_seg != 0;
            }
            if (!k0v) v0 = -INFINITY;
            if (!k1v) v1 = -INFINITY;
          }
          float p0 = fast_exp2(fmaf(a, v0, neg));
          float p1 = fast_exp2(fmaf(a, v1, neg));
          if (m_new == -INFINITY) { p0 = 0.f; p1 = 0.f; }
          rsum += p0 + p1;
          pk[e] = pack_bf16(p0, p1);
        }
        // chunk c of P (16 packed columns) lands inside columns this thread has already read
        tmem_st_32x32b_x16(src + c * 16, pk);
      }
      l = l * alpha + rsum;
      m = m_new;
      if (i > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        if (!mbar_wait(bar(PV_DONE), (i - 1) & 1, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; continue; }
        tc_fence_after();
#pragma unroll 1
        for (int c = half; c < D / 32; c += 2) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem + lane_off + COL_O + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
          tmem_st_32x32b_x32(tmem + lane_off + COL_O + c * 32, r);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar(P_READY));
    }
    x_sum[half * 128 + row] = l;
    if (ok && n_kt > 0 && !mbar_wait(bar(PV_DONE), (n_kt - 1) & 1, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ok = false;
    named_bar_sync(1, SM_THREADS);
    if (ok) {
      tc_fence_after();
      const float lt = l + x_sum[(half ^ 1) * 128 + row];
      const float inv_l = lt > 0.f ? 1.f / lt : 0.f;
#pragma unroll 1
      for (int c = half; c < D / 32; c += 2) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem + lane_off + COL_O + c * 32, r);
        tmem_ld_wait();
        const uint32_t box = sQ + (c >> 1) * 16384;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t o4[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            o4[e] = pack_bf16(__uint_as_float(r[8 * j + 2 * e]) * inv_l, __uint_as_float(r[8 * j + 2 * e + 1]) * inv_l);
          const int chunk = (c & 1) * 4 + j;
          const uint32_t dst = box + row * 128 + ((chunk ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(o4[0]), "r"(o4[1]), "r"(o4[2]), "r"(o4[3]) : "memory");
        }
      }
      if (half == 0 && p.lse) p.lse[((long)b * p.Hq + h) * p.S + qg] = (lt > 0.f) ? (p.scale * m + logf(lt)) : -INFINITY;
      fence_proxy_async_smem();
    }
    named_bar_sync(2, SM_THREADS);
    if (et == 0 && *abort_flag == 0) {
#pragma unroll
      for (int j = 0; j < NBOX; ++j) tma_store_2d(&map_o, sQ + j * 16384, h * D + j * 64, row_base + q0);
      tma_commit_group();
      tma_wait_group<0>();
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

// tokens x (heads*D) view with row stride `ld` elements; box {64 columns, 128 rows}
static int tok_map(CUtensorMap* m, const void* ptr, long rows, long cols, long ld) {
  EncodeFn enc = encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t es[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

static int g_fwd_variant = 1;      // 1 = one CTA per SM with double buffering (default: measured 1.45 ms vs 1.79 ms at B2 S8192 H32/8 D128), 2 = two CTAs per SM

template <int D>
static int run2(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo, const Params& p, cudaStream_t st) {
  const int smem = 3 * 128 * D * 2 + (int)sizeof(Ctl) + 2560 + 1024;
  static bool cfg = false;
  if (!cfg) {
    if (cudaFuncSetAttribute(flash_fwd2_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -2;
    cfg = true;
  }
  flash_fwd2_kernel<D><<<dim3(p.S / 128, p.Hq, p.B), THREADS, smem, st>>>(mq, mk, mv, mo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <int D>
static int run(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo, const Params& p, cudaStream_t st) {
  if (g_fwd_variant == 2) return run2<D>(mq, mk, mv, mo, p, st);
  const int smem = 5 * 128 * D * 2 + (int)sizeof(Ctl) + 4096 + 1024;
  static bool cfg = false;
  if (!cfg) {
    if (cudaFuncSetAttribute(flash_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -2;
    cfg = true;
  }
  flash_fwd_kernel<D><<<dim3(p.S / 128, p.Hq, p.B), THREADS, smem, st>>>(mq, mk, mv, mo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace fwd
}  // namespace mt

// q/k/v/out: token-major views, ld* = row stride in elements (tokens of one batch are consecutive rows).
extern "C" int mt_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* seg, int B, int S, int Hq,
                            int Hkv, int D, long ldq, long ldk, long ldv, long ldo, float scale, int window, int* status,
                            cudaStream_t st) {
  using namespace mt::fwd;
  if ((D != 128 && D != 64) || S % 128 || Hq % Hkv) return -1;
  CUtensorMap mq, mk, mv, mo;
  const long rows = (long)B * S;
  if (tok_map(&mq, q, rows, (long)Hq * D, ldq) || tok_map(&mk, k, rows, (long)Hkv * D, ldk) ||
      tok_map(&mv, v, rows, (long)Hkv * D, ldv) || tok_map(&mo, out, rows, (long)Hq * D, ldo))
    return -3;
  Params p{B, S, Hq, Hkv, D, window, scale, seg, lse, status};
  if (D == 128) return run<128>(mq, mk, mv, mo, p, st);
  return run<64>(mq, mk, mv, mo, p, st);
}

extern "C" int mt_flash_fwd_set_variant(int v) {   // tuning hook: 1 or 2 (see flash_fwd2_kernel)
  if (v != 1 && v != 2) return -1;
  mt::fwd::g_fwd_variant = v;
  return 0;
}
