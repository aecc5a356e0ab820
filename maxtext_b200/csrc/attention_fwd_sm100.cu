// Flash attention forward for sm_100a on tcgen05 / TMEM.
//
// Layout: q [B,Sq,Hq,Dqk], k [B,Skv,Hkv,Dqk], v [B,Skv,Hkv,Dv], out [B,Sq,Hq,Dv] as (possibly strided) views of packed
// projections: each is a 3-D tensor {heads*D, tokens, batch} for TMA, so a sequence length that is not a multiple of
// the tile is zero-filled on load and clipped on store. bf16 in / out, fp32 softmax statistics, log-sum-exp out.
//
// CTA = TWO 128-query tiles of one head (256 consecutive queries), 320 threads:
//   warp 0      TMA producer: Q tiles once, then K / V tiles through two-stage rings
//   warp 1      MMA issuer / TMEM owner
//   warps 2..5  softmax of query tile 0, one thread per query row (all 128 key columns in registers)
//   warps 6..9  softmax of query tile 1
// The tensor core alternates between the two query tiles:  P0 V -> S0(next) -> P1 V -> S1(next) -> ...  so while the
// softmax threads of one tile turn scores into probabilities the other tile's products run. S_i lives in its own 128
// TMEM columns; P_i (bf16) is written over the first 64 of them and consumed by tcgen05.mma as the TMEM operand; O_i
// stays in TMEM for the whole key loop. A softmax thread walks its 128 score columns twice, 32 at a time with the next
// tensor-memory load in flight (maximum, then probabilities with packed two-float arithmetic), so no score is spilled;
// the first 64 probabilities are announced as soon as they are written and the P V product starts on them. A row's
// reference maximum is only moved when the new maximum exceeds it by more than 2^8 (probabilities then stay below 256,
// exact in the final normalisation), so rescaling O is rare and is done by the row's own softmax thread once the
// previous P V product has retired.
//
// Masks: causal on positions, sliding window, chunked (block-local) attention, segment ids, keys beyond Skv. Positions
// are token indices (queries offset by q_off) or come from arrays (context parallelism: the keys are a block of a
// longer sequence); with arrays, per-tile (min, max) tables let every role skip fully masked key tiles. Optional logit
// soft-cap and per-head sink logits. Every wait is bounded; a timeout records a status code and the CTA drains and exits.
// The backward lives in attention_bwd_sm100.cu.
#include "attention_mask.cuh"
#include "sm100_ptx.cuh"
#include <cuda_bf16.h>
#include <type_traits>

namespace mt {
namespace fwd {

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr float RESCALE_THRESHOLD = 8.f;     // log2 units

struct Params {
  int B, Hq, Hkv;
  int n_pairs;           // CTAs per (batch, head): ceil(Sq / (128 * query tiles per CTA))
  int head_major;        // CTA order: 1 = all query pairs of a head together, 0 = heaviest pairs of all heads first
  attn::Mask mk;
  float scale;           // logits = scale * q.k
  float softcap;         // 0 = none; logits = softcap * tanh(scale * q.k / softcap)
  const float* sinks;    // [Hq] or nullptr
  float* lse;            // [B,Hq,Sq]
  int* status;
};

// [128 rows x D] bf16 tile stored as D/64 TMA boxes {64, 128} (16 KB each)
__device__ __forceinline__ uint64_t kmajor(uint32_t tile, int k) { return make_smem_desc(tile + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024); }
__device__ __forceinline__ uint64_t mnmajor(uint32_t tile, int k) { return make_smem_desc(tile + k * 2048, 16384, 1024); }

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct alignas(8) Ctl {
  uint64_t bars[20];
  uint32_t tmem_base;
  int abort_flag;
  int pad[2];
};

template <int DQK, int DV, int NQ>
__device__ __forceinline__ void flash_fwd_body(const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v,
                                               const CUtensorMap& map_o, const Params& p) {
  constexpr int QT = 128 * DQK * 2;          // bytes of a Q or K tile
  constexpr int VT = 128 * DV * 2;           // bytes of a V tile
  constexpr int NBQ = DQK / 64, NBV = DV / 64;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0, COL_O = 256;            // S_i at i*128, O_i at 256 + i*128
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base;                              // Q_i at sQ + i*QT
  const uint32_t sK = sQ + NQ * QT;                      // stage s at sK + s*QT
  const uint32_t sV = sK + 2 * QT;                       // stage s at sV + s*VT
  uint8_t* after = smem_raw + (base - smem_u32(smem_raw)) + NQ * QT + 2 * QT + 2 * VT;
  Ctl* ctl = reinterpret_cast<Ctl*>(after);
  int* sk_pos = reinterpret_cast<int*>(ctl + 1);         // [tile i][parity][128]
  int* sk_seg = sk_pos + 2 * 2 * 128;                    // [tile i][parity][128]
  const uint32_t bar0 = smem_u32(&ctl->bars[0]);
  enum { Q_FULL = 0, K_FULL0, K_FULL1, V_FULL0, V_FULL1, K_EMPTY0, K_EMPTY1, V_EMPTY0, V_EMPTY1, S_FULL0, S_FULL1, PA_READY0, PA_READY1,
         PV_DONE0, PV_DONE1, PB_READY0, PB_READY1 };
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heaviest CTAs first: for causal masks the last query pairs see the most keys
  const int hb = p.Hq * p.B;
  int pair, h, b;
  if (p.head_major) {
    pair = p.n_pairs - 1 - (int)(blockIdx.x % p.n_pairs);
    h = (int)(blockIdx.x / p.n_pairs) % p.Hq; b = (int)(blockIdx.x / p.n_pairs) / p.Hq;
  } else {
    pair = p.n_pairs - 1 - (int)(blockIdx.x / hb);
    h = (int)(blockIdx.x % hb) % p.Hq; b = (int)(blockIdx.x % hb) / p.Hq;
  }
  const int hk = h / (p.Hq / p.Hkv);

  const attn::Mask& mk = p.mk;
  attn::Span qt[NQ];
  int q0s[NQ];
  // key tiles [kt_lo, kt_hi) that any query tile of this CTA may need (exact in index mode, everything in array mode)
  int kt_lo = INT_MAX, kt_hi = 0;
#pragma unroll
  for (int i = 0; i < NQ; ++i) {
    q0s[i] = (pair * NQ + i) * 128;
    qt[i] = attn::q_span(mk, b, pair * NQ + i);
    int lo, hi;
    attn::k_tiles_for(mk, qt[i], lo, hi);
    if (qt[i].rows) { kt_lo = lo < kt_lo ? lo : kt_lo; kt_hi = hi > kt_hi ? hi : kt_hi; }
  }
  if (kt_lo == INT_MAX) kt_lo = 0;
  if (kt_hi < kt_lo) kt_hi = kt_lo;
  const int n_u = kt_hi - kt_lo;

  if (threadIdx.x == 0) {
    ctl->abort_flag = 0;
    mbar_init(bar(Q_FULL), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(K_FULL0 + s), 1); mbar_init(bar(V_FULL0 + s), 1); mbar_init(bar(K_EMPTY0 + s), 1); mbar_init(bar(V_EMPTY0 + s), 1);
      mbar_init(bar(S_FULL0 + s), 1); mbar_init(bar(PV_DONE0 + s), 1);
      mbar_init(bar(PA_READY0 + s), 4); mbar_init(bar(PB_READY0 + s), 4);          // one arrival per softmax warp
    }
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
    // ================================================================ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(bar(Q_FULL), NQ * QT);
#pragma unroll
      for (int i = 0; i < NQ; ++i)
#pragma unroll
        for (int j = 0; j < NBQ; ++j) tma_load_3d(sQ + i * QT + j * 16384, &map_q, bar(Q_FULL), h * DQK + j * 64, q0s[i], b);
      for (int u = 0; u < n_u; ++u) {
        const int s = u & 1;
        const uint32_t ph = (u >> 1) & 1;
        const int k0 = (kt_lo + u) * 128;
        if (!mbar_wait(bar(K_EMPTY0 + s), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_arrive_expect_tx(bar(K_FULL0 + s), QT);
#pragma unroll
        for (int j = 0; j < NBQ; ++j) tma_load_3d(sK + s * QT + j * 16384, &map_k, bar(K_FULL0 + s), hk * DQK + j * 64, k0, b);
        if (!mbar_wait(bar(V_EMPTY0 + s), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_arrive_expect_tx(bar(V_FULL0 + s), VT);
#pragma unroll
        for (int j = 0; j < NBV; ++j) tma_load_3d(sV + s * VT + j * 16384, &map_v, bar(V_FULL0 + s), hk * DV + j * 64, k0, b);
      }
    }
  } else if (warp == 1) {
    // ================================================================ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, DV, false, true);
      int cnt[NQ];
#pragma unroll
      for (int i = 0; i < NQ; ++i) cnt[i] = 0;
      auto issue_s = [&](int i, int u) {
        if (attn::classify(mk, qt[i], attn::k_span(mk, b, kt_lo + u)) == 0) return;
        const uint32_t sk = sK + (u & 1) * QT;
#pragma unroll
        for (int k = 0; k < DQK / 16; ++k) umma_f16_ss(tmem + COL_S + i * 128, kmajor(sQ + i * QT, k), kmajor(sk, k), idesc_qk, k != 0);
        umma_commit(bar(S_FULL0 + i));
      };
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag, p.status, ST_TIMEOUT_MMA);
      if (ok && n_u > 0) {
        ok = mbar_wait(bar(K_FULL0), 0, abort_flag, p.status, ST_TIMEOUT_MMA);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int i = 0; i < NQ; ++i) issue_s(i, 0);
          umma_commit(bar(K_EMPTY0));
        }
      }
      for (int u = 0; u < n_u && ok; ++u) {
        const int s = u & 1;
        if (!mbar_wait(bar(V_FULL0 + s), (u >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
        const uint32_t sv = sV + s * VT;
#pragma unroll
        for (int i = 0; i < NQ; ++i) {
          if (attn::classify(mk, qt[i], attn::k_span(mk, b, kt_lo + u)) != 0) {
            // the probabilities arrive in two halves of 64 keys; the product starts on the first while the second is computed
            if (!mbar_wait(bar(PA_READY0 + i), cnt[i] & 1, abort_flag, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_f16_ts(tmem + COL_O + i * 128, tmem + COL_S + i * 128 + k * 8, mnmajor(sv, k), idesc_pv, (cnt[i] | k) != 0);
            if (!mbar_wait(bar(PB_READY0 + i), cnt[i] & 1, abort_flag, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int k = 4; k < 8; ++k)
              umma_f16_ts(tmem + COL_O + i * 128, tmem + COL_S + i * 128 + k * 8, mnmajor(sv, k), idesc_pv, 1);
            umma_commit(bar(PV_DONE0 + i));
            ++cnt[i];
          }
          if (u + 1 < n_u) {
            if (i == 0) {
              if (!mbar_wait(bar(K_FULL0 + (s ^ 1)), ((u + 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
              tc_fence_after();
            }
            issue_s(i, u + 1);
            if (i == NQ - 1) umma_commit(bar(K_EMPTY0 + (s ^ 1)));
          }
          if (i == NQ - 1) umma_commit(bar(V_EMPTY0 + s));
        }
      }
    }
  } else {
    // ================================================================ softmax: warps 2..5 tile 0, warps 6..9 tile 1
    const int i = (warp - 2) >> 2;
    const int qd = warp & 3;                           // TMEM lane quarter this warp may touch
    const int row = qd * 32 + lane;
    const int wt = threadIdx.x - 64 - i * 128;         // 0..127 inside the group
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const uint32_t tS = tmem + lane_off + COL_S + i * 128;
    const uint32_t tO = tmem + lane_off + COL_O + i * 128;
    const attn::Span t = qt[i];
    const int tq0 = q0s[i];
    const int qg = tq0 + row;
    const bool row_ok = row < t.rows;
    const bool has_seg = mk.seg_q != nullptr;
    const bool arrays = mk.pos_k != nullptr;
    const bool cap = p.softcap > 0.f;
    const float a = cap ? p.softcap * LOG2E : p.scale * LOG2E;     // y = a * s' is the logit in log2 units
    float m = -INFINITY, l = 0.f;                                  // reference maximum (log2 units) and row sum
    int cnt = 0;
    bool ok = true;

    auto max32 = [](const uint32_t (&r)[32]) {
      float v0 = fmax3(__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]));
      float v1 = fmax3(__uint_as_float(r[3]), __uint_as_float(r[4]), __uint_as_float(r[5]));
#pragma unroll
      for (int e = 6; e < 30; e += 4) {
        v0 = fmax3(v0, __uint_as_float(r[e]), __uint_as_float(r[e + 1]));
        v1 = fmax3(v1, __uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
      }
      return fmax3(v0, v1, fmaxf(__uint_as_float(r[30]), __uint_as_float(r[31])));
    };

    // One key tile of this row in two passes over its 128 score columns (maximum, then probabilities), 32 columns at a time so
    // that a row never holds more than two chunks in registers. MASKED tiles (and soft-capped logits) take the same route with
    // the mask state derived here, so the unmasked fast path carries none of it.
    auto tile = [&](auto masked_t, int k0, int par) {
      constexpr bool MASKED = decltype(masked_t)::value;
      int lo_p = 0, my_seg = 1;
      uint32_t span = 0;
      bool none = false;
      [[maybe_unused]] const bool has_seg = MASKED && mk.seg_q != nullptr;
      [[maybe_unused]] const bool arrays = MASKED && mk.pos_k != nullptr;
      float pre = 1.f;
      if constexpr (MASKED) {
        const int qpos = mk.pos_q ? (row_ok ? mk.pos_q[(long)b * mk.Sq + qg] : 0) : qg + mk.q_off;
        if (has_seg) my_seg = row_ok ? mk.seg_q[(long)b * mk.Sq + qg] : 0;
        int hi_p;
        attn::key_interval(mk, qpos, lo_p, hi_p);                   // keys this row may attend to, as a closed position interval
        span = (uint32_t)hi_p - (uint32_t)lo_p;                     // lo_p <= position <= hi_p as one unsigned comparison
        none = hi_p < lo_p;
        if (cap) pre = p.scale / p.softcap;
      }
      // soft-cap and mask of 32 score columns starting at column c0 of the tile
      auto prepare = [&](uint32_t (&r)[32], int c0) {
        if constexpr (MASKED) {
          if (cap) {
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(fast_tanh(__uint_as_float(r[e]) * pre));
          }
          if (arrays) {
            const int* kp = sk_pos + (i * 2 + par) * 128 + c0;
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if ((uint32_t)kp[e] - (uint32_t)lo_p > span || none) r[e] = 0xff800000u;
          } else {
            const uint32_t e_lo = (uint32_t)lo_p - (uint32_t)(k0 + c0);
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if ((uint32_t)e - e_lo > span || none) r[e] = 0xff800000u;
          }
          if (has_seg) {
            const int* ks = sk_seg + (i * 2 + par) * 128 + c0;
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (ks[e] != my_seg || my_seg == 0) r[e] = 0xff800000u;
          }
        }
      };
      // pass 1: exact row maximum of the tile; the loads run one 32-column chunk ahead of the arithmetic
      uint32_t r0[32], r1[32];
      float tmax;
      tmem_ld_32x32b_x32(tS, r0);
      tmem_ld_wait_dep(r0);
      tmem_ld_32x32b_x32(tS + 32, r1);
      prepare(r0, 0);
      tmax = max32(r0);
      tmem_ld_wait_dep(r1);
      tmem_ld_32x32b_x32(tS + 64, r0);
      prepare(r1, 32);
      tmax = fmaxf(tmax, max32(r1));
      tmem_ld_wait_dep(r0);
      tmem_ld_32x32b_x32(tS + 96, r1);
      prepare(r0, 64);
      tmax = fmaxf(tmax, max32(r0));
      tmem_ld_wait_dep(r1);
      tmem_ld_32x32b_x32(tS, r0);              // first chunk of pass 2
      prepare(r1, 96);
      tmax = fmaxf(tmax, max32(r1));
      const float mt_ = a * tmax;                                    // -inf when the whole row is masked
      const bool grow = mt_ > m + RESCALE_THRESHOLD;                 // m = -inf: any finite maximum grows it
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = grow ? fast_exp2(m - mt_) : 1.f;
        if (cnt > 0) {
          // O may only be touched once the previous P V product of this tile has retired
          if (!mbar_wait(bar(PV_DONE0 + i), (cnt - 1) & 1, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) { ok = false; return; }
          tc_fence_after();
          tmem_ld_wait_dep(r0);
#pragma unroll 1
          for (int c = 0; c < DV / 32; ++c) {
            tmem_ld_32x32b_x32(tO + c * 32, r1);
            tmem_ld_wait_dep(r1);
#pragma unroll
            for (int e = 0; e < 32; ++e) r1[e] = __float_as_uint(__uint_as_float(r1[e]) * alpha);
            tmem_st_32x32b_x32(tO + c * 32, r1);
          }
        }
        if (grow) { l *= alpha; m = mt_; }
      }
      // pass 2: probabilities, written over the row's own (already read) score columns chunk by chunk
      const float neg = (m == -INFINITY) ? 0.f : -m;
      // packed two-float arithmetic (fma.f32x2 / add.f32x2): half the issue slots of the scale-and-shift and of the row sum
      const float2 a2 = make_float2(a, a), neg2 = make_float2(neg, neg);
      float2 rsa = make_float2(0.f, 0.f), rsb = make_float2(0.f, 0.f);
      auto exps = [&](uint32_t (&r)[32], int c) {
        prepare(r, c * 32);
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1])), a2, neg2);
          const float2 pp = make_float2(fast_exp2(x.x), fast_exp2(x.y));
          if (e & 1) rsb = __fadd2_rn(rsb, pp); else rsa = __fadd2_rn(rsa, pp);
          pk[e] = pack_bf16(pp.x, pp.y);
        }
        tmem_st_32x32b_x16(tS + c * 16, pk);
      };
      tmem_ld_wait_dep(r0);
      tmem_ld_32x32b_x32(tS + 32, r1);
      exps(r0, 0);
      tmem_ld_wait_dep(r1);
      tmem_ld_32x32b_x32(tS + 64, r0);
      exps(r1, 1);
      tmem_ld_wait_dep(r0);
      tmem_ld_32x32b_x32(tS + 96, r1);
      // the first 64 keys' probabilities are in place: the P V product may start on them
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(PA_READY0 + i));
      exps(r0, 2);
      tmem_ld_wait_dep(r1);
      exps(r1, 3);
      l += (rsa.x + rsa.y) + (rsb.x + rsb.y);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(PB_READY0 + i));
    };

    for (int u = 0; u < n_u; ++u) {
      const int kt = kt_lo + u;
      const int cls = attn::classify(mk, t, attn::k_span(mk, b, kt));
      if (cls == 0) continue;
      const int k0 = kt * 128;
      const int par = cnt & 1;
      const bool masked = cls == 2 || cap;
      if (masked && (mk.pos_k != nullptr || mk.seg_q != nullptr)) {
        const int kg = k0 + wt;
        if (mk.pos_k) sk_pos[(i * 2 + par) * 128 + wt] = kg < mk.Skv ? mk.pos_k[(long)b * mk.Skv + kg] : INT_MAX;
        if (mk.seg_q) sk_seg[(i * 2 + par) * 128 + wt] = kg < mk.Skv ? mk.seg_k[(long)b * mk.Skv + kg] : 0;
        named_bar_sync(1 + i, 128);
      }
      if (ok && !mbar_wait(bar(S_FULL0 + i), cnt & 1, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ok = false;
      if (ok) {
        tc_fence_after();
        if (masked) tile(std::true_type{}, k0, par);
        else tile(std::false_type{}, k0, par);
      }
      ++cnt;
    }
    // ---------------------------------------------------------------- epilogue of this query tile
    if (t.rows > 0) {
      if (ok && cnt > 0 && !mbar_wait(bar(PV_DONE0 + i), (cnt - 1) & 1, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ok = false;
      if (ok && cnt == 0 && !mbar_wait(bar(Q_FULL), 0, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ok = false;   // Q's buffer becomes the staging area
      if (ok) {
        tc_fence_after();
        float lt = l;
        if (p.sinks) {
          const float sk = p.sinks[h] * LOG2E;
          if (m == -INFINITY) { m = sk; lt = 1.f; } else lt += fast_exp2(sk - m);
        }
        const float inv_l = lt > 0.f ? 1.f / lt : 0.f;
        // all Q K^T products of this tile retired: stage the output in Q's shared memory, 128-byte swizzled rows
#pragma unroll 1
        for (int c = 0; c < DV / 32; ++c) {
          uint32_t r[32];
          if (cnt > 0) {
            tmem_ld_32x32b_x32(tO + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = 0u;
          }
          const uint32_t box = sQ + i * QT + (c >> 1) * 16384;
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
        if (row_ok && p.lse) p.lse[((long)b * p.Hq + h) * mk.Sq + qg] = (lt > 0.f) ? (m + log2f(lt)) * LN2 : -INFINITY;
        fence_proxy_async_smem();
      }
      named_bar_sync(1 + i, 128);
      if (wt == 0 && *abort_flag == 0) {
#pragma unroll
        for (int j = 0; j < NBV; ++j) tma_store_3d(&map_o, sQ + i * QT + j * 16384, h * DV + j * 64, tq0, b);
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

// The register file gives 320 threads 168 registers each (warps are allocated in groups of four, so ten warps cost twelve):
// the 128 scores of a row stay in registers with a few spilled temporaries.
template <int DQK, int DV, int NQ>
__global__ void __launch_bounds__(64 + 128 * NQ, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o, const __grid_constant__ Params p) {
  flash_fwd_body<DQK, DV, NQ>(map_q, map_k, map_v, map_o, p);
}

// (min, max) of every 128-token tile of a position array [B, S]; tiles beyond S are not written. One warp per tile.
__global__ void tile_minmax_kernel(const int* __restrict__ pos, int B, int S, int n_tiles, int* __restrict__ out) {
  const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (w >= B * n_tiles) return;
  const int b = w / n_tiles, t = w % n_tiles;
  int mn = INT_MAX, mx = INT_MIN;
  for (int e = lane; e < 128; e += 32) {
    const int idx = t * 128 + e;
    if (idx < S) { const int v = pos[(long)b * S + idx]; mn = v < mn ? v : mn; mx = v > mx ? v : mx; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const int a = __shfl_xor_sync(0xffffffffu, mn, o), c = __shfl_xor_sync(0xffffffffu, mx, o);
    mn = a < mn ? a : mn;
    mx = c > mx ? c : mx;
  }
  if (lane == 0) { out[(long)w * 2] = mn; out[(long)w * 2 + 1] = mx; }
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

// {heads*D, tokens, batch} view with row stride `ld` and batch stride `bs` (elements); box {64 columns, 128 rows, 1}
static int tok_map(CUtensorMap* m, const void* ptr, long batch, long tokens, long cols, long ld, long bs) {
  EncodeFn enc = encode_fn();
  if (!enc) return -1;
  if (batch == 1) bs = tokens * ld;      // a one-batch view may carry any batch stride
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)tokens, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)bs * 2};
  cuuint32_t box[3] = {64, 128, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

template <int DQK, int DV, int NQ>
static int run(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo, const Params& p, cudaStream_t st) {
  const int smem = NQ * 128 * DQK * 2 + 2 * 128 * DQK * 2 + 2 * 128 * DV * 2 + (int)sizeof(Ctl) + 4096 + 1024;
  static bool cfg = false;
  if (!cfg) {
    if (cudaFuncSetAttribute(flash_fwd_kernel<DQK, DV, NQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -2;
    cfg = true;
  }
  const long ctas = (long)p.n_pairs * p.Hq * p.B;
  flash_fwd_kernel<DQK, DV, NQ><<<(unsigned)ctas, 64 + 128 * NQ, smem, st>>>(mq, mk, mv, mo, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace fwd
}  // namespace mt

extern "C" {

// Shapes this kernel covers: (Dqk, Dv) in {(64,64), (128,128), (192,128)}.
int mt_flash_fwd_supported(int Dqk, int Dv) { return (Dqk == 64 && Dv == 64) || (Dqk == 128 && Dv == 128) || (Dqk == 192 && Dv == 128); }

// ints of scratch (`tiles`) that the attention kernels need when position arrays are given
long mt_attn_tile_ints(int B, int Sq, int Skv) { return 2l * B * ((Sq + 127) / 128 + (Skv + 127) / 128); }

// (min, max) position of every 128-token tile of pos [B, S] -> out [B, ceil(S/128), 2]
void mt_attn_tile_minmax(const int* pos, int B, int S, int* out, cudaStream_t st) {
  const int nt = (S + 127) / 128;
  mt::fwd::tile_minmax_kernel<<<(B * nt * 32 + 255) / 256, 256, 0, st>>>(pos, B, S, nt, out);
}

// q/k/v/out: token-major views; ld* = row stride, bs* = batch stride (elements). seg_q/seg_k, pos_q/pos_k, sinks may be null;
// pos_q and pos_k come together and need `tiles` (mt_flash_fwd_tile_ints ints of scratch).
int mt_flash_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* seg_q, const int* seg_k, const int* pos_q,
                 const int* pos_k, int* tiles, const float* sinks, int B, int Sq, int Skv, int Hq, int Hkv, int Dqk, int Dv, long ldq, long bsq,
                 long ldk, long bsk, long ldv, long bsv, long ldo, long bso, float scale, float softcap, int causal, int window, int chunk,
                 int q_off, int* status, cudaStream_t st) {
  using namespace mt::fwd;
  if (!mt_flash_fwd_supported(Dqk, Dv) || Hq % Hkv || Sq < 1 || Skv < 1 || (pos_q == nullptr) != (pos_k == nullptr) ||
      (seg_q == nullptr) != (seg_k == nullptr) || (pos_q && !tiles))
    return -1;
  CUtensorMap mq, mk, mv, mo;
  if (tok_map(&mq, q, B, Sq, (long)Hq * Dqk, ldq, bsq) || tok_map(&mk, k, B, Skv, (long)Hkv * Dqk, ldk, bsk) ||
      tok_map(&mv, v, B, Skv, (long)Hkv * Dv, ldv, bsv) || tok_map(&mo, out, B, Sq, (long)Hq * Dv, ldo, bso))
    return -3;
  const int nq = Dqk == 192 ? 1 : 2;
  Params p{};
  p.B = B; p.Hq = Hq; p.Hkv = Hkv;
  p.n_pairs = (Sq + 128 * nq - 1) / (128 * nq);
  p.scale = scale; p.softcap = softcap; p.sinks = sinks; p.lse = lse; p.status = status;
  p.head_major = 0;                       // tile-major: longest query tiles of every head first
  mt::attn::Mask& msk = p.mk;
  msk.Sq = Sq; msk.Skv = Skv; msk.n_qt = (Sq + 127) / 128; msk.n_kt = (Skv + 127) / 128;
  msk.q_off = q_off; msk.causal = causal; msk.window = window; msk.chunk = chunk;
  msk.seg_q = seg_q; msk.seg_k = seg_k; msk.pos_q = pos_q; msk.pos_k = pos_k;
  if (pos_q) {
    mt_attn_tile_minmax(pos_q, B, Sq, tiles, st);
    mt_attn_tile_minmax(pos_k, B, Skv, tiles + 2l * B * msk.n_qt, st);
    msk.tile_q = tiles;
    msk.tile_k = tiles + 2l * B * msk.n_qt;
  }
  if (Dqk == 128) return run<128, 128, 2>(mq, mk, mv, mo, p, st);
  if (Dqk == 64) return run<64, 64, 2>(mq, mk, mv, mo, p, st);
  return run<192, 128, 1>(mq, mk, mv, mo, p, st);
}

}  // extern "C"
