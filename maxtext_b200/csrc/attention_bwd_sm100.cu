// Flash attention backward for sm_100a: deterministic (no atomics), two software-pipelined kernels.
//
//   delta = rowsum(dO * O)                                  (small pre-pass)
//   kernel A, CTA = 128 keys of one kv head, K and V resident in shared memory. It walks the query heads
//     of its GQA group and the 128-query tiles that can see its keys (Q / dO tiles double buffered):
//        S^T = K Q^T, dP^T = V dO^T  (128 x 128 fp32 in TMEM)
//        P^T = exp(S^T - lse), dS^T = scale * P^T * (dP^T - delta)  -> bf16, written back into TMEM
//        dV += P^T dO, dK += dS^T Q  (TMEM operands, accumulators stay in TMEM until the end)
//     The MMA warp interleaves the next tile's S^T / dP^T between dV and dK, so the 256 softmax threads and the
//     tensor core work at the same time.
//   kernel B, CTA = 128 queries of one head, Q and dO resident, K / V tiles double buffered:
//        S = Q K^T, dP = dO V^T, dS = scale * P * (dP - delta) -> TMEM, dQ += dS K.
// P is recomputed from the saved log-sum-exp in both kernels (sink logits only enter through it). Masks are those of
// the forward kernel (attention_mask.cuh): causal, sliding window, chunks, segment ids, positions from indices or arrays,
// ragged sequence lengths (TMA zero-fills loads and clips stores), different query and key lengths; a logit soft-cap
// multiplies dS by 1 - tanh^2. All waits are bounded; a timeout sets the status word.
//
// Both kernels are templates over (DQK, DV, NT): head dims of Q/K and of V/O, and the row count of the streamed tiles. Equal head
// dims of 64 or 128 stream 128-row tiles. Multi-head latent attention (DQK 192, DV 128) streams 64-row tiles: the resident
// tiles, two stages of streamed ones and the accumulators (dV 128 + dK 192 columns, or dQ 192) then fit 227 KB of shared memory
// and the 512 columns of tensor memory.
#include "attention_mask.cuh"
#include "sm100_ptx.cuh"
#include <cuda_bf16.h>
#include <type_traits>

namespace mt {
namespace bwd {

constexpr int THREADS = 320;        // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2..9: softmax / epilogue
constexpr int SM_THREADS = 256;
constexpr float LOG2E = 1.4426950408889634f;

struct Params {
  int B, Hq, Hkv;
  attn::Mask mk;
  float scale;
  float softcap;         // 0 = none
  const float* lse;      // [B,Hq,Sq]
  const float* delta;    // [B,Hq,Sq]
  int* status;
};

__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// [R x D] tile held as D/64 boxes {64 cols, R rows} (R * 128 bytes each)
template <int R>
__device__ __forceinline__ uint64_t big_kmajor(uint32_t tile, int k) { return make_smem_desc(tile + (k >> 2) * (R * 128) + (k & 3) * 32, 16, 1024); }
// the same tile read with its R rows as the contraction index and d as N (MN-major): 16 rows = 2048 B per k-step
template <int R>
__device__ __forceinline__ uint64_t big_mnmajor(uint32_t tile, int k) { return make_smem_desc(tile + k * 2048, R * 128, 1024); }
// TMEM column of k-step k (16 of NT contraction indices) of a bf16 operand written by two groups of threads: the group that owns
// indices [h * NT/2, (h + 1) * NT/2) packs them into NT/4 columns starting at column h * NT/2 of the fp32 tile it replaces
template <int NT>
__device__ __forceinline__ uint32_t tmem_a_col(int k) { return (uint32_t)((k / (NT / 32)) * (NT / 2) + (k % (NT / 32)) * 8); }

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
// zeros in place of stage_rows_bf16 (a tile whose accumulator was never written)
__device__ __forceinline__ void stage_rows_zero(uint32_t box, int row, int c) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int chunk = (c & 1) * 4 + j;
    const uint32_t dst = box + row * 128 + ((chunk ^ (row & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
  }
}

// ================================================================================================ delta
// delta[b,h,s] = sum_d dout[b,s,h,d] * out[b,s,h,d] for contiguous [B,S,H,D] tensors; one warp per (b,s,h)
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
//
// The work list of a CTA is the sequence of (query head of the group, query tile) pairs whose tile pair is not fully
// masked, in a fixed order that the producer, the MMA issuer and the softmax threads each derive for themselves.
// A 128-query tile is visited as SUBS pieces of 128 / SUBS rows (q0 = first row of the piece), all of the tile's class.
template <int SUBS>
struct QueryWalk {
  const attn::Mask& mk;
  attn::Span ks;
  int b, G, qt_lo, qt_hi, g, qt, sub, cls, q0;
  __device__ QueryWalk(const attn::Mask& m, const attn::Span& k, int b_, int G_, int lo, int hi)
      : mk(m), ks(k), b(b_), G(G_), qt_lo(lo), qt_hi(hi), g(0), qt(lo - 1), sub(SUBS - 1), cls(0), q0(0) {}
  // advances to the next piece that takes part; returns its class (1 unmasked, 2 mixed) or 0 at the end
  __device__ __forceinline__ int next() {
    if (qt_hi <= qt_lo) return 0;
    if (SUBS > 1 && cls && ++sub < SUBS) { q0 += 128 / SUBS; return cls; }
    for (;;) {
      if (++qt >= qt_hi) { qt = qt_lo; if (++g >= G) return cls = 0; }
      cls = attn::classify(mk, attn::q_span(mk, b, qt), ks);
      if (cls) { sub = 0; q0 = qt * 128; return cls; }
    }
  }
};

template <int DQK, int DV, int NT>
__global__ void __launch_bounds__(THREADS, 1)
dkv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
           const __grid_constant__ CUtensorMap map_do, const __grid_constant__ CUtensorMap map_dk, const __grid_constant__ CUtensorMap map_dv,
           const __grid_constant__ Params p) {
  constexpr int RES_K = 128 * DQK * 2, RES_V = 128 * DV * 2;          // resident K / V tiles
  constexpr int ST_Q = NT * DQK * 2, ST_DO = NT * DV * 2, STG = ST_Q + ST_DO;   // one stage: Q piece then dO piece
  constexpr int BOX = NT * 128;                                        // bytes of one {64 columns, NT rows} box of a stage
  constexpr int NBQ = DQK / 64, NBV = DV / 64;
  constexpr int HC = NT / 2;                                           // query columns per softmax thread
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_ST = 0, COL_DPT = NT, COL_DV = 2 * NT, COL_DK = 2 * NT + DV;
  static_assert(2 * NT + DV + DQK <= 512 && 2 * STG >= RES_K + RES_V, "accumulators / staging do not fit");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sK = base, sV = base + RES_K, sStage = base + RES_K + RES_V;
  Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + (base - smem_u32(smem_raw)) + RES_K + RES_V + 2 * STG);
  float* s_lse = reinterpret_cast<float*>(ctl + 1);      // [2][NT], pre-multiplied by log2(e); +inf for queries beyond Sq
  float* s_delta = s_lse + 256;                          // [2][NT]
  int* s_seg = reinterpret_cast<int*>(s_delta + 256);    // [2][NT] query segment ids
  int* s_pos = s_seg + 256;                              // [2][NT] query positions (array mode)
  const uint32_t bar0 = smem_u32(&ctl->bars[0]);
  enum { KV_FULL = 0, Q_FULL0, Q_FULL1, Q_EMPTY0, Q_EMPTY1, ST_FULL, DP_FULL, P_READY, DS_READY, ACC_FULL };
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const attn::Mask& mk = p.mk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Head-major order: the CTAs that run at the same time work on few (batch, head) pairs, so the Q / dO tiles they all
  // stream stay in L2. Within a head the key tiles ascend: under a causal mask the first ones see the most queries.
  const int kt = (int)(blockIdx.x % mk.n_kt);
  const int hk = (int)(blockIdx.x / mk.n_kt) % p.Hkv, b = (int)(blockIdx.x / mk.n_kt) / p.Hkv;
  const int G = p.Hq / p.Hkv;
  const int k0 = kt * 128;
  const attn::Span ks = attn::k_span(mk, b, kt);
  int qt_lo, qt_hi;
  attn::q_tiles_for(mk, ks, qt_lo, qt_hi);

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
      mbar_arrive_expect_tx(bar(KV_FULL), RES_K + RES_V);
#pragma unroll
      for (int j = 0; j < NBQ; ++j) tma_load_3d(sK + j * 16384, &map_k, bar(KV_FULL), hk * DQK + j * 64, k0, b);
#pragma unroll
      for (int j = 0; j < NBV; ++j) tma_load_3d(sV + j * 16384, &map_v, bar(KV_FULL), hk * DV + j * 64, k0, b);
      QueryWalk<128 / NT> w(mk, ks, b, G, qt_lo, qt_hi);
      for (int it = 0; w.next(); ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int h = hk * G + w.g;
        const int q0 = w.q0;
        if (!mbar_wait(bar(Q_EMPTY0 + s), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_arrive_expect_tx(bar(Q_FULL0 + s), STG);
        const uint32_t sq = sStage + s * STG, sdo = sq + ST_Q;
#pragma unroll
        for (int j = 0; j < NBQ; ++j) tma_load_3d(sq + j * BOX, &map_q, bar(Q_FULL0 + s), h * DQK + j * 64, q0, b);
#pragma unroll
        for (int j = 0; j < NBV; ++j) tma_load_3d(sdo + j * BOX, &map_do, bar(Q_FULL0 + s), h * DV + j * 64, q0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_nt = make_idesc_bf16(128, NT, false, false);    // [128 kv x d] . [NT q x d]^T
      constexpr uint32_t idesc_dv = make_idesc_bf16(128, DV, false, true);     // TMEM [128 kv x NT q] . [NT q x d]
      constexpr uint32_t idesc_dk = make_idesc_bf16(128, DQK, false, true);
      auto stage_q = [&](int it) { return sStage + (it & 1) * STG; };
      auto issue_st = [&](int it) {
#pragma unroll
        for (int k = 0; k < DQK / 16; ++k) umma_f16_ss(tmem + COL_ST, big_kmajor<128>(sK, k), big_kmajor<NT>(stage_q(it), k), idesc_nt, k != 0);
        umma_commit(bar(ST_FULL));
      };
      auto issue_dpt = [&](int it) {
#pragma unroll
        for (int k = 0; k < DV / 16; ++k)
          umma_f16_ss(tmem + COL_DPT, big_kmajor<128>(sV, k), big_kmajor<NT>(stage_q(it) + ST_Q, k), idesc_nt, k != 0);
        umma_commit(bar(DP_FULL));
      };
      QueryWalk<128 / NT> w(mk, ks, b, G, qt_lo, qt_hi);
      bool more = w.next() != 0;
      bool ok = mbar_wait(bar(KV_FULL), 0, abort_flag, p.status, ST_TIMEOUT_MMA);
      if (ok && more) {
        ok = mbar_wait(bar(Q_FULL0), 0, abort_flag, p.status, ST_TIMEOUT_MMA);
        if (ok) { tc_fence_after(); issue_st(0); issue_dpt(0); }
      }
      for (int it = 0; more && ok; ++it) {
        const uint32_t ph = it & 1;
        const bool next = w.next() != 0;
        if (!mbar_wait(bar(P_READY), ph, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < NT / 16; ++k)
          umma_f16_ts(tmem + COL_DV, tmem + COL_ST + tmem_a_col<NT>(k), big_mnmajor<NT>(stage_q(it) + ST_Q, k), idesc_dv, (it | k) != 0);
        if (next) {
          if (!mbar_wait(bar(Q_FULL0 + ((it + 1) & 1)), ((it + 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
          tc_fence_after();
          issue_st(it + 1);        // overwrites P^T_it only after dV_it (issued above) has consumed it: MMAs retire in order
        }
        if (!mbar_wait(bar(DS_READY), ph, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < NT / 16; ++k)
          umma_f16_ts(tmem + COL_DK, tmem + COL_DPT + tmem_a_col<NT>(k), big_mnmajor<NT>(stage_q(it), k), idesc_dk, (it | k) != 0);
        umma_commit(bar(Q_EMPTY0 + (it & 1)));
        if (next) issue_dpt(it + 1);
        else umma_commit(bar(ACC_FULL));
        more = next;
      }
    }
  } else {
    // ---------------------------------------------------------------- 256 softmax threads: (key row, half of the query columns)
    const int sw = warp - 2;                    // 0..7
    const int qd = warp & 3;                    // TMEM lane quarter this warp may touch
    const int half = sw >> 2;                   // which HC of the NT query columns
    const int row = qd * 32 + lane;             // key row
    const int et = threadIdx.x - 64;            // 0..255
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const bool cap = p.softcap > 0.f;
    const float a = cap ? p.softcap * LOG2E : p.scale * LOG2E;
    const float pre = cap ? p.scale / p.softcap : 1.f;
    const bool has_seg = mk.seg_q != nullptr;
    const bool arrays = mk.pos_q != nullptr;
    const int kg = k0 + row;
    const bool key_ok = row < ks.rows;
    const int my_seg = has_seg ? (key_ok ? mk.seg_k[(long)b * mk.Skv + kg] : 0) : 1;
    const int kpos = arrays ? (key_ok ? mk.pos_k[(long)b * mk.Skv + kg] : 0) : kg;
    // query positions that may attend to this key, as a closed interval
    int lo_p, hi_p;
    attn::query_interval(mk, kpos, lo_p, hi_p);
    const uint32_t span = (uint32_t)hi_p - (uint32_t)lo_p;
    const bool none = hi_p < lo_p || !key_ok;
    bool ok = true;
    int n_done = 0;
    QueryWalk<128 / NT> w(mk, ks, b, G, qt_lo, qt_hi);
    for (int it = 0;; ++it) {
      const int cls = w.next();
      if (!cls) break;
      n_done = it + 1;
      const int s = it & 1;
      const uint32_t ph = it & 1;
      const int h = hk * G + w.g;
      const int q0 = w.q0;
      if (et < NT) {
        const int qi = q0 + et;
        const bool q_ok = qi < mk.Sq;
        const long idx = ((long)b * p.Hq + h) * mk.Sq + qi;
        s_lse[s * NT + et] = q_ok ? p.lse[idx] * LOG2E : INFINITY;     // queries beyond the sequence get probability 0
        s_delta[s * NT + et] = q_ok ? p.delta[idx] : 0.f;
        if (has_seg) s_seg[s * NT + et] = q_ok ? mk.seg_q[(long)b * mk.Sq + qi] : 0;
        if (arrays) s_pos[s * NT + et] = q_ok ? mk.pos_q[(long)b * mk.Sq + qi] : INT_MAX;
      }
      // One thread waits for the MMAs; its verdict is sticky. A failed CTA keeps meeting at the named barriers
      // (so nobody is left waiting there) but does no further tensor-memory work.
      if (et == 128 && !mbar_wait(bar(ST_FULL), ph, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ctl->ok_flag = 0;
      named_bar_sync(1, SM_THREADS);
      if (*reinterpret_cast<volatile int*>(&ctl->ok_flag) == 0) ok = false;
      const bool need_mask = cls == 2;
      const float* lse_s = s_lse + s * NT + half * HC;
      const float* del_s = s_delta + s * NT + half * HC;
      const int* seg_s = s_seg + s * NT + half * HC;
      const int* pos_s = s_pos + s * NT + half * HC;
      // index mode: query column e of this half has position q0 + half*HC + e + q_off
      const uint32_t e_lo = (uint32_t)lo_p - (uint32_t)(q0 + half * HC + mk.q_off);
      float pr[HC];      // what multiplies (dP - delta): P, or P * (1 - tanh^2) under a soft-cap
      // the soft-cap and the mask are compile-time switches of this loop, so the common case stays three instructions per score
      auto phase1 = [&](auto cap_t, auto mask_t) {
        constexpr bool CAP = decltype(cap_t)::value, MASK = decltype(mask_t)::value;
#pragma unroll
        for (int c = 0; c < HC / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem + lane_off + COL_ST + half * HC + c * 32, r);
          tmem_ld_wait();
          float pv[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int col = c * 32 + e;
            float sv = __uint_as_float(r[e]);
            float dt = 1.f;
            if constexpr (CAP) { sv = fast_tanh(sv * pre); dt = 1.f - sv * sv; }
            float v = fast_exp2(fmaf(a, sv, -lse_s[col]));
            if constexpr (MASK) {
              bool keep = arrays ? ((uint32_t)pos_s[col] - (uint32_t)lo_p <= span) : ((uint32_t)col - e_lo <= span);
              if (has_seg) keep = keep && seg_s[col] == my_seg && my_seg != 0;
              if (!keep || none) v = 0.f;
            }
            pv[e] = v;
            pr[col] = CAP ? v * dt : v;
          }
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = pack_bf16(pv[2 * e], pv[2 * e + 1]);
          // P^T of this thread's HC queries: HC/2 packed columns at the start of its own HC score columns, so the two
          // halves never write over each other's unread scores
          tmem_st_32x32b_x16(tmem + lane_off + COL_ST + half * HC + c * 16, pk);
        }
      };
      if (ok) {
        tc_fence_after();
        if (cap) phase1(std::true_type{}, std::true_type{});
        else if (need_mask) phase1(std::false_type{}, std::true_type{});
        else phase1(std::false_type{}, std::false_type{});
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
      for (int c = 0; c < HC / 32; ++c) {
        uint32_t d[32];
        tmem_ld_32x32b_x32(tmem + lane_off + COL_DPT + half * HC + c * 32, d);
        tmem_ld_wait();
        uint32_t dk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int col = c * 32 + 2 * e;
          const float d0 = pr[col] * (__uint_as_float(d[2 * e]) - del_s[col]) * p.scale;
          const float d1 = pr[col + 1] * (__uint_as_float(d[2 * e + 1]) - del_s[col + 1]) * p.scale;
          dk[e] = pack_bf16(d0, d1);
        }
        tmem_st_32x32b_x16(tmem + lane_off + COL_DPT + half * HC + c * 16, dk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar(DS_READY));
    }
    if (et == 0 && ok && !mbar_wait(bar(n_done > 0 ? ACC_FULL : KV_FULL), 0, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ctl->ok_flag = 0;
    named_bar_sync(1, SM_THREADS);
    ok = *reinterpret_cast<volatile int*>(&ctl->ok_flag) != 0;
    if (ok && ks.rows > 0) {
      tc_fence_after();
      // all MMAs have retired: the Q/dO stages become the staging area, dV first then dK (zeros when no query sees these keys)
      for (int c = half; c < DV / 32; c += 2) {
        if (n_done > 0) stage_rows_bf16(tmem + lane_off + COL_DV + c * 32, sStage + (c >> 1) * 16384, row, c);
        else stage_rows_zero(sStage + (c >> 1) * 16384, row, c);
      }
      for (int c = half; c < DQK / 32; c += 2) {
        if (n_done > 0) stage_rows_bf16(tmem + lane_off + COL_DK + c * 32, sStage + NBV * 16384 + (c >> 1) * 16384, row, c);
        else stage_rows_zero(sStage + NBV * 16384 + (c >> 1) * 16384, row, c);
      }
      fence_proxy_async_smem();
    }
    named_bar_sync(2, SM_THREADS);
    if (ok && ks.rows > 0 && et == 0) {
#pragma unroll
      for (int j = 0; j < NBV; ++j) tma_store_3d(&map_dv, sStage + j * 16384, hk * DV + j * 64, k0, b);
#pragma unroll
      for (int j = 0; j < NBQ; ++j) tma_store_3d(&map_dk, sStage + NBV * 16384 + j * 16384, hk * DQK + j * 64, k0, b);
      tma_commit_group();
      tma_wait_group<0>();
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
// A 128-key tile is visited as SUBS pieces of 128 / SUBS rows (k0 = first row of the piece), all of the tile's class.
template <int SUBS>
struct KeyWalk {
  const attn::Mask& mk;
  attn::Span qs;
  int b, kt_hi, kt, sub, cls, k0;
  __device__ KeyWalk(const attn::Mask& m, const attn::Span& q, int b_, int lo, int hi)
      : mk(m), qs(q), b(b_), kt_hi(hi), kt(lo - 1), sub(SUBS - 1), cls(0), k0(0) {}
  // advances to the next piece that takes part; returns its class (1 unmasked, 2 mixed) or 0 at the end
  __device__ __forceinline__ int next() {
    if (SUBS > 1 && cls && ++sub < SUBS) { k0 += 128 / SUBS; return cls; }
    while (++kt < kt_hi) {
      cls = attn::classify(mk, qs, attn::k_span(mk, b, kt));
      if (cls) { sub = 0; k0 = kt * 128; return cls; }
    }
    return cls = 0;
  }
};

template <int DQK, int DV, int NT>
__global__ void __launch_bounds__(THREADS, 1)
dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
          const __grid_constant__ CUtensorMap map_do, const __grid_constant__ CUtensorMap map_dq, const __grid_constant__ Params p) {
  constexpr int RES_Q = 128 * DQK * 2, RES_DO = 128 * DV * 2;         // resident Q / dO tiles
  constexpr int ST_K = NT * DQK * 2, ST_V = NT * DV * 2, STG = ST_K + ST_V;     // one stage: K piece then V piece
  constexpr int BOX = NT * 128;
  constexpr int NBQ = DQK / 64, NBV = DV / 64;
  constexpr int HC = NT / 2;                                           // key columns per softmax thread
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0, COL_DP = NT, COL_DQ = 2 * NT;
  static_assert(2 * NT + DQK <= 512 && 2 * STG >= RES_Q, "accumulator / staging do not fit");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sDO = base + RES_Q, sStage = base + RES_Q + RES_DO;
  Ctl* ctl = reinterpret_cast<Ctl*>(smem_raw + (base - smem_u32(smem_raw)) + RES_Q + RES_DO + 2 * STG);
  int* s_seg = reinterpret_cast<int*>(ctl + 1);          // [2][NT] key segment ids
  int* s_pos = s_seg + 256;                              // [2][NT] key positions (array mode)
  const uint32_t bar0 = smem_u32(&ctl->bars[0]);
  enum { Q_FULL = 0, KV_FULL0, KV_FULL1, KV_EMPTY0, KV_EMPTY1, S_FULL, DP_FULL, S_DONE, DS_READY, ACC_FULL };
  auto bar = [&](int i) { return bar0 + 8u * i; };

  const attn::Mask& mk = p.mk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Head-major order (the K / V tiles that concurrent CTAs stream stay in L2); within a head the heaviest query tiles
  // first: under a causal mask the last ones see the most keys.
  const int qt = mk.n_qt - 1 - (int)(blockIdx.x % mk.n_qt);
  const int h = (int)(blockIdx.x / mk.n_qt) % p.Hq, b = (int)(blockIdx.x / mk.n_qt) / p.Hq;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qt * 128;
  const attn::Span qs = attn::q_span(mk, b, qt);
  int kt_lo, kt_hi;
  attn::k_tiles_for(mk, qs, kt_lo, kt_hi);

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
      mbar_arrive_expect_tx(bar(Q_FULL), RES_Q + RES_DO);
#pragma unroll
      for (int j = 0; j < NBQ; ++j) tma_load_3d(sQ + j * 16384, &map_q, bar(Q_FULL), h * DQK + j * 64, q0, b);
#pragma unroll
      for (int j = 0; j < NBV; ++j) tma_load_3d(sDO + j * 16384, &map_do, bar(Q_FULL), h * DV + j * 64, q0, b);
      KeyWalk<128 / NT> w(mk, qs, b, kt_lo, kt_hi);
      for (int it = 0; w.next(); ++it) {
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        const int kk = w.k0;
        if (!mbar_wait(bar(KV_EMPTY0 + s), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_PRODUCER)) break;
        mbar_arrive_expect_tx(bar(KV_FULL0 + s), STG);
        const uint32_t sk = sStage + s * STG, sv = sk + ST_K;
#pragma unroll
        for (int j = 0; j < NBQ; ++j) tma_load_3d(sk + j * BOX, &map_k, bar(KV_FULL0 + s), hk * DQK + j * 64, kk, b);
#pragma unroll
        for (int j = 0; j < NBV; ++j) tma_load_3d(sv + j * BOX, &map_v, bar(KV_FULL0 + s), hk * DV + j * 64, kk, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_nt = make_idesc_bf16(128, NT, false, false);
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, DQK, false, true);
      auto stage_k = [&](int it) { return sStage + (it & 1) * STG; };
      auto issue_s = [&](int it) {
#pragma unroll
        for (int k = 0; k < DQK / 16; ++k) umma_f16_ss(tmem + COL_S, big_kmajor<128>(sQ, k), big_kmajor<NT>(stage_k(it), k), idesc_nt, k != 0);
        umma_commit(bar(S_FULL));
      };
      auto issue_dp = [&](int it) {
#pragma unroll
        for (int k = 0; k < DV / 16; ++k)
          umma_f16_ss(tmem + COL_DP, big_kmajor<128>(sDO, k), big_kmajor<NT>(stage_k(it) + ST_K, k), idesc_nt, k != 0);
        umma_commit(bar(DP_FULL));
      };
      KeyWalk<128 / NT> w(mk, qs, b, kt_lo, kt_hi);
      bool more = w.next() != 0;
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag, p.status, ST_TIMEOUT_MMA);
      if (ok && more) {
        ok = mbar_wait(bar(KV_FULL0), 0, abort_flag, p.status, ST_TIMEOUT_MMA);
        if (ok) { tc_fence_after(); issue_s(0); issue_dp(0); }
      }
      for (int it = 0; more && ok; ++it) {
        const uint32_t ph = it & 1;
        const bool next = w.next() != 0;
        if (next) {
          // the score buffer is free as soon as the softmax threads have read it
          if (!mbar_wait(bar(S_DONE), ph, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
          if (!mbar_wait(bar(KV_FULL0 + ((it + 1) & 1)), ((it + 1) >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
          tc_fence_after();
          issue_s(it + 1);
        }
        if (!mbar_wait(bar(DS_READY), ph, abort_flag, p.status, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < NT / 16; ++k)
          umma_f16_ts(tmem + COL_DQ, tmem + COL_DP + tmem_a_col<NT>(k), big_mnmajor<NT>(stage_k(it), k), idesc_acc, (it | k) != 0);
        umma_commit(bar(KV_EMPTY0 + (it & 1)));
        if (next) issue_dp(it + 1);
        else umma_commit(bar(ACC_FULL));
        more = next;
      }
    }
  } else {
    const int sw = warp - 2;
    const int qd = warp & 3;
    const int half = sw >> 2;                   // which HC of the NT key columns
    const int row = qd * 32 + lane;             // query row
    const int et = threadIdx.x - 64;
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const bool cap = p.softcap > 0.f;
    const float a = cap ? p.softcap * LOG2E : p.scale * LOG2E;
    const float pre = cap ? p.scale / p.softcap : 1.f;
    const bool has_seg = mk.seg_q != nullptr;
    const bool arrays = mk.pos_k != nullptr;
    const int qg = q0 + row;
    const bool row_ok = row < qs.rows;
    const int my_seg = has_seg ? (row_ok ? mk.seg_q[(long)b * mk.Sq + qg] : 0) : 1;
    const int qpos = mk.pos_q ? (row_ok ? mk.pos_q[(long)b * mk.Sq + qg] : 0) : qg + mk.q_off;
    int lo_p, hi_p;
    attn::key_interval(mk, qpos, lo_p, hi_p);
    const uint32_t span = (uint32_t)hi_p - (uint32_t)lo_p;
    const bool none = hi_p < lo_p;
    const long sidx = ((long)b * p.Hq + h) * mk.Sq + qg;
    const float my_lse = row_ok ? p.lse[sidx] * LOG2E : INFINITY;      // rows beyond the sequence get probability 0
    const float my_delta = row_ok ? p.delta[sidx] : 0.f;
    bool ok = true;
    int n_done = 0;
    KeyWalk<128 / NT> w(mk, qs, b, kt_lo, kt_hi);
    for (int it = 0;; ++it) {
      const int cls = w.next();
      if (!cls) break;
      n_done = it + 1;
      const int s = it & 1;
      const uint32_t ph = it & 1;
      const int kk = w.k0;
      if (et < NT && cls == 2) {
        const int ki = kk + et;
        if (has_seg) s_seg[s * NT + et] = ki < mk.Skv ? mk.seg_k[(long)b * mk.Skv + ki] : 0;
        if (arrays) s_pos[s * NT + et] = ki < mk.Skv ? mk.pos_k[(long)b * mk.Skv + ki] : INT_MAX;
      }
      if (et == 128 && !mbar_wait(bar(S_FULL), ph, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ctl->ok_flag = 0;
      named_bar_sync(1, SM_THREADS);
      if (*reinterpret_cast<volatile int*>(&ctl->ok_flag) == 0) ok = false;
      const bool need_mask = cls == 2;
      const int* seg_s = s_seg + s * NT + half * HC;
      const int* pos_s = s_pos + s * NT + half * HC;
      const uint32_t e_lo = (uint32_t)lo_p - (uint32_t)(kk + half * HC);     // index mode: key column e of this half has position kk + half*HC + e
      float pr[HC];      // what multiplies (dP - delta): P, or P * (1 - tanh^2) under a soft-cap
      auto phase1 = [&](auto cap_t, auto mask_t) {
        constexpr bool CAP = decltype(cap_t)::value, MASK = decltype(mask_t)::value;
#pragma unroll
        for (int c = 0; c < HC / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem + lane_off + COL_S + half * HC + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int col = c * 32 + e;
            float sv = __uint_as_float(r[e]);
            float dt = 1.f;
            if constexpr (CAP) { sv = fast_tanh(sv * pre); dt = 1.f - sv * sv; }
            float v = fast_exp2(fmaf(a, sv, -my_lse));
            if constexpr (CAP) v *= dt;
            if constexpr (MASK) {
              bool keep = arrays ? ((uint32_t)pos_s[col] - (uint32_t)lo_p <= span) : ((uint32_t)col - e_lo <= span);
              if (has_seg) keep = keep && seg_s[col] == my_seg && my_seg != 0;
              if (!keep || none) v = 0.f;
            }
            pr[col] = v;
          }
        }
      };
      if (ok) {
        tc_fence_after();
        if (cap) phase1(std::true_type{}, std::true_type{});
        else if (need_mask) phase1(std::false_type{}, std::true_type{});
        else phase1(std::false_type{}, std::false_type{});
        tc_fence_before();
        mbar_arrive(bar(S_DONE));
      }
      if (et == 128 && ok && !mbar_wait(bar(DP_FULL), ph, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ctl->ok_flag = 0;
      named_bar_sync(2, SM_THREADS);
      if (*reinterpret_cast<volatile int*>(&ctl->ok_flag) == 0) ok = false;
      if (!ok) continue;
      tc_fence_after();
      uint32_t dk[HC / 2];
#pragma unroll
      for (int c = 0; c < HC / 32; ++c) {
        uint32_t d[32];
        tmem_ld_32x32b_x32(tmem + lane_off + COL_DP + half * HC + c * 32, d);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const int col = c * 32 + 2 * e;
          dk[c * 16 + e] = pack_bf16(pr[col] * (__uint_as_float(d[2 * e]) - my_delta) * p.scale,
                                     pr[col + 1] * (__uint_as_float(d[2 * e + 1]) - my_delta) * p.scale);
        }
      }
      // dS over this thread's own (already read) dP columns
      if constexpr (HC == 64) tmem_st_32x32b_x32(tmem + lane_off + COL_DP + half * HC, dk);
      else tmem_st_32x32b_x16(tmem + lane_off + COL_DP + half * HC, dk);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar(DS_READY));
    }
    if (et == 0 && ok && !mbar_wait(bar(n_done > 0 ? ACC_FULL : Q_FULL), 0, abort_flag, p.status, ST_TIMEOUT_EPILOGUE)) ctl->ok_flag = 0;
    named_bar_sync(1, SM_THREADS);
    ok = *reinterpret_cast<volatile int*>(&ctl->ok_flag) != 0;
    if (ok && qs.rows > 0) {
      tc_fence_after();
      for (int c = half; c < DQK / 32; c += 2) {
        if (n_done > 0) stage_rows_bf16(tmem + lane_off + COL_DQ + c * 32, sStage + (c >> 1) * 16384, row, c);
        else stage_rows_zero(sStage + (c >> 1) * 16384, row, c);          // no key is visible from these queries
      }
      fence_proxy_async_smem();
    }
    named_bar_sync(2, SM_THREADS);
    if (ok && qs.rows > 0 && et == 0) {
#pragma unroll
      for (int j = 0; j < NBQ; ++j) tma_store_3d(&map_dq, sStage + j * 16384, h * DQK + j * 64, q0, b);
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

// {heads*D, tokens, batch} view with row stride `ld` and batch stride `bs` (elements); box {64 columns, `rows` rows, 1}
static int tok_map(CUtensorMap* m, const void* ptr, long batch, long tokens, long cols, long ld, long bs, int rows = 128) {
  EncodeFn enc = encode_fn();
  if (!enc) return -1;
  if (batch == 1) bs = tokens * ld;      // a one-batch view may carry any batch stride
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)tokens, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)bs * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)rows, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

template <typename K>
static int set_smem(K kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess ? 0 : -2;
}

// Tensors of one call: resident tiles are loaded and results stored with 128-row boxes, streamed tiles with NT-row boxes.
struct Tensors {
  const void *q, *k, *v, *dout;
  void *dq, *dk, *dv;
  long ldq, bsq, ldk, bsk, ldv, bsv, lddq, bsdq, lddk, bsdk, lddv, bsdv;
};

template <int DQK, int DV, int NT>
static int run(const Tensors& t, const Params& p, cudaStream_t st) {
  const int B = p.B, Sq = p.mk.Sq, Skv = p.mk.Skv;
  const long cq = (long)p.Hq * DQK, ck = (long)p.Hkv * DQK, cvq = (long)p.Hq * DV, cvk = (long)p.Hkv * DV;
  CUtensorMap q_res, q_str, k_res, k_str, v_res, v_str, do_res, do_str, mdq, mdk, mdv;
  if (tok_map(&q_res, t.q, B, Sq, cq, t.ldq, t.bsq) || tok_map(&k_res, t.k, B, Skv, ck, t.ldk, t.bsk) ||
      tok_map(&v_res, t.v, B, Skv, cvk, t.ldv, t.bsv) || tok_map(&do_res, t.dout, B, Sq, cvq, cvq, (long)Sq * cvq) ||
      tok_map(&mdq, t.dq, B, Sq, cq, t.lddq, t.bsdq) || tok_map(&mdk, t.dk, B, Skv, ck, t.lddk, t.bsdk) ||
      tok_map(&mdv, t.dv, B, Skv, cvk, t.lddv, t.bsdv))
    return -3;
  if (NT == 128) {
    q_str = q_res; k_str = k_res; v_str = v_res; do_str = do_res;
  } else if (tok_map(&q_str, t.q, B, Sq, cq, t.ldq, t.bsq, NT) || tok_map(&k_str, t.k, B, Skv, ck, t.ldk, t.bsk, NT) ||
             tok_map(&v_str, t.v, B, Skv, cvk, t.ldv, t.bsv, NT) || tok_map(&do_str, t.dout, B, Sq, cvq, cvq, (long)Sq * cvq, NT)) {
    return -3;
  }
  const int smem = 128 * (DQK + DV) * 2 + 2 * NT * (DQK + DV) * 2 + (int)sizeof(Ctl) + 4096 + 1024;
  static bool cfg = false;
  if (!cfg) {
    if (set_smem(dkv_kernel<DQK, DV, NT>, smem) || set_smem(dq_kernel<DQK, DV, NT>, smem)) return -2;
    cfg = true;
  }
  dkv_kernel<DQK, DV, NT><<<(unsigned)((long)p.mk.n_kt * p.Hkv * p.B), THREADS, smem, st>>>(q_str, k_res, v_res, do_str, mdk, mdv, p);
  dq_kernel<DQK, DV, NT><<<(unsigned)((long)p.mk.n_qt * p.Hq * p.B), THREADS, smem, st>>>(q_res, k_str, v_str, do_res, mdq, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace bwd
}  // namespace mt

extern "C" void mt_attn_tile_minmax(const int* pos, int B, int S, int* out, cudaStream_t st);      // attention_fwd_sm100.cu

// Shapes the backward kernels cover: Dqk = Dv in {64, 128}, and multi-head latent attention's 192 / 128.
extern "C" int mt_flash_bwd_supported(int Dqk, int Dv) { return (Dqk == Dv && (Dqk == 64 || Dqk == 128)) || (Dqk == 192 && Dv == 128); }

// dout/out: contiguous [B,Sq,Hq,Dv]; delta: scratch [B,Hq,Sq] fp32; q/k/v and dq/dk/dv: token-major views with their own row (ld*) and
// batch (bs*) strides in elements. seg_*, pos_* may be null (pos_* need `tiles`, mt_attn_tile_ints ints of scratch).
extern "C" int mt_flash_bwd(const void* dout, const void* q, const void* k, const void* v, const void* out, const float* lse, float* delta,
                            void* dq, void* dk, void* dv, const int* seg_q, const int* seg_k, const int* pos_q, const int* pos_k, int* tiles,
                            int B, int Sq, int Skv, int Hq, int Hkv, int D, int Dv, long ldq, long bsq, long ldk, long bsk, long ldv, long bsv,
                            long lddq, long bsdq, long lddk, long bsdk, long lddv, long bsdv, float scale, float softcap, int causal, int window,
                            int chunk, int q_off, int* status, cudaStream_t st) {
  using namespace mt::bwd;
  if (!mt_flash_bwd_supported(D, Dv) || Hq % Hkv || Sq < 1 || Skv < 1 || (pos_q == nullptr) != (pos_k == nullptr) ||
      (seg_q == nullptr) != (seg_k == nullptr) || (pos_q && !tiles))
    return -1;
  {
    const long warps = (long)B * Sq * Hq;
    const int threads = 256;
    const long blocks = (warps * 32 + threads - 1) / threads;
    delta_kernel<<<(unsigned)blocks, threads, 0, st>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, delta, B, Sq, Hq, Dv);
  }
  Tensors t{q, k, v, dout, dq, dk, dv, ldq, bsq, ldk, bsk, ldv, bsv, lddq, bsdq, lddk, bsdk, lddv, bsdv};
  Params p{};
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.scale = scale; p.softcap = softcap; p.lse = lse; p.delta = delta; p.status = status;
  mt::attn::Mask& m = p.mk;
  m.Sq = Sq; m.Skv = Skv; m.n_qt = (Sq + 127) / 128; m.n_kt = (Skv + 127) / 128;
  m.q_off = q_off; m.causal = causal; m.window = window; m.chunk = chunk;
  m.seg_q = seg_q; m.seg_k = seg_k; m.pos_q = pos_q; m.pos_k = pos_k;
  if (pos_q) {
    mt_attn_tile_minmax(pos_q, B, Sq, tiles, st);
    mt_attn_tile_minmax(pos_k, B, Skv, tiles + 2l * B * m.n_qt, st);
    m.tile_q = tiles;
    m.tile_k = tiles + 2l * B * m.n_qt;
  }
  if (D == 192) return run<192, 128, 64>(t, p, st);
  if (D == 128) return run<128, 128, 128>(t, p, st);
  return run<64, 64, 128>(t, p, st);
}
