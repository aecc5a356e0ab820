// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared-memory ring -> tcgen05.mma with
// fp32 accumulators in tensor memory -> epilogue through shared memory and TMA stores.
//
//   C[M,N] (+)= op(A) * op(B)      op(A) is M x K, op(B) is K x N
//
// Operand storage (row-major, leading stride a multiple of 8 elements):
//   A "K-major"  : A[M,K]      A "MN-major": A[K,M]   (i.e. the transposed operand, no copy needed)
//   B "K-major"  : B[N,K]      B "MN-major": B[K,N]
// so the three products of a linear layer map to   fwd  y  = x  W^T : (A K-major,  B K-major)
//                                                  dX   dx = dy W   : (A K-major,  B MN-major)
//                                                  dW   dW = dy^T x : (A MN-major, B MN-major)
// Output is bf16 (plain store) or fp32 (plain store, or a TMA reduce-add when accumulating into an
// existing gradient buffer, which makes beta = 1 free of any read in the kernel).
//
// CTA layout (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2..5 =
// epilogue (each reads its own 32-lane quarter of tensor memory). One CTA per SM, grid = min(tiles,
// SMs); tiles are walked in groups of GROUP_M row-blocks so that concurrently running CTAs share A and
// B tiles in L2. Accumulators are double buffered in TMEM (2 x BN columns) so the epilogue of tile i
// overlaps the main loop of tile i+1. Every wait is bounded (see mbar_wait): on a timeout the kernel
// records a code in the status word, drains, frees its tensor memory and returns.
#include "sm100_ptx.cuh"
#include <cuda_bf16.h>

namespace mt {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int GROUP_M = 16;
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;

template <int BN>
struct GemmCfg {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_BYTES = 2 * BM * 128;  // two staging buffers of 128 rows x 128 B
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES + 1024;  // + alignment slack
  static constexpr int TMEM_COLS = 2 * BN;  // power of two >= 32
};

struct GemmParams {
  int M, N, K;
  int accumulate;  // fp32 output only: C += result (TMA reduce-add)
  int* status;
  // Fused FSDP all-gather (forward layout only, B = W[N,K] inside a flat parameter unit). When g_comm_ctas > 0 the
  // last g_comm_ctas CTAs of the launch copy the peers' shards of the whole unit into the local full buffer, one
  // segment at a time, publishing a flag per segment; the TMA producers of the other CTAs wait for the segments
  // that hold the rows of their B tile before loading it. Remote data is read with plain ld.global by the copier.
  int g_comm_ctas;
  int g_world;
  int g_segs_per_chunk;
  int g_first_seg;
  long g_chunk_vec;      // 16-byte vectors per rank chunk
  long g_seg_vec;        // 16-byte vectors per segment
  long g_chunk_elems;    // bf16 elements per rank chunk
  long g_seg_elems;
  long g_b_offset;       // element offset of W inside the unit
  const uint4* const* g_peer_shards;
  uint4* g_full;
  int* g_seg_flags;
  // Grouped (mixture-of-experts) products. Rows are grouped by expert and every group is padded to a multiple of BM
  // rows, so each 128-row block belongs to one expert: x_offs[e] is the first padded row of expert e (x_offs[E] = rows in
  // use, read on the device, so no host synchronisation is needed), x_blk_expert[mb] the expert of row block mb.
  //   1: y = x W_e^T      B = W [E*N, K] K-major, B tile rows start at e*N
  //   2: dx = dy W_e      B = W [E*Kc, N] MN-major, contraction rows start at e*Kc (Kc = p.K)
  //   3: dW_e = dy_e^T x_e  A = dy [R, x_nw] and B = x [R, N] MN-major, contraction over the rows of group e,
  //                          C = [E*x_nw, N] fp32; an empty group writes zeros (or nothing when accumulating)
  // Fused reduce-scatter of the output over a tensor-parallel group (fp32 output only): row block mb belongs to rank
  // (mb * BM) / r_rows; its tile is added into that rank's accumulation buffer (peer memory) by a TMA reduce-add through
  // r_maps[owner] (tensor maps in global memory, one per rank, each over a [r_rows, N] fp32 buffer).
  const CUtensorMap* r_maps;
  int r_rows;
  // 8-bit operands (FP8 template flag): formats per operand (0 = E4M3, 1 = E5M2) and the de-quantisation factors, read from
  // device memory so that scales derived from a running amax never visit the host. out = acc * (*q_scale_a) * (*q_scale_b).
  int raster_n;          // tile walk: 0 = groups of row blocks (A slice stays in L2, B streams), 1 = groups of column blocks
  int q_fmt_a, q_fmt_b;
  const float* q_scale_a;
  const float* q_scale_b;
  int x_mode;
  int x_experts;
  int x_nw;
  const int* x_offs;
  const int* x_blk_expert;
};

struct TileInfo {
  int a_m0, b_n0, c_m0, k0a, k0b, num_kb;
};

__device__ __forceinline__ TileInfo tile_info(const GemmParams& p, int mb, int nb, int BN, int num_kb_full) {
  TileInfo t{mb * BM, nb * BN, mb * BM, 0, 0, num_kb_full};
  if (p.x_mode == 1) {
    t.b_n0 += p.x_blk_expert[mb] * p.N;
  } else if (p.x_mode == 2) {
    t.k0b = p.x_blk_expert[mb] * p.K;
  } else if (p.x_mode == 3) {
    const int e = (mb * BM) / p.x_nw;
    t.a_m0 = mb * BM - e * p.x_nw;
    t.k0a = t.k0b = p.x_offs[e];
    t.num_kb = (p.x_offs[e + 1] - p.x_offs[e]) / BK;
  }
  return t;
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Wait (bounded) until every segment covering unit elements [lo, hi) has been published.
__device__ __forceinline__ bool wait_segments(const GemmParams& p, long lo, long hi, volatile int* abort_flag) {
  long e = lo;
  while (e < hi) {
    const long r = e / p.g_chunk_elems;
    const long j = (e - r * p.g_chunk_elems) / p.g_seg_elems;
    const int* f = p.g_seg_flags + r * p.g_segs_per_chunk + j;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (ld_acquire_gpu(f) == 0) {
      if ((++spins & 0xFF) == 0) {
        if (*abort_flag) return false;
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > 4000000000ull) {
          *abort_flag = 1;
          if (p.status) atomicCAS(p.status, 0, ST_TIMEOUT_FLAG);
          return false;
        }
      }
    }
    const long seg_end = r * p.g_chunk_elems + (j + 1) * p.g_seg_elems;
    const long chunk_end = (r + 1) * p.g_chunk_elems;
    e = seg_end < chunk_end ? seg_end : chunk_end;
  }
  asm volatile("fence.proxy.async.global;" ::: "memory");   // peer data was written with generic stores, TMA reads it next
  return true;
}

__device__ int g_group_m = GROUP_M;     // row blocks per tile group; set from the host (mt_gemm_set_group_m) for tuning runs

__device__ __forceinline__ void tile_coords(int t, int m_blocks, int n_blocks, int& mb, int& nb, int raster_n = 0) {
  if (raster_n) {        // the same walk with the roles of the two dimensions exchanged
    tile_coords(t, n_blocks, m_blocks, nb, mb, 0);
    return;
  }
  const int gm = g_group_m;
  const int per_group = gm * n_blocks;
  const int g = t / per_group;
  const int first_m = g * gm;
  const int gsz = min(gm, m_blocks - first_m);
  const int r = t - g * per_group;
  mb = first_m + (r % gsz);
  nb = r / gsz;
}

template <int BN, bool A_MN, bool B_MN, typename OutT, bool FP8 = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_a0 = smem_base;
  const uint32_t smem_b0 = smem_base + STAGES * Cfg::A_BYTES;
  const uint32_t smem_epi = smem_base + STAGES * Cfg::STAGE_BYTES;
  const uint32_t bar_base = smem_epi + Cfg::EPI_BYTES;
  // barrier slots (8 bytes each)
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
  const uint32_t abort_slot = tmem_slot + 8;
  uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + (tmem_slot - smem_base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + (abort_slot - smem_base));
  volatile int* epi_ok = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_blocks = (p.x_mode == 1 || p.x_mode == 2) ? p.x_offs[p.x_experts] / BM : (p.M + BM - 1) / BM;
  const int n_blocks = (p.N + BN - 1) / BN;
  const int num_tiles = m_blocks * n_blocks;
  constexpr int BKE = FP8 ? 2 * BK : BK;      // elements per 128-byte smem row: the byte layout of a stage is the same for both widths
  static_assert(!FP8 || (!A_MN && !B_MN), "8-bit operands are K-major only");
  const int num_kb = (p.K + BKE - 1) / BKE;
  const int cta_stride = (int)gridDim.x - p.g_comm_ctas;        // CTAs that compute tiles
  const bool is_comm_cta = (int)blockIdx.x >= cta_stride;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), EPI_THREADS);
    }
    fence_barrier_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    prefetch_tensormap(&map_c);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (is_comm_cta) {
    // ------------------------------------------------------------ all-gather copier (one thread drives the copy engine)
    // Peer shard -> shared memory -> local full buffer with untiled bulk copies (cp.async.bulk, per-CTA form), four
    // 48 KB pieces in flight per CTA, so NVLink latency is covered by bytes in flight rather than by threads.
    if (threadIdx.x == 0) {
      constexpr uint32_t PIECE = Cfg::STAGE_BYTES;          // the GEMM's smem ring doubles as the staging area
      const int n_segs = p.g_segs_per_chunk * p.g_world;
      const long seg_bytes = p.g_seg_vec * 16, chunk_bytes = p.g_chunk_vec * 16;
      uint32_t issued = 0, stored = 0;                      // pieces loaded / stored so far (ring position = count % STAGES)
      bool ok = true;
      // a piece in flight: where it goes and how long it is
      long pend_dst[STAGES];
      uint32_t pend_len[STAGES];
      auto store_one = [&]() {
        const uint32_t sidx = stored % STAGES;
        if (!mbar_wait(full_bar(sidx), (stored / STAGES) & 1, abort_flag, p.status, ST_TIMEOUT_FLAG)) { ok = false; return; }
        const uint64_t gdst = reinterpret_cast<uint64_t>(p.g_full) + (uint64_t)pend_dst[sidx];
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_a0 + sidx * PIECE),
                     "r"(pend_len[sidx]) : "memory");
        tma_commit_group();
        ++stored;
      };
      for (int k = (int)blockIdx.x - cta_stride; k < n_segs && ok; k += p.g_comm_ctas) {
        const int sgm = (p.g_first_seg + k) % n_segs;
        const int r = sgm / p.g_segs_per_chunk;
        const long lo = (long)(sgm % p.g_segs_per_chunk) * seg_bytes;
        const long hi = lo + seg_bytes < chunk_bytes ? lo + seg_bytes : chunk_bytes;
        const uint64_t src = reinterpret_cast<uint64_t>(p.g_peer_shards[r]);
        for (long off = lo; off < hi && ok; off += PIECE) {
          const uint32_t len = (uint32_t)(hi - off < (long)PIECE ? hi - off : (long)PIECE);
          if (issued - stored == STAGES) store_one();       // ring full: retire the oldest piece first
          if (!ok) break;
          const uint32_t sidx = issued % STAGES;
          if (issued >= STAGES) tma_wait_group_read<0>();            // the stage's previous store has finished reading smem
          mbar_arrive_expect_tx(full_bar(sidx), len);
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_a0 + sidx * PIECE),
                       "l"(src + (uint64_t)off), "r"(len), "r"(full_bar(sidx)) : "memory");
          pend_dst[sidx] = (long)r * chunk_bytes + off;
          pend_len[sidx] = len;
          ++issued;
        }
        while (ok && stored < issued) store_one();          // drain this segment, then publish it
        if (!ok) break;
        tma_wait_group<0>();
        __threadfence();
        atomicExch(p.g_seg_flags + sgm, 1);
      }
      tma_wait_group<0>();
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one thread)
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += cta_stride) {
        int mb, nb;
        tile_coords(t, m_blocks, n_blocks, mb, nb, p.raster_n);
        if (p.g_seg_flags) {
          const long n1 = (long)(nb + 1) * BN < p.N ? (long)(nb + 1) * BN : p.N;
          if (!wait_segments(p, p.g_b_offset + (long)nb * BN * p.K, p.g_b_offset + n1 * p.K, abort_flag)) { ok = false; break; }
        }
        const TileInfo ti = tile_info(p, mb, nb, BN, num_kb);
        for (int kb = 0; kb < ti.num_kb; ++kb) {
          if (!mbar_wait(empty_bar(s), phase ^ 1, abort_flag, p.status, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
          mbar_arrive_expect_tx(full_bar(s), Cfg::STAGE_BYTES);
          const uint32_t sa = smem_a0 + s * Cfg::A_BYTES;
          const uint32_t sb = smem_b0 + s * Cfg::B_BYTES;
          if (!A_MN) {
            tma_load_2d(sa, &map_a, full_bar(s), ti.k0a + kb * BKE, ti.a_m0);             // box {128 B of k, 128 m}
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)                                             // boxes {64 m, 64 k}
              tma_load_2d(sa + j * 8192, &map_a, full_bar(s), ti.a_m0 + j * 64, ti.k0a + kb * BK);
          }
          if (!B_MN) {
            tma_load_2d(sb, &map_b, full_bar(s), ti.k0b + kb * BKE, ti.b_n0);             // box {128 B of k, BN n}
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)                                             // boxes {64 n, 64 k}
              tma_load_2d(sb + j * 8192, &map_b, full_bar(s), ti.b_n0 + j * 64, ti.k0b + kb * BK);
          }
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      const uint32_t idesc = FP8 ? make_idesc_fp8(BM, BN, (uint32_t)p.q_fmt_a, (uint32_t)p.q_fmt_b) : make_idesc_bf16(BM, BN, A_MN, B_MN);
      constexpr uint32_t A_LBO = A_MN ? 8192 : 16, B_LBO = B_MN ? 8192 : 16;
      constexpr uint32_t A_KSTEP = A_MN ? 2048 : 32, B_KSTEP = B_MN ? 2048 : 32;  // bytes per UMMA_K
      int s = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += cta_stride) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, abort_flag, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        int tile_kb = num_kb;
        if (p.x_mode == 3) {
          int mb, nb;
          tile_coords(t, m_blocks, n_blocks, mb, nb, p.raster_n);
          tile_kb = tile_info(p, mb, nb, BN, num_kb).num_kb;
        }
        for (int kb = 0; kb < tile_kb; ++kb) {
          if (!mbar_wait(full_bar(s), phase, abort_flag, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint64_t da = make_smem_desc(smem_a0 + s * Cfg::A_BYTES, A_LBO, 1024);
          const uint64_t db = make_smem_desc(smem_b0 + s * Cfg::B_BYTES, B_LBO, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            if (FP8) umma_f8_ss(d_tmem, da + (uint64_t)((k * A_KSTEP) >> 4), db + (uint64_t)((k * B_KSTEP) >> 4), idesc,
                                (kb | k) != 0 ? 1u : 0u);
            else umma_f16_ss(d_tmem, da + (uint64_t)((k * A_KSTEP) >> 4), db + (uint64_t)((k * B_KSTEP) >> 4), idesc,
                             (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(s));   // frees the smem stage when these MMAs retire
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));   // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (128 threads)
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;          // row of the tile owned by this thread
    const int et = threadIdx.x - 64;        // 0..127 within the epilogue group
    constexpr bool OUT_F32 = sizeof(OutT) == 4;
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    bool ok = true;
    if (p.r_maps && et == 0) {
      // the owners' tensor maps live in global memory (written by the host before the launch): order them for the tensor-map proxy
      for (int r = 0; r < p.M / p.r_rows; ++r)
        asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(p.r_maps + r) : "memory");
    }
    for (int t = blockIdx.x; t < num_tiles && ok; t += cta_stride) {
      int mb, nb;
      tile_coords(t, m_blocks, n_blocks, mb, nb, p.raster_n);
      const bool empty_tile = p.x_mode == 3 && tile_info(p, mb, nb, BN, num_kb).num_kb == 0;   // nothing was accumulated
      // one thread waits, the verdict is shared so that all 128 threads leave the loop together
      if (et == 0) *epi_ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, ST_TIMEOUT_EPILOGUE) ? 1 : 0;
      named_bar_sync(3, EPI_THREADS);
      if (*epi_ok == 0) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_addr + c * 32, r);
        tmem_ld_wait();
        if (empty_tile) {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (FP8) {
          const float qs = __ldg(p.q_scale_a) * __ldg(p.q_scale_b);
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * qs);
        }
        if (c == BN / 32 - 1) {
          // whole accumulator is in registers: hand the TMEM buffer back to the MMA warp
          tc_fence_before();
          mbar_arrive(tempty_bar(acc));
        }
        const bool new_store = OUT_F32 ? true : ((c & 1) == 0);
        if (new_store) {
          // the staging buffer we are about to overwrite must have been read by its previous TMA store
          if (et == 0) tma_wait_group_read<1>();
          named_bar_sync(1, EPI_THREADS);
        }
        const uint32_t sbuf = smem_epi + buf * (BM * 128);
        if (OUT_F32) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {     // 8 chunks of 16 B (4 floats) per 128-byte row
            const uint32_t dst = sbuf + row * 128 + ((j ^ (row & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(r[4 * j]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]),
                         "r"(r[4 * j + 3])
                         : "memory");
          }
        } else {
          const int half = c & 1;           // which 32-column half of the 64-column store tile
#pragma unroll
          for (int j = 0; j < 4; ++j) {     // 4 chunks of 16 B (8 bf16)
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * e]), __uint_as_float(r[8 * j + 2 * e + 1]));
              pk[e] = *reinterpret_cast<uint32_t*>(&v);
            }
            const int chunk = half * 4 + j;
            const uint32_t dst = sbuf + row * 128 + ((chunk ^ (row & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3])
                         : "memory");
          }
        }
        const bool do_store = OUT_F32 ? true : ((c & 1) == 1);
        if (do_store) {
          fence_proxy_async_smem();
          named_bar_sync(2, EPI_THREADS);
          if (et == 0) {
            const int col0 = nb * BN + (OUT_F32 ? c * 32 : (c >> 1) * 64);
            if (col0 < p.N && !(empty_tile && p.accumulate)) {
              if (p.r_maps) {
                // fused reduce-scatter: fp32 tiles are added into the owner's accumulator, bf16 tiles are stored into the
                // owner's staging area for this source rank (plain stores; the owner sums the staged copies afterwards)
                const int owner = (mb * BM) / p.r_rows;
                if (OUT_F32) tma_reduce_add_2d(p.r_maps + owner, sbuf, col0, mb * BM - owner * p.r_rows);
                else tma_store_2d(p.r_maps + owner, sbuf, col0, mb * BM - owner * p.r_rows);
              } else if (OUT_F32 && p.accumulate) {
                tma_reduce_add_2d(&map_c, sbuf, col0, mb * BM);
              } else {
                tma_store_2d(&map_c, sbuf, col0, mb * BM);
              }
            }
            tma_commit_group();
          }
          buf ^= 1;
        }
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (et == 0) tma_wait_group<0>();
  }

  // ------------------------------------------------------------ teardown
  if (*abort_flag) {
    // a wait ran out: give in-flight bulk copies time to land before shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess || !ptr) return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] with leading stride `ld` elements; box = {box_cols, box_rows}, 128B swizzle.
static int make_map_2d(CUtensorMap* map, const void* ptr, CUtensorMapDataType dt, int elem_bytes, uint64_t rows, uint64_t cols,
                       uint64_t ld, uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// Which operand should stay resident in L2 while the other streams? Groups of 16 row blocks (2048 rows) re-read B once per
// group: M / 2048 times N * K elements; groups of 16 column blocks (4096 columns) re-read A N / 4096 times M * K elements.
static int g_raster_override = -1;
static int pick_raster(int M, int N) {
  if (g_raster_override >= 0) return g_raster_override;
  const double by_rows = (double)((M + 2047) / 2048) * N, by_cols = (double)((N + 4095) / 4096) * M;
  return by_cols < by_rows ? 1 : 0;
}

template <int BN, bool A_MN, bool B_MN, typename OutT, bool FP8 = false>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, GemmParams p, int num_sms, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, OutT, FP8>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) return -2;
    configured = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  kern<<<grid, NUM_THREADS, Cfg::SMEM_BYTES, stream>>>(ma, mb, mc, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace mt

// a: A operand storage, lda its leading stride (elements); a_mn = 1 when stored [K, M].
// b: B operand storage; b_mn = 1 when stored [K, N] (else [N, K]).
// c: output [M, N] with leading stride ldc; out_f32 selects fp32 output; accumulate needs out_f32.
// status: device int that receives a non-zero code if a bounded wait timed out. Returns 0 on a successful launch.
extern "C" int mt_gemm_bf16(const void* a, const void* b, void* c, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                            int a_mn, int b_mn, int out_f32, int accumulate, int* status, int num_sms, cudaStream_t stream) {
  using namespace mt;
  if (accumulate && !out_f32) return -10;
  const int BN = (N % 256 == 0 || N > 1024) ? 256 : 128;
  CUtensorMap ma, mb, mc;
  int e;
  if (!a_mn) e = make_map_2d(&ma, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BK, BM);
  else e = make_map_2d(&ma, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, 64, BK);
  if (e) return 100 + e;
  if (!b_mn) e = make_map_2d(&mb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, BK, BN);
  else e = make_map_2d(&mb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, 64, BK);
  if (e) return 200 + e;
  if (out_f32) e = make_map_2d(&mc, c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldc, 32, BM);
  else e = make_map_2d(&mc, c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, ldc, 64, BM);
  if (e) return 300 + e;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.accumulate = accumulate; p.status = status;
  p.raster_n = pick_raster(M, N);
#define MT_DISPATCH(BN_)                                                                                             \
  do {                                                                                                               \
    if (!a_mn && !b_mn) return out_f32 ? launch<BN_, false, false, float>(ma, mb, mc, p, num_sms, stream)            \
                                       : launch<BN_, false, false, __nv_bfloat16>(ma, mb, mc, p, num_sms, stream);   \
    if (!a_mn && b_mn) return out_f32 ? launch<BN_, false, true, float>(ma, mb, mc, p, num_sms, stream)              \
                                      : launch<BN_, false, true, __nv_bfloat16>(ma, mb, mc, p, num_sms, stream);     \
    if (a_mn && b_mn) return out_f32 ? launch<BN_, true, true, float>(ma, mb, mc, p, num_sms, stream)                \
                                     : launch<BN_, true, true, __nv_bfloat16>(ma, mb, mc, p, num_sms, stream);       \
    return out_f32 ? launch<BN_, true, false, float>(ma, mb, mc, p, num_sms, stream)                                 \
                   : launch<BN_, true, false, __nv_bfloat16>(ma, mb, mc, p, num_sms, stream);                        \
  } while (0)
  if (BN == 256) MT_DISPATCH(256);
  MT_DISPATCH(128);
#undef MT_DISPATCH
}

// Forward GEMM out[M,N] = a[M,K] . W[N,K]^T fused with the FSDP all-gather of the flat parameter unit that holds W.
//   peer_shards: device array of `world` pointers, entry r = rank r's compute-dtype shard of this unit (chunk_elems bf16)
//   full: local full buffer of the unit (world * chunk_elems bf16); W = full + b_offset, leading stride K
//   seg_flags: device ints, one per segment (world * ceil(chunk/seg)); cleared here, stream-ordered
// `comm_ctas` CTAs of the launch do the copying. After the kernel the whole unit is resident in `full`.
extern "C" int mt_gemm_bf16_ag(const void* a, void* c, int M, int N, int K, int64_t lda, int64_t ldc, const void* const* peer_shards,
                               void* full, long chunk_elems, long seg_elems, long b_offset, int world, int* seg_flags, int comm_ctas,
                               int* status, int num_sms, cudaStream_t stream) {
  using namespace mt;
  if (chunk_elems % 8 || seg_elems % 8 || b_offset % 8 || comm_ctas < 1 || comm_ctas >= num_sms) return -10;
  constexpr int BN = 256;
  const char* w = reinterpret_cast<const char*>(full) + b_offset * 2;
  CUtensorMap ma, mb, mc;
  int e = make_map_2d(&ma, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BK, BM);
  if (e) return 100 + e;
  e = make_map_2d(&mb, w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, K, BK, BN);
  if (e) return 200 + e;
  e = make_map_2d(&mc, c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, ldc, 64, BM);
  if (e) return 300 + e;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.accumulate = 0; p.status = status;
  p.g_comm_ctas = comm_ctas; p.g_world = world;
  p.g_chunk_elems = chunk_elems; p.g_seg_elems = seg_elems;
  p.g_chunk_vec = chunk_elems / 8; p.g_seg_vec = seg_elems / 8;
  p.g_segs_per_chunk = (int)((chunk_elems + seg_elems - 1) / seg_elems);
  p.g_b_offset = b_offset;
  p.g_first_seg = (int)(b_offset / chunk_elems) * p.g_segs_per_chunk + (int)((b_offset % chunk_elems) / seg_elems);
  p.g_peer_shards = reinterpret_cast<const uint4* const*>(peer_shards);
  p.g_full = reinterpret_cast<uint4*>(full);
  p.g_seg_flags = seg_flags;
  if (cudaMemsetAsync(seg_flags, 0, sizeof(int) * (size_t)p.g_segs_per_chunk * world, stream) != cudaSuccess) return -11;
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_bf16_kernel<BN, false, false, __nv_bfloat16>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess) return -2;
    configured = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int compute = tiles < num_sms - comm_ctas ? tiles : num_sms - comm_ctas;
  kern<<<compute + comm_ctas, NUM_THREADS, Cfg::SMEM_BYTES, stream>>>(ma, mb, mc, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Grouped (mixture-of-experts) products over rows grouped by expert, every group padded to a multiple of 128 rows.
//   offs: E + 1 device ints, first padded row of each expert, offs[E] = rows in use (<= rows_max)
//   blk_expert: device ints, expert of each 128-row block (rows_max / 128 entries)
//   mode 1  y[r, :]  = x[r, :] . W[e(r)]^T     a = x [rows_max, k_in], b = W [E, n_out, k_in],  c = y  [rows_max, n_out] bf16
//   mode 2  dx[r, :] = dy[r, :] . W[e(r)]      a = dy [rows_max, n_out], b = W [E, n_out, k_in], c = dx [rows_max, k_in] bf16
//   mode 3  dW[e] (+)= dy_e^T . x_e            a = dy [rows_max, n_out], b = x [rows_max, k_in], c = dW [E, n_out, k_in] fp32
// The tile count depends on offs[E], which stays on the device: the grid is sized for rows_max and surplus CTAs exit.
// lda / ldb / ldc: leading strides (elements) of the row-grouped operands a, b (mode 3 only) and of c (modes 1, 2), so that
// column slices of wider buffers (gate | up halves) can be used in place; 0 = dense.
extern "C" int mt_gemm_bf16_grouped(int mode, const void* a, const void* b, void* c, int rows_max, int n_out, int k_in, int experts,
                                    const int* offs, const int* blk_expert, int accumulate, long lda, long ldb, long ldc, int* status,
                                    int num_sms, cudaStream_t stream) {
  using namespace mt;
  if (rows_max % BM || n_out % 128 || k_in % 128 || experts < 1 || lda % 8 || ldb % 8 || ldc % 8) return -10;
  if (accumulate && mode != 3) return -11;
  CUtensorMap ma, mb, mc;
  GemmParams p{};
  p.accumulate = accumulate; p.status = status;
  p.x_mode = mode; p.x_experts = experts; p.x_offs = offs; p.x_blk_expert = blk_expert; p.x_nw = n_out;
  int e = 0;
  if (mode == 1) {
    p.M = rows_max; p.N = n_out; p.K = k_in;
    const int BN = (n_out % 256 == 0) ? 256 : 128;
    if ((e = make_map_2d(&ma, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_max, k_in, lda ? lda : k_in, BK, BM))) return 100 + e;
    if ((e = make_map_2d(&mb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)experts * n_out, k_in, k_in, BK, BN))) return 200 + e;
    if ((e = make_map_2d(&mc, c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_max, n_out, ldc ? ldc : n_out, 64, BM))) return 300 + e;
    return BN == 256 ? launch<256, false, false, __nv_bfloat16>(ma, mb, mc, p, num_sms, stream)
                     : launch<128, false, false, __nv_bfloat16>(ma, mb, mc, p, num_sms, stream);
  }
  if (mode == 2) {
    p.M = rows_max; p.N = k_in; p.K = n_out;
    const int BN = (k_in % 256 == 0) ? 256 : 128;
    if ((e = make_map_2d(&ma, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_max, n_out, lda ? lda : n_out, BK, BM))) return 100 + e;
    if ((e = make_map_2d(&mb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)experts * n_out, k_in, k_in, 64, BK))) return 200 + e;
    if ((e = make_map_2d(&mc, c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_max, k_in, ldc ? ldc : k_in, 64, BM))) return 300 + e;
    return BN == 256 ? launch<256, false, true, __nv_bfloat16>(ma, mb, mc, p, num_sms, stream)
                     : launch<128, false, true, __nv_bfloat16>(ma, mb, mc, p, num_sms, stream);
  }
  if (mode == 3) {
    p.M = experts * n_out; p.N = k_in; p.K = rows_max;
    const int BN = (k_in % 256 == 0) ? 256 : 128;
    if ((e = make_map_2d(&ma, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_max, n_out, lda ? lda : n_out, 64, BK))) return 100 + e;
    if ((e = make_map_2d(&mb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows_max, k_in, ldb ? ldb : k_in, 64, BK))) return 200 + e;
    if ((e = make_map_2d(&mc, c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (uint64_t)experts * n_out, k_in, k_in, 32, BM))) return 300 + e;
    return BN == 256 ? launch<256, true, true, float>(ma, mb, mc, p, num_sms, stream)
                     : launch<128, true, true, float>(ma, mb, mc, p, num_sms, stream);
  }
  return -12;
}


// Tensor maps for the fused reduce-scatter epilogue: entry r covers rank r's fp32 accumulation buffer [rows, N].
// `out_maps` is host memory (world * sizeof(CUtensorMap) bytes); the caller copies it to the device once.
extern "C" int mt_gemm_rs_encode_maps(void* out_maps, const void* const* bufs, int world, int rows, int N, int bf16) {
  using namespace mt;
  CUtensorMap* m = reinterpret_cast<CUtensorMap*>(out_maps);
  for (int r = 0; r < world; ++r) {
    const int e = bf16 ? make_map_2d(&m[r], bufs[r], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, N, N, 64, BM)
                       : make_map_2d(&m[r], bufs[r], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, rows, N, N, 32, BM);
    if (e) return 100 + e;
  }
  return 0;
}

extern "C" int mt_tensor_map_bytes() { return (int)sizeof(CUtensorMap); }

// out_r[M / world, N] (fp32, zeroed by the caller) += rows of a . op(b) that rank r owns, for every rank r of the group:
// a [M, K] (K-major), b [N, K] (b_mn = 0) or [K, N] (b_mn = 1). dev_maps: device copy of mt_gemm_rs_encode_maps' output.
// out_bf16 = 1: tiles are stored (not added) as bf16 through maps that point at the owner's staging area for THIS rank.
extern "C" int mt_gemm_bf16_rs(const void* a, const void* b, int M, int N, int K, int64_t lda, int64_t ldb, int b_mn, const void* dev_maps,
                               int world, int out_bf16, int* status, int num_sms, cudaStream_t stream) {
  using namespace mt;
  if (M % (world * BM) || N % 32) return -10;
  const int BN = (N % 256 == 0 || N > 1024) ? 256 : 128;
  CUtensorMap ma, mb;
  int e = make_map_2d(&ma, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BK, BM);
  if (e) return 100 + e;
  if (!b_mn) e = make_map_2d(&mb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, BK, BN);
  else e = make_map_2d(&mb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, 64, BK);
  if (e) return 200 + e;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.accumulate = out_bf16 ? 0 : 1; p.status = status;
  p.r_maps = reinterpret_cast<const CUtensorMap*>(dev_maps);
  p.r_rows = M / world;
  // map_c is not used on this path; the A map stands in so that the prefetch has a valid descriptor
  if (out_bf16) {
    if (BN == 256) return b_mn ? launch<256, false, true, __nv_bfloat16>(ma, mb, ma, p, num_sms, stream)
                               : launch<256, false, false, __nv_bfloat16>(ma, mb, ma, p, num_sms, stream);
    return b_mn ? launch<128, false, true, __nv_bfloat16>(ma, mb, ma, p, num_sms, stream)
                : launch<128, false, false, __nv_bfloat16>(ma, mb, ma, p, num_sms, stream);
  }
  if (BN == 256) return b_mn ? launch<256, false, true, float>(ma, mb, ma, p, num_sms, stream) : launch<256, false, false, float>(ma, mb, ma, p, num_sms, stream);
  return b_mn ? launch<128, false, true, float>(ma, mb, ma, p, num_sms, stream) : launch<128, false, false, float>(ma, mb, ma, p, num_sms, stream);
}


// C[M,N] (+)= (A . B^T) * (*scale_a) * (*scale_b) with 8-bit floating point operands: a [M, K], b [N, K], both K-major,
// formats a_fmt / b_fmt (0 = E4M3, 1 = E5M2); fp32 accumulation in tensor memory; output bf16 or fp32 (accumulate needs fp32).
extern "C" int mt_gemm_fp8(const void* a, const void* b, void* c, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int a_fmt,
                           int b_fmt, int out_f32, int accumulate, const float* scale_a, const float* scale_b, int* status, int num_sms,
                           cudaStream_t stream) {
  using namespace mt;
  if ((accumulate && !out_f32) || K % 128 || lda % 16 || ldb % 16) return -10;
  const int BN = (N % 256 == 0 || N > 1024) ? 256 : 128;
  CUtensorMap ma, mb, mc;
  int e = make_map_2d(&ma, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, 2 * BK, BM);
  if (e) return 100 + e;
  if ((e = make_map_2d(&mb, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, 2 * BK, BN))) return 200 + e;
  if (out_f32) e = make_map_2d(&mc, c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldc, 32, BM);
  else e = make_map_2d(&mc, c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, ldc, 64, BM);
  if (e) return 300 + e;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.accumulate = accumulate; p.status = status;
  p.q_fmt_a = a_fmt; p.q_fmt_b = b_fmt; p.q_scale_a = scale_a; p.q_scale_b = scale_b;
  if (BN == 256) return out_f32 ? launch<256, false, false, float, true>(ma, mb, mc, p, num_sms, stream)
                                : launch<256, false, false, __nv_bfloat16, true>(ma, mb, mc, p, num_sms, stream);
  return out_f32 ? launch<128, false, false, float, true>(ma, mb, mc, p, num_sms, stream)
                 : launch<128, false, false, __nv_bfloat16, true>(ma, mb, mc, p, num_sms, stream);
}


// Tuning hook: row blocks per tile group of the persistent tile walk (default 16).
extern "C" int mt_gemm_set_raster(int v) {     // tuning hook: -1 = heuristic, 0 = row groups, 1 = column groups
  mt::g_raster_override = v;
  return 0;
}

extern "C" int mt_gemm_set_group_m(int v) {
  if (v < 1 || v > 1024) return -1;
  return cudaMemcpyToSymbol(mt::g_group_m, &v, sizeof(int)) == cudaSuccess ? 0 : -2;
}

// ================================================================================================ CTA-pair variant
// Same pipeline with cta_group::2: two CTAs of a cluster (consecutive block ids, two SMs) compute one 256 x 256 output tile.
// Each CTA loads its own 128 rows of A and only HALF of the B tile (128 of the 256 columns); the leader CTA's single MMA thread
// issues tcgen05.mma.cta_group::2 instructions that read both CTAs' shared memory and write 128 accumulator rows into each
// CTA's tensor memory. Per output tile that halves the B traffic from L2 into shared memory, and with 32 KB per stage the
// ring is six stages deep. Barrier protocol:
//   full[s]   leader only: armed by the leader's producer with the bytes of BOTH CTAs; both producers' TMA loads complete on it
//   empty[s]  in each CTA: the leader's MMA thread commits to both after the MMAs that read stage s have finished
//   tfull[a]  in each CTA: committed to both when a tile's accumulation is complete
//   tempty[a] leader only, count 2: one epilogue thread per CTA arrives when its accumulator half has been read
// Every wait is bounded exactly as in the single-CTA kernel; the two cluster-wide barriers (start, end) are reached by both
// CTAs on every path.
namespace mt {

constexpr int PAIR_STAGES = 6;
constexpr int PAIR_BN = 256;               // columns of the pair's tile; each CTA stages PAIR_BN / 2 of them
constexpr int PAIR_A_BYTES = BM * BK * 2;
constexpr int PAIR_B_BYTES = (PAIR_BN / 2) * BK * 2;
constexpr int PAIR_STAGE_BYTES = PAIR_A_BYTES + PAIR_B_BYTES;
constexpr int PAIR_EPI_BYTES = 2 * BM * 128;
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + PAIR_EPI_BYTES + 256 + 1024;

__device__ __forceinline__ void pair_tile_coords(int t, int m_blocks, int n_blocks, int& mb, int& nb, int raster_n = 0) {
  if (raster_n) {
    pair_tile_coords(t, n_blocks, m_blocks, nb, mb, 0);
    return;
  }
  constexpr int GM = 8;                    // 8 x 256 rows (or columns) per group
  const int per_group = GM * n_blocks;
  const int g = t / per_group;
  const int first_m = g * GM;
  const int gsz = min(GM, m_blocks - first_m);
  const int r = t - g * per_group;
  mb = first_m + (r % gsz);
  nb = r / gsz;
}

template <bool A_MN, bool B_MN, typename OutT, bool FP8 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_c, GemmParams p) {
  constexpr int STAGES = PAIR_STAGES;
  constexpr int BN = PAIR_BN;
  constexpr int BNH = PAIR_BN / 2;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_a0 = smem_base;
  const uint32_t smem_b0 = smem_base + STAGES * PAIR_A_BYTES;
  const uint32_t smem_epi = smem_base + STAGES * PAIR_STAGE_BYTES;
  const uint32_t bar_base = smem_epi + PAIR_EPI_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
  const uint32_t abort_slot = tmem_slot + 8;
  uint8_t* gen_base = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen_base + (tmem_slot - smem_base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + (abort_slot - smem_base));
  volatile int* epi_ok = abort_flag + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();           // 0 = leader
  const int pair = (int)blockIdx.x >> 1;
  const int pair_stride = (int)gridDim.x >> 1;
  const int m_blocks = (p.M + 2 * BM - 1) / (2 * BM);
  const int n_blocks = (p.N + BN - 1) / BN;
  const int num_tiles = m_blocks * n_blocks;
  constexpr int BKE = FP8 ? 2 * BK : BK;               // elements per 128-byte row of a stage
  static_assert(!FP8 || (!A_MN && !B_MN), "8-bit operands are K-major only");
  const int num_kb = (p.K + BKE - 1) / BKE;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 2);
    }
    fence_barrier_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    prefetch_tensormap(&map_c);
  }
  if (warp == 1) {                                   // the same warp in both CTAs, the same destination slot
    tmem_alloc_2cta(tmem_slot, 2 * BN);
    tmem_relinquish_2cta();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one thread per CTA)
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += pair_stride) {
        int mb, nb;
        pair_tile_coords(t, m_blocks, n_blocks, mb, nb, p.raster_n);
        const int m0 = mb * 2 * BM + (int)rank * BM;          // this CTA's rows of the pair tile
        const int n0 = nb * BN + (int)rank * BNH;             // this CTA's half of the B tile
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(s), phase ^ 1, abort_flag, p.status, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
          if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * PAIR_STAGE_BYTES);
          const uint32_t fb = mapa_shared(full_bar(s), 0);    // the leader's barrier counts both CTAs' bytes
          const uint32_t sa = smem_a0 + s * PAIR_A_BYTES;
          const uint32_t sb = smem_b0 + s * PAIR_B_BYTES;
          if (!A_MN) {
            tma_load_2d_pair(sa, &map_a, fb, kb * BKE, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sa + j * 8192, &map_a, fb, m0 + j * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &map_b, fb, kb * BKE, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(sb + j * 8192, &map_b, fb, n0 + j * 64, kb * BK);
          }
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (one thread of the leader CTA)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = FP8 ? make_idesc_fp8(2 * BM, BN, (uint32_t)p.q_fmt_a, (uint32_t)p.q_fmt_b) : make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      constexpr uint32_t A_LBO = A_MN ? 8192 : 16, B_LBO = B_MN ? 8192 : 16;
      constexpr uint32_t A_KSTEP = A_MN ? 2048 : 32, B_KSTEP = B_MN ? 2048 : 32;
      int s = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += pair_stride) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, abort_flag, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(s), phase, abort_flag, p.status, ST_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint64_t da = make_smem_desc(smem_a0 + s * PAIR_A_BYTES, A_LBO, 1024);
          const uint64_t db = make_smem_desc(smem_b0 + s * PAIR_B_BYTES, B_LBO, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            if (FP8) umma_f8_ss_2cta(d_tmem, da + (uint64_t)((k * A_KSTEP) >> 4), db + (uint64_t)((k * B_KSTEP) >> 4), idesc,
                                     (kb | k) != 0 ? 1u : 0u);
            else umma_f16_ss_2cta(d_tmem, da + (uint64_t)((k * A_KSTEP) >> 4), db + (uint64_t)((k * B_KSTEP) >> 4), idesc,
                                  (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_2cta(mapa_shared(empty_bar(s), 0));      // frees the stage in both CTAs
          umma_commit_2cta(mapa_shared(empty_bar(s), 1));
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_2cta(mapa_shared(tfull_bar(acc), 0));       // accumulator complete, both halves
        umma_commit_2cta(mapa_shared(tfull_bar(acc), 1));
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps (128 threads per CTA, own accumulator half)
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int et = threadIdx.x - 64;
    constexpr bool OUT_F32 = sizeof(OutT) == 4;
    int acc = 0;
    uint32_t acc_phase = 0;
    int buf = 0;
    bool ok = true;
    const uint32_t leader_tempty0 = mapa_shared(tempty_bar(0), 0), leader_tempty1 = mapa_shared(tempty_bar(1), 0);
    for (int t = pair; t < num_tiles && ok; t += pair_stride) {
      int mb, nb;
      pair_tile_coords(t, m_blocks, n_blocks, mb, nb, p.raster_n);
      const int m0 = mb * 2 * BM + (int)rank * BM;
      if (et == 0) *epi_ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, ST_TIMEOUT_EPILOGUE) ? 1 : 0;
      named_bar_sync(3, EPI_THREADS);
      if (*epi_ok == 0) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_addr + c * 32, r);
        tmem_ld_wait();
        if (FP8) {
          const float qs = __ldg(p.q_scale_a) * __ldg(p.q_scale_b);
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * qs);
        }
        if (c == BN / 32 - 1) {
          tc_fence_before();
          named_bar_sync(4, EPI_THREADS);                       // all 128 threads have read their rows
          if (et == 0) mbar_arrive_cluster(acc == 0 ? leader_tempty0 : leader_tempty1);
        }
        const bool new_store = OUT_F32 ? true : ((c & 1) == 0);
        if (new_store) {
          if (et == 0) tma_wait_group_read<1>();
          named_bar_sync(1, EPI_THREADS);
        }
        const uint32_t sbuf = smem_epi + buf * (BM * 128);
        if (OUT_F32) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t dst = sbuf + row * 128 + ((j ^ (row & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(r[4 * j]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]),
                         "r"(r[4 * j + 3])
                         : "memory");
          }
        } else {
          const int half = c & 1;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * e]), __uint_as_float(r[8 * j + 2 * e + 1]));
              pk[e] = *reinterpret_cast<uint32_t*>(&v);
            }
            const int chunk = half * 4 + j;
            const uint32_t dst = sbuf + row * 128 + ((chunk ^ (row & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3])
                         : "memory");
          }
        }
        const bool do_store = OUT_F32 ? true : ((c & 1) == 1);
        if (do_store) {
          fence_proxy_async_smem();
          named_bar_sync(2, EPI_THREADS);
          if (et == 0) {
            const int col0 = nb * BN + (OUT_F32 ? c * 32 : (c >> 1) * 64);
            if (col0 < p.N && m0 < p.M) {
              if (OUT_F32 && p.accumulate) tma_reduce_add_2d(&map_c, sbuf, col0, m0);
              else tma_store_2d(&map_c, sbuf, col0, m0);
            }
            tma_commit_group();
          }
          buf ^= 1;
        }
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (et == 0) tma_wait_group<0>();
  }

  // ------------------------------------------------------------ teardown
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                  // the peer may still read this CTA's shared memory / signal its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2cta(tmem_base, 2 * BN);
  }
}

template <bool A_MN, bool B_MN, typename OutT, bool FP8 = false>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, GemmParams p, int num_sms, cudaStream_t stream) {
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN, OutT, FP8>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES) != cudaSuccess) return -2;
    configured = true;
  }
  const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + PAIR_BN - 1) / PAIR_BN);
  int pairs = num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  kern<<<2 * pairs, NUM_THREADS, PAIR_SMEM_BYTES, stream>>>(ma, mb, mc, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace mt

// Same contract as mt_gemm_bf16, computed by CTA pairs (cta_group::2). N must be a multiple of 128 so that every CTA's half
// tile starts inside the matrix.
extern "C" int mt_gemm_bf16_pair(const void* a, const void* b, void* c, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                                 int a_mn, int b_mn, int out_f32, int accumulate, int* status, int num_sms, cudaStream_t stream) {
  using namespace mt;
  if ((accumulate && !out_f32) || N % 128) return -10;
  CUtensorMap ma, mb, mc;
  int e;
  if (!a_mn) e = make_map_2d(&ma, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, BK, BM);
  else e = make_map_2d(&ma, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, lda, 64, BK);
  if (e) return 100 + e;
  if (!b_mn) e = make_map_2d(&mb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldb, BK, PAIR_BN / 2);
  else e = make_map_2d(&mb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, ldb, 64, BK);
  if (e) return 200 + e;
  if (out_f32) e = make_map_2d(&mc, c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldc, 32, BM);
  else e = make_map_2d(&mc, c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, ldc, 64, BM);
  if (e) return 300 + e;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.accumulate = accumulate; p.status = status;
  p.raster_n = pick_raster(M, N);
  if (!a_mn && !b_mn) return out_f32 ? launch_pair<false, false, float>(ma, mb, mc, p, num_sms, stream)
                                     : launch_pair<false, false, __nv_bfloat16>(ma, mb, mc, p, num_sms, stream);
  if (!a_mn && b_mn) return out_f32 ? launch_pair<false, true, float>(ma, mb, mc, p, num_sms, stream)
                                    : launch_pair<false, true, __nv_bfloat16>(ma, mb, mc, p, num_sms, stream);
  if (a_mn && b_mn) return out_f32 ? launch_pair<true, true, float>(ma, mb, mc, p, num_sms, stream)
                                   : launch_pair<true, true, __nv_bfloat16>(ma, mb, mc, p, num_sms, stream);
  return out_f32 ? launch_pair<true, false, float>(ma, mb, mc, p, num_sms, stream)
                 : launch_pair<true, false, __nv_bfloat16>(ma, mb, mc, p, num_sms, stream);
}


// 8-bit operands on CTA pairs (see mt_gemm_fp8 for the contract); N a multiple of 128.
extern "C" int mt_gemm_fp8_pair(const void* a, const void* b, void* c, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int a_fmt,
                                int b_fmt, int out_f32, int accumulate, const float* scale_a, const float* scale_b, int* status, int num_sms,
                                cudaStream_t stream) {
  using namespace mt;
  if ((accumulate && !out_f32) || K % 128 || lda % 16 || ldb % 16 || N % 128) return -10;
  CUtensorMap ma, mb, mc;
  int e = make_map_2d(&ma, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, 2 * BK, BM);
  if (e) return 100 + e;
  if ((e = make_map_2d(&mb, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldb, 2 * BK, PAIR_BN / 2))) return 200 + e;
  if (out_f32) e = make_map_2d(&mc, c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldc, 32, BM);
  else e = make_map_2d(&mc, c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, ldc, 64, BM);
  if (e) return 300 + e;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.accumulate = accumulate; p.status = status;
  p.q_fmt_a = a_fmt; p.q_fmt_b = b_fmt; p.q_scale_a = scale_a; p.q_scale_b = scale_b;
  p.raster_n = pick_raster(M, N);
  return out_f32 ? launch_pair<false, false, float, true>(ma, mb, mc, p, num_sms, stream)
                 : launch_pair<false, false, __nv_bfloat16, true>(ma, mb, mc, p, num_sms, stream);
}
