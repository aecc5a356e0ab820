// out[M, N] = x[M, K] . W[N, K]^T for M <= 64 (decode: M = live slots), bf16 operands, fp32 accumulation, bf16 result.
//
// At these sizes the product is a stream of W through the SMs: every weight is read once from HBM and meets M activations, so
// the kernel is built around bytes in flight and around NOT re-reading x: a CTA that owns R rows of W reads all of x's K-slice
// (M / R extra bytes per weight byte; a first version with R = 16 spent most of its time on those L2 reads at M >= 8).
//
//  * CTA tile: 128 rows of W (four warps x two m16 tiles, the weight rows in the MMA's M position and the activations in its
//    N position: out^T = W . x^T), K-slice walked in chunks of 64 through a 4-stage cp.async ring shared by the CTA (rows
//    padded to 144 bytes so that ldmatrix reads hit distinct banks); mma.sync m16n8k16 from ldmatrix fragments.
//  * Split-K inside a thread-block cluster: S = 1, 2, 4 or 8 CTAs of a cluster take consecutive K-slices of the same 128 rows,
//    so that even a 4096-row weight puts 256 CTAs on the machine. Each leaves its fp32 partial tile in its own shared memory;
//    after a cluster barrier CTA r sums rows [r * 128 / S, (r + 1) * 128 / S) over all S partials through distributed shared
//    memory, in rank order (deterministic, no workspace, no atomics), and writes bf16.
//
// Requirements checked by the launcher: K % 64 == 0, 16-byte aligned rows (ld % 8 == 0), M <= 64. N is arbitrary (rows past N
// are clamped on load and not stored).
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cg = cooperative_groups;

namespace {

constexpr int ROWS = 128;     // rows of W per CTA
constexpr int KC = 64;        // k per chunk
constexpr int LDS = KC + 8;   // padded smem row (elements): 144 bytes
constexpr int STAGES = 4;
constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int src_bytes) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x2(unsigned& r0, unsigned& r1, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(s));
}
__device__ __forceinline__ void mma16816(float* d, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// MT = number of 8-wide activation tiles (M padded to 8 * MT). Grid (S, ceil(N / 128)), cluster (S, 1, 1).
template <int MT>
__global__ void __launch_bounds__(THREADS) small_m_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                          __nv_bfloat16* __restrict__ out, int M, int N, int K, long ldx, long ldw, long ldo) {
  constexpr int MP = 8 * MT;
  constexpr int STAGE_ELEMS = (ROWS + MP) * LDS;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* ring = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  cg::cluster_group cluster = cg::this_cluster();
  const int S = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.y * ROWS;
  const int chunks = K / KC;
  const int c_lo = (int)((long)chunks * rank / S), c_hi = (int)((long)chunks * (rank + 1) / S);
  const int mine = c_hi - c_lo;

  auto issue = [&](int i) {
    __nv_bfloat16* st = ring + (size_t)(i % STAGES) * STAGE_ELEMS;
    const long k0 = (long)(c_lo + i) * KC;
    // W: 128 rows x 8 pieces of 16 bytes, 8 per thread
#pragma unroll
    for (int p = threadIdx.x; p < ROWS * 8; p += THREADS) {
      const int r = p >> 3, c = (p & 7) * 8;
      int row = n0 + r;
      row = row < N ? row : N - 1;
      cp_async16(st + r * LDS + c, w + (long)row * ldw + k0 + c, 16);
    }
    // x: MP rows x 8 pieces; rows past M are zero-filled (source size 0, address clamped)
    for (int p = threadIdx.x; p < MP * 8; p += THREADS) {
      const int r = p >> 3, c = (p & 7) * 8;
      const int row = r < M ? r : M - 1;
      cp_async16(st + (ROWS + r) * LDS + c, x + (long)row * ldx + k0 + c, r < M ? 16 : 0);
    }
  };

  float acc[2][MT][4];
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int t = 0; t < MT; ++t)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[h][t][j] = 0.f;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < mine) issue(s);
    cp_commit();
  }
  for (int i = 0; i < mine; ++i) {
    cp_wait<STAGES - 2>();
    __syncthreads();                     // chunk i has landed for every thread, and every warp is done with chunk i - 1
    const int nxt = i + STAGES - 1;
    if (nxt < mine) issue(nxt);          // goes into the stage of chunk i - 1
    cp_commit();
    const __nv_bfloat16* st = ring + (size_t)(i % STAGES) * STAGE_ELEMS;
    const __nv_bfloat16* sw = st + (warp * 32) * LDS;
    const __nv_bfloat16* sx = st + ROWS * LDS;
#pragma unroll
    for (int ks = 0; ks < KC / 16; ++ks) {
      unsigned a[2][4];
      // matrices of one m16 tile: (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
#pragma unroll
      for (int h = 0; h < 2; ++h)
        ldmatrix_x4(a[h][0], a[h][1], a[h][2], a[h][3], sw + (h * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDS + ks * 16 + 8 * (lane >> 4));
      if constexpr (MT == 1) {
        unsigned b0, b1;
        ldmatrix_x2(b0, b1, sx + (lane & 7) * LDS + ks * 16 + 8 * ((lane >> 3) & 1));
        mma16816(acc[0][0], a[0], b0, b1);
        mma16816(acc[1][0], a[1], b0, b1);
      } else {
#pragma unroll
        for (int tp = 0; tp < MT / 2; ++tp) {
          unsigned b0, b1, b2, b3;
          // matrices: (m 0-7, k 0-7), (m 0-7, k 8-15), (m 8-15, k 0-7), (m 8-15, k 8-15) of this pair of activation tiles
          ldmatrix_x4(b0, b1, b2, b3, sx + (tp * 16 + (lane & 7) + 8 * (lane >> 4)) * LDS + ks * 16 + 8 * ((lane >> 3) & 1));
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            mma16816(acc[h][2 * tp], a[h], b0, b1);
            mma16816(acc[h][2 * tp + 1], a[h], b2, b3);
          }
        }
      }
    }
  }
  cp_wait<0>();
  __syncthreads();                       // the ring is free: it now holds this CTA's partial tile
  float* red = reinterpret_cast<float*>(smem_raw);           // [ROWS][MP]
  {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int tm = 0; tm < MT; ++tm) {
        float* base = red + (size_t)(warp * 32 + h * 16) * MP + tm * 8 + 2 * t;
        base[(size_t)g * MP] = acc[h][tm][0];
        base[(size_t)g * MP + 1] = acc[h][tm][1];
        base[(size_t)(g + 8) * MP] = acc[h][tm][2];
        base[(size_t)(g + 8) * MP + 1] = acc[h][tm][3];
      }
  }
  cluster.sync();                        // every CTA of the cluster has published its partial tile
  {
    const int per = ROWS / S, r0 = rank * per;
    const float* parts[8];
    for (int q = 0; q < S; ++q) parts[q] = cluster.map_shared_rank(red, q);
    for (int idx = threadIdx.x; idx < per * M; idx += THREADS) {
      const int m = idx % M, r = r0 + idx / M;
      if (n0 + r < N) {
        float v = 0.f;
        for (int q = 0; q < S; ++q) v += parts[q][(size_t)r * MP + m];
        out[(long)m * ldo + n0 + r] = __float2bfloat16(v);
      }
    }
  }
  cluster.sync();                        // nobody leaves (and frees its shared memory) while a peer may still read it
}

template <int MT>
int launch(const void* x, const void* w, void* out, int M, int N, int K, long ldx, long ldw, long ldo, int S, cudaStream_t stream) {
  constexpr int MP = 8 * MT;
  size_t ring = (size_t)STAGES * (ROWS + MP) * LDS * sizeof(__nv_bfloat16);
  size_t red = (size_t)ROWS * MP * sizeof(float);
  size_t smem = ring > red ? ring : red;
  static bool set = false;               // per instantiation; the attribute is idempotent, a race sets the same value twice
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(small_m_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(S, (N + ROWS - 1) / ROWS, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = S;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
  const __nv_bfloat16* wp = (const __nv_bfloat16*)w;
  __nv_bfloat16* op = (__nv_bfloat16*)out;
  cudaError_t e = cudaLaunchKernelEx(&cfg, small_m_kernel<MT>, xp, wp, op, M, N, K, ldx, ldw, ldo);
  return (int)e;
}

}  // namespace

extern "C" int mt_gemm_small_m_supported(int M, int N, int K, long ldx, long ldw, long ldo) {
  return M >= 1 && M <= 64 && N >= 1 && K >= KC && K % KC == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ldo >= N;
}

// K-slices per 128-row tile: enough CTAs for two per SM, at least four chunks per slice, at most 8 (portable cluster size)
extern "C" int mt_gemm_small_m_splits(int N, int K, int num_sms) {
  const int tiles = (N + ROWS - 1) / ROWS, chunks = K / KC;
  int S = 1;
  while (S < 8 && tiles * S < 2 * num_sms && chunks / (2 * S) >= 4) S *= 2;
  return S;
}

extern "C" int mt_gemm_small_m(const void* x, const void* w, void* out, int M, int N, int K, long ldx, long ldw, long ldo, int num_sms,
                               cudaStream_t stream) {
  if (!mt_gemm_small_m_supported(M, N, K, ldx, ldw, ldo)) return -1;
  const int S = mt_gemm_small_m_splits(N, K, num_sms);
  if (M <= 8) return launch<1>(x, w, out, M, N, K, ldx, ldw, ldo, S, stream);
  if (M <= 16) return launch<2>(x, w, out, M, N, K, ldx, ldw, ldo, S, stream);
  if (M <= 32) return launch<4>(x, w, out, M, N, K, ldx, ldw, ldo, S, stream);
  return launch<8>(x, w, out, M, N, K, ldx, ldw, ldo, S, stream);
}
