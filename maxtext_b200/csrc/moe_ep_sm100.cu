// Expert-parallel dispatch / return over NVLink peer memory (symmetric buffers), replacing the variable-size all-to-all.
//
// Every rank sorts its (token, choice) pairs by GLOBAL expert (moe_sm100.cu). The per-expert counts of all ranks are put
// into every peer's count matrix; from that matrix each rank derives, on the device and without a host round trip,
//   * the padded row layout of the experts it owns (rows of one expert: source rank 0's rows, then rank 1's, ...; each
//     expert padded to a multiple of 128 rows for the grouped GEMM), and
//   * for every global expert, the row on the owner at which its own first row of that expert lands.
// `push` then stores rows straight into the owners' receive buffers (st.global to peer addresses), `pull` loads result
// rows back from the owners' buffers (ld.global from peer addresses). Ordering between ranks uses the epoch flags of
// comm_sm100.cu (release / acquire at system scope, bounded waits); no kernel here waits on another rank.
// The reference reaches the same data movement with ragged_all_to_all (src/maxtext/layers/moe.py:1202-1361).
#include <cuda_runtime.h>
#include <stdint.h>

namespace mt {

constexpr int EP_PAD = 128;
constexpr int EP_MAX_EXPERTS = 512;
constexpr int EP_ST_OVERFLOW = 8;      // receive buffer too small for the routed rows: rows beyond it are dropped, status is set

// counts_peer[p][my_rank * E + e] = sizes[e] for every peer p (block p).
__global__ void ep_put_counts_kernel(const int* __restrict__ sizes, int E, int my_rank, int* const* __restrict__ counts_peer) {
  int* dst = counts_peer[blockIdx.x] + (long)my_rank * E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) dst[e] = sizes[e];
}

// One CTA. counts [ep][E] (source rank major). Outputs for this rank:
//   offs[el + 1], blk_expert[cap / 128]     padded layout of the owned experts (as the grouped GEMM wants it)
//   valid_rows[el]                          rows of each owned expert that carry data (the rest of the group is padding)
//   send_base[E]                            row on the owner of expert e where this rank's first row of e goes
__global__ void __launch_bounds__(512)
ep_index_kernel(const int* __restrict__ counts, int ep, int E, int my_rank, int cap, int* __restrict__ offs, int* __restrict__ blk_expert,
                int* __restrict__ valid_rows, int* __restrict__ send_base, int* __restrict__ status) {
  __shared__ int total[EP_MAX_EXPERTS];       // rows of expert e over all sources
  __shared__ int before[EP_MAX_EXPERTS];      // rows of expert e from sources below my_rank
  __shared__ int start[EP_MAX_EXPERTS + 1];   // padded start of expert e inside ITS owner's buffer
  const int el = E / ep;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0, b = 0;
    for (int s = 0; s < ep; ++s) {
      const int c = counts[s * E + e];
      if (s < my_rank) b += c;
      t += c;
    }
    total[e] = t;
    before[e] = b;
  }
  __syncthreads();
  if (threadIdx.x < ep) {                      // thread o lays out owner o's experts
    const int o = threadIdx.x;
    int acc = 0;
    for (int j = 0; j < el; ++j) {
      start[o * el + j] = acc;
      acc += (total[o * el + j] + EP_PAD - 1) / EP_PAD * EP_PAD;
    }
    if (o == my_rank) {
      start[E] = acc;
      if (acc > cap) atomicOr(status, EP_ST_OVERFLOW);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) send_base[e] = start[e] + before[e];
  const int used = start[E] < cap ? start[E] : cap;
  for (int j = threadIdx.x; j <= el; j += blockDim.x) {
    const int v = j < el ? start[my_rank * el + j] : start[E];
    offs[j] = v < cap ? v : cap / EP_PAD * EP_PAD;
    if (j < el) valid_rows[j] = total[my_rank * el + j];
  }
  for (int b = threadIdx.x; b < cap / EP_PAD; b += blockDim.x) {
    const int r = b * EP_PAD;
    int e = 0;
    if (r < used) {
      int lo = 0, hi = el - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (start[my_rank * el + mid] <= r) lo = mid; else hi = mid - 1;
      }
      e = lo;
    }
    blk_expert[b] = e;
  }
}

// Pair j (expert idx[j], stable rank dest[j] - offs_local[idx[j]] inside this rank's rows of that expert) goes to
// owner idx[j] / el, row send_base[idx[j]] + rank. Records (owner, row) for the later pull.
__global__ void __launch_bounds__(256)
ep_push_kernel(const uint4* __restrict__ src, int src_div, const int* __restrict__ idx, const int* __restrict__ dest_local,
               const int* __restrict__ offs_local, const int* __restrict__ send_base, int n, int el, int cap, int vec_per_row,
               uint4* const* __restrict__ peer_buf, int* __restrict__ pair_owner, int* __restrict__ pair_row) {
  for (int j = blockIdx.x; j < n; j += gridDim.x) {
    const int e = idx[j];
    const int o = e / el;
    const int row = send_base[e] + dest_local[j] - offs_local[e];
    if (threadIdx.x == 0) {
      pair_owner[j] = o;
      pair_row[j] = row;
    }
    if (row >= cap) continue;                 // overflow already flagged by the index kernel
    const uint4* s = src + (long)(j / src_div) * vec_per_row;
    uint4* d = peer_buf[o] + (long)row * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) d[i] = s[i];
  }
}

// out[j, :] = peer_buf[pair_owner[j]][pair_row[j], :]
__global__ void __launch_bounds__(256)
ep_pull_kernel(uint4* const* __restrict__ peer_buf, const int* __restrict__ pair_owner, const int* __restrict__ pair_row, int n, int cap,
               int vec_per_row, uint4* __restrict__ out) {
  for (int j = blockIdx.x; j < n; j += gridDim.x) {
    const int row = pair_row[j];
    uint4* d = out + (long)j * vec_per_row;
    if (row >= cap) {
      for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) d[i] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const uint4* s = peer_buf[pair_owner[j]] + (long)row * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) d[i] = s[i];
  }
}

// Zero the padding rows of every owned expert group: rows [offs[e] + valid[e], offs[e + 1]).
__global__ void __launch_bounds__(256)
ep_zero_pads_kernel(uint4* __restrict__ buf, const int* __restrict__ offs, const int* __restrict__ valid_rows, int el, int vec_per_row) {
  const int e = blockIdx.x;
  if (e >= el) return;
  const int lo = offs[e] + valid_rows[e], hi = offs[e + 1];
  for (int r = lo + blockIdx.y; r < hi; r += gridDim.y) {
    uint4* d = buf + (long)r * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) d[i] = make_uint4(0, 0, 0, 0);
  }
}

}  // namespace mt

using namespace mt;

extern "C" int mt_ep_put_counts(const int* sizes, int E, int my_rank, int ep, int* const* counts_peer, cudaStream_t st) {
  ep_put_counts_kernel<<<ep, 128, 0, st>>>(sizes, E, my_rank, counts_peer);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int mt_ep_index(const int* counts, int ep, int E, int my_rank, int cap, int* offs, int* blk_expert, int* valid_rows,
                           int* send_base, int* status, cudaStream_t st) {
  if (E > EP_MAX_EXPERTS || E % ep || cap % EP_PAD || ep > 512) return -1;
  ep_index_kernel<<<1, 512, 0, st>>>(counts, ep, E, my_rank, cap, offs, blk_expert, valid_rows, send_base, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int mt_ep_push(const void* src, int src_div, const int* idx, const int* dest_local, const int* offs_local, const int* send_base,
                          int n, int el, int cap, int D, void* const* peer_buf, int* pair_owner, int* pair_row, int sms, cudaStream_t st) {
  if (D % 8 || n < 1) return -1;
  const int grid = n < sms * 8 ? n : sms * 8;
  ep_push_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint4*>(src), src_div, idx, dest_local, offs_local, send_base, n, el, cap,
                                       D / 8, reinterpret_cast<uint4* const*>(peer_buf), pair_owner, pair_row);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int mt_ep_pull(void* const* peer_buf, const int* pair_owner, const int* pair_row, int n, int cap, int D, void* out, int sms,
                          cudaStream_t st) {
  if (D % 8 || n < 1) return -1;
  const int grid = n < sms * 8 ? n : sms * 8;
  ep_pull_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<uint4* const*>(peer_buf), pair_owner, pair_row, n, cap, D / 8,
                                       reinterpret_cast<uint4*>(out));
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int mt_ep_zero_pads(void* buf, const int* offs, const int* valid_rows, int el, int D, cudaStream_t st) {
  if (D % 8) return -1;
  ep_zero_pads_kernel<<<dim3(el, 8), 256, 0, st>>>(reinterpret_cast<uint4*>(buf), offs, valid_rows, el, D / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
