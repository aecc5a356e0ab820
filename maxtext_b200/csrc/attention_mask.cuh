// Mask description shared by the attention forward and backward kernels, at two granularities:
//   * 128 x 128 tile pairs are classified as skipped / unmasked / mixed from position bounds, so that all roles of a CTA
//     (TMA producer, MMA issuer, softmax threads) agree on which key tiles take part without talking to each other;
//   * inside a mixed tile a row tests "position of the other side lies in [lo, hi]" with one unsigned comparison.
// Positions are token indices (queries offset by q_off) or come from arrays (keys that are a block of a longer sequence,
// or packed rows under chunked attention); with arrays, per-tile (min, max) tables give the bounds.
#pragma once
#include <limits.h>
#include <stdint.h>

namespace mt {
namespace attn {

struct Mask {
  int Sq, Skv;
  int n_qt, n_kt;        // 128-token tiles of the query / key sequence
  int q_off;             // index mode: position of query row i is i + q_off, of key row j is j
  int causal, window, chunk;
  const int* seg_q;      // [B,Sq]  segment ids (0 = padding) or nullptr
  const int* seg_k;      // [B,Skv]
  const int* pos_q;      // [B,Sq]  positions, or nullptr: index mode
  const int* pos_k;      // [B,Skv]
  const int* tile_q;     // [B, n_qt, 2] (min, max) position per query tile (array mode)
  const int* tile_k;     // [B, n_kt, 2]
};

struct Span {
  int rows;        // valid tokens of the tile (0: the tile lies beyond the sequence)
  int pmin, pmax;  // smallest / largest position among them
};

__device__ __forceinline__ Span q_span(const Mask& m, int b, int qt) {
  Span s;
  const int q0 = qt * 128;
  s.rows = q0 >= m.Sq ? 0 : (m.Sq - q0 < 128 ? m.Sq - q0 : 128);
  if (m.pos_q && s.rows) {
    s.pmin = m.tile_q[((long)b * m.n_qt + qt) * 2];
    s.pmax = m.tile_q[((long)b * m.n_qt + qt) * 2 + 1];
  } else {
    s.pmin = q0 + m.q_off;
    s.pmax = q0 + (s.rows ? s.rows - 1 : 0) + m.q_off;
  }
  return s;
}

__device__ __forceinline__ Span k_span(const Mask& m, int b, int kt) {
  Span s;
  const int k0 = kt * 128;
  s.rows = k0 >= m.Skv ? 0 : (m.Skv - k0 < 128 ? m.Skv - k0 : 128);
  if (m.pos_k && s.rows) {
    s.pmin = m.tile_k[((long)b * m.n_kt + kt) * 2];
    s.pmax = m.tile_k[((long)b * m.n_kt + kt) * 2 + 1];
  } else {
    s.pmin = k0;
    s.pmax = k0 + (s.rows ? s.rows - 1 : 0);
  }
  return s;
}

// 0: every (query, key) pair of the two tiles is masked; 1: none is (all 128 keys exist, no segment test); 2: mixed.
__device__ __forceinline__ int classify(const Mask& m, const Span& q, const Span& k) {
  if (q.rows == 0 || k.rows == 0) return 0;
  if (m.causal && k.pmin > q.pmax) return 0;
  if (m.window > 0 && q.pmin - k.pmax >= m.window) return 0;
  bool full = k.rows == 128 && !m.seg_q;
  if (m.causal && k.pmax > q.pmin) full = false;
  if (m.window > 0 && q.pmax - k.pmin >= m.window) full = false;
  if (m.chunk > 0) {
    const int c0 = q.pmin / m.chunk;
    const bool q_one = q.pmax / m.chunk == c0;
    if (q_one && (k.pmax < c0 * m.chunk || (!m.causal && k.pmin >= (c0 + 1) * m.chunk))) return 0;
    if (!(q_one && k.pmin / m.chunk == c0 && k.pmax / m.chunk == c0)) full = false;
  }
  return full ? 1 : 2;
}

// Closed interval of key positions a query at `qpos` may attend to (empty when hi < lo).
__device__ __forceinline__ void key_interval(const Mask& m, int qpos, int& lo, int& hi) {
  lo = INT_MIN;
  hi = INT_MAX - 1;                 // INT_MAX marks a key beyond the sequence in array mode
  if (m.causal) hi = qpos;
  if (m.window > 0) lo = qpos - m.window + 1;
  if (m.chunk > 0) {
    const int c = (qpos / m.chunk) * m.chunk;
    lo = lo > c ? lo : c;
    hi = hi < c + m.chunk - 1 ? hi : c + m.chunk - 1;
  }
  if (!m.pos_k && hi > m.Skv - 1) hi = m.Skv - 1;
}

// Closed interval of query positions that may attend to a key at `kpos`.
__device__ __forceinline__ void query_interval(const Mask& m, int kpos, int& lo, int& hi) {
  lo = INT_MIN;
  hi = INT_MAX - 1;
  if (m.causal) lo = kpos;
  if (m.window > 0) hi = kpos + m.window - 1;
  if (m.chunk > 0) {
    const int c = (kpos / m.chunk) * m.chunk;
    lo = lo > c ? lo : c;
    hi = hi < c + m.chunk - 1 ? hi : c + m.chunk - 1;
  }
  if (!m.pos_q && hi > m.Sq - 1 + m.q_off) hi = m.Sq - 1 + m.q_off;
}

// Index mode: key tiles [lo, hi) a query tile can need (exact up to tile granularity); array mode: all of them.
__device__ __forceinline__ void k_tiles_for(const Mask& m, const Span& q, int& lo, int& hi) {
  lo = 0;
  hi = m.n_kt;
  if (m.pos_q || q.rows == 0) { if (q.rows == 0) hi = 0; return; }
  if (m.causal) hi = q.pmax < 0 ? 0 : (q.pmax / 128 + 1 < m.n_kt ? q.pmax / 128 + 1 : m.n_kt);
  int lp = INT_MIN;
  if (m.window > 0) lp = q.pmin - m.window + 1;
  if (m.chunk > 0 && q.pmin >= 0) { const int c = (q.pmin / m.chunk) * m.chunk; lp = lp > c ? lp : c; }
  if (lp > 0) lo = lp / 128;
  if (hi < lo) hi = lo;
}

// Index mode: query tiles [lo, hi) that can see a key tile.
__device__ __forceinline__ void q_tiles_for(const Mask& m, const Span& k, int& lo, int& hi) {
  lo = 0;
  hi = m.n_qt;
  if (m.pos_q || k.rows == 0) { if (k.rows == 0) hi = 0; return; }
  if (m.causal) { const int qi = k.pmin - m.q_off; lo = qi > 0 ? qi / 128 : 0; }      // query index >= key position - q_off
  int hp = INT_MAX;
  if (m.window > 0) hp = k.pmax + m.window - 1;
  if (m.chunk > 0) { const int c = (k.pmax / m.chunk) * m.chunk + m.chunk - 1; hp = hp < c ? hp : c; }
  if (hp != INT_MAX) { const int qi = hp - m.q_off; hi = qi < 0 ? 0 : (qi / 128 + 1 < m.n_qt ? qi / 128 + 1 : m.n_qt); }
  if (hi < lo) hi = lo;
}

}  // namespace attn
}  // namespace mt
