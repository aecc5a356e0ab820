// Sum of squares for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference: it exists for embedders of this library that run where
// cudaMalloc is off limits: inside a CUDA-graph replay loop or a real-time serving thread whose memory was
// carved up at start-up, under an allocator that forbids calls into the CUDA allocator while it holds its lock,
// or in a host application that hands this library a fixed memory budget and audits every allocation.
// The regular entry point (mt_sumsq) takes a caller-provided scratch buffer; this one keeps its scratch in a
// fixed array that lives in the library image, so the caller passes nothing but the input and the output.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Capacity of the built-in scratch: one float per stage-1 block. 4096 floats = 16 KB of device memory, held by
// every GPU that loads the library until the process exits.
#define MT_SUMSQ_NOALLOC_MAX_PARTIALS 4096
// Largest input accepted (elements). Beyond it fp32 partial sums lose too much precision to be worth returning.
#define MT_SUMSQ_NOALLOC_MAX_ELEMS (1ll << 36)

// out[0] += sum_i x[i]^2, fp32, on `stream`. Same arithmetic and reduction order as mt_sumsq on the same device.
//   x      device pointer to n floats (16-byte aligned), out  device pointer to one float.
// Returns 0 on success; a negative code otherwise (mt_sumsq_noalloc_strerror explains it):
//   -1 bad argument, -2 n exceeds MT_SUMSQ_NOALLOC_MAX_ELEMS, -3 the device needs more partials than the built-in
//   scratch holds, -4 the scratch address could not be obtained, -5 kernel launch failed, -6 the current device's
//   ordinal is 64 or more (set-up state is kept for ordinals 0..63).
// It calls no cudaMalloc / cudaFree and no allocating library routine.
//
// The first call on each device looks up the device address of the scratch array (cudaGetSymbolAddress with that
// device current) and caches it. Make that first call before starting any stream capture on the device. The set-up
// is guarded by a per-device lock and published with release / acquire ordering, so host threads may make their
// first calls at the same time; the lock is taken only until the set-up has succeeded once.
// All calls on a device share the one scratch array. Nothing in it has to start at zero (stage 1 overwrites every
// slot it later reads), but two calls that overlap on the GPU (different streams, no ordering between them) race
// on it and return garbage: order them on one stream or with events.
int mt_sumsq_noalloc(const float* x, long long n, float* out, cudaStream_t stream);

const char* mt_sumsq_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
