// Block-wide reductions and the order-preserving float key shared by the selection kernels.
#pragma once

#include "qx_common.cuh"

namespace qx {

// Order-preserving map float -> uint32 (larger float = larger key; +0 and -0 share a key).
__device__ __forceinline__ uint32_t float_key(float v) {
  uint32_t u = __float_as_uint(v);
  if (v == 0.0f) u = 0u;
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct BlockScratch {
  float fv[32];
  int iv[32];
  unsigned hist[256];
  unsigned u[8];
};

__device__ __forceinline__ void block_argmax(float& v, int& id, BlockScratch& s) {
  warp_argmax(v, id);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) { s.fv[warp] = v; s.iv[warp] = id; }
  __syncthreads();
  v = lane < nw ? s.fv[lane] : QX_NEG_INF;
  id = lane < nw ? s.iv[lane] : 0x7fffffff;
  warp_argmax(v, id);
}
__device__ __forceinline__ float block_sum(float v, BlockScratch& s) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) s.fv[warp] = v;
  __syncthreads();
  v = lane < nw ? s.fv[lane] : 0.f;
  return warp_sum(v);
}
// sum of f and bitwise OR of u over the block, one pair of barriers
__device__ __forceinline__ void block_sum_or(float& f, unsigned& u, BlockScratch& s) {
  f = warp_sum(f);
  u = __reduce_or_sync(0xffffffffu, u);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) { s.fv[warp] = f; s.iv[warp] = (int)u; }
  __syncthreads();
  f = warp_sum(lane < nw ? s.fv[lane] : 0.f);
  u = __reduce_or_sync(0xffffffffu, lane < nw ? (unsigned)s.iv[lane] : 0u);
}
__device__ __forceinline__ float block_max(float v, BlockScratch& s) {
  v = warp_max(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) s.fv[warp] = v;
  __syncthreads();
  v = lane < nw ? s.fv[lane] : QX_NEG_INF;
  return warp_max(v);
}
__device__ __forceinline__ int block_min_int(int v, BlockScratch& s) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, off));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) s.iv[warp] = v;
  __syncthreads();
  v = lane < nw ? s.iv[lane] : 0x7fffffff;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}
__device__ __forceinline__ unsigned block_sum_u(unsigned v, BlockScratch& s) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) s.iv[warp] = (int)v;
  __syncthreads();
  v = lane < nw ? (unsigned)s.iv[lane] : 0u;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// The k-th largest of the keys key(j, out), j in [0, n) (key returns false for an absent entry;
// 1 <= k <= number of present entries).  tau = that key, count_eq = entries equal to tau,
// remaining = how many of those belong to the k largest.  Histogram passes of up to 8 bits over
// keys rebased to their minimum, starting at the highest bit in which they differ: the float keys
// of a candidate pool share their sign and most exponent bits, and unrebased the first passes would
// put every key into one or two bins and serialise the shared-memory atomics.
template <typename KeyFn>
__device__ __forceinline__ void block_radix_select(long long n, KeyFn key, unsigned k, BlockScratch& S,
                                                   uint32_t& tau, unsigned& remaining, unsigned& count_eq) {
  const int tid = threadIdx.x, nth = blockDim.x;
  constexpr int U = 8;                           // keys fetched per thread before any is consumed:
  //                                                the loads of a batch overlap instead of paying the
  //                                                memory latency once per key
  int lo = 0x7fffffff, hi = 0x7fffffff;          // min of key and of ~key, as sign-flipped ints
  for (long long j0 = tid; j0 < n; j0 += (long long)nth * U) {
    uint32_t kx[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long j = j0 + (long long)u * nth;
      kx[u] = 0u;
      ok[u] = j < n && key(j, kx[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (ok[u]) {
        lo = min(lo, (int)(kx[u] ^ 0x80000000u));
        hi = min(hi, (int)(~kx[u] ^ 0x80000000u));
      }
  }
  lo = block_min_int(lo, S);
  hi = block_min_int(hi, S);
  const uint32_t kmin = (uint32_t)lo ^ 0x80000000u, kmax = ~((uint32_t)hi ^ 0x80000000u);
  const uint32_t range = kmax - kmin;
  int shift = range ? 32 - __clz((int)range) : 0;
  uint32_t prefix = 0u, mask = 0u;
  remaining = k; count_eq = 0u;
  do {
    const int width = min(8, shift);
    shift -= width;
    const uint32_t bmask = (1u << width) - 1u;
    for (int b = tid; b < 256; b += nth) S.hist[b] = 0u;
    __syncthreads();
    for (long long j0 = tid; j0 < n; j0 += (long long)nth * U) {
      uint32_t kx[U];
      bool ok[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long j = j0 + (long long)u * nth;
        kx[u] = 0u;
        ok[u] = j < n && key(j, kx[u]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t kn = kx[u] - kmin;
        if (ok[u] && (kn & mask) == prefix) atomicAdd(&S.hist[(kn >> shift) & bmask], 1u);
      }
    }
    __syncthreads();
    if (tid < 32) {
      // the highest bin b with (entries in bins above b) + hist[b] >= remaining, found by the first
      // warp: 8 bins per lane, a suffix sum over the lanes, then each lane tests its own bins
      unsigned h[8], sum = 0u;
#pragma unroll
      for (int i = 0; i < 8; ++i) { h[i] = S.hist[tid * 8 + i]; sum += h[i]; }
      unsigned suffix = sum;                                  // entries in this lane's bins and above
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const unsigned v = __shfl_down_sync(0xffffffffu, suffix, off);
        if (tid + off < 32) suffix += v;
      }
      unsigned c = suffix - sum, c_at = 0u;
      int found = -1;
#pragma unroll
      for (int i = 7; i >= 0; --i) {
        if (found < 0 && c + h[i] >= remaining) { found = tid * 8 + i; c_at = c; }
        c += h[i];
      }
      const int b = max(0, (int)__reduce_max_sync(0xffffffffu, found));
      const unsigned above = __shfl_sync(0xffffffffu, c_at, b >> 3);
      if (tid == 0) { S.u[0] = (unsigned)b; S.u[1] = remaining - above; S.u[2] = S.hist[b]; }
    }
    __syncthreads();
    prefix |= S.u[0] << shift;
    mask |= bmask << shift;
    remaining = S.u[1];
    count_eq = S.u[2];
    __syncthreads();
  } while (shift > 0);
  tau = prefix + kmin;
}

}  // namespace qx
