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

// hist[bin] += 1 for every lane with `pred`; the lanes of a warp that hit the same bin share one
// atomic (the top byte of float keys takes only a few values, so unaggregated atomics serialise).
// Every lane of the warp must call it.
__device__ __forceinline__ void hist_add(unsigned* hist, bool pred, unsigned bin) {
  const unsigned lane = threadIdx.x & 31u;
  const unsigned peers = __match_any_sync(0xffffffffu, pred ? bin : (0x100u + lane));
  if (pred && (unsigned)(__ffs((int)peers) - 1) == lane) atomicAdd(&hist[bin], (unsigned)__popc(peers));
}

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

}  // namespace qx
