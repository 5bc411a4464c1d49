// The seams that hand quantised activations to the projections:
//   * residual add + RMSNorm with an optional quantising tail
//     (kernels/norms/add_norm/add_norm.metal:26-65 plain, :181-218 static fp8, :220-265 per-row
//     dynamic fp8, :268-312 per-row int8, :327-392 per-128-block fp8 / int8 with optional
//     power-of-two scales);
//   * gated activation (SwiGLU, or the clamped alpha-scaled variant) straight to per-token or
//     per-group fp8 / per-token int8 codes (kernels/quantization/act_quant/act_quant.metal:26-160,
//     activation math include/metal/common/glu_eval.metal:49-66).
// Everything is computed in fp32 from the I/O-dtype inputs; the sum x + residual is written back
// rounded to the I/O dtype while the norm continues on the unrounded fp32 sum; the quantisers see
// the unrounded fp32 values, as in the reference.  One CTA per row, the row kept in shared memory.
#include "qx_common.cuh"
#include "qx_kernels.h"

namespace qx {

constexpr int SEAM_THREADS = 256;

__device__ __forceinline__ float seam_block_reduce(float v, bool is_max, float* red) {
  v = is_max ? warp_max(v) : warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int i = 1; i < SEAM_THREADS / 32; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];
  return r;
}

// scale for an absolute maximum: amax / qmax, or (pow2) the next power of two at or above it
__device__ __forceinline__ float seam_scale(float amax, float qmax, int pow2) {
  if (pow2 && amax > 0.f) {
    const int e = min(max(ceil_log2(fmaxf(amax, 1e-10f) / qmax), -126), 127);   // >= -42 by the clamp on amax
    return __uint_as_float((uint32_t)(e + 127) << 23);
  }
  return amax / qmax;
}

// Elements move in 16-byte vectors (8 two-byte or 4 four-byte elements per load / store; codes as
// 8- or 4-byte words) when VEC > 1: D % VEC == 0 and 16-byte aligned rows, checked by the launcher.
template <typename T, int VEC>
__device__ __forceinline__ void seam_load(const T* __restrict__ p, size_t i, float (&v)[VEC]) {
  if constexpr (VEC == 1) {
    v[0] = to_f32<T>(p[i]);
  } else {
    T tmp[VEC];
    *reinterpret_cast<uint4*>(tmp) = *reinterpret_cast<const uint4*>(p + i);
#pragma unroll
    for (int e = 0; e < VEC; ++e) v[e] = to_f32<T>(tmp[e]);
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void seam_store(T* __restrict__ p, size_t i, const float (&v)[VEC]) {
  if constexpr (VEC == 1) {
    p[i] = from_f32<T>(v[0]);
  } else {
    T tmp[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) tmp[e] = from_f32<T>(v[e]);
    *reinterpret_cast<uint4*>(p + i) = *reinterpret_cast<const uint4*>(tmp);
  }
}
// Position of row element c in the shared-memory copy of the row.  With 8-element vectors a thread
// owns 8 consecutive elements; keeping them contiguous would put consecutive lanes 32 bytes apart
// (bank conflicts on every access), so the two halves of a vector live in two planes of D / 2
// floats, each holding one float4 per vector: consecutive lanes, consecutive float4s.
template <int VEC>
__device__ __forceinline__ int seam_sidx(int c, int D) {
  if constexpr (VEC == 8) return ((c >> 2) & 1) * (D >> 1) + ((c >> 3) << 2) + (c & 3);
  else return c;
}
// the VEC elements from c (a multiple of VEC) to / from the shared row
template <int VEC>
__device__ __forceinline__ void seam_row_put(float* __restrict__ row, int c, int D, const float (&v)[VEC]) {
  if constexpr (VEC == 1) row[c] = v[0];
  else {
#pragma unroll
    for (int q = 0; q < VEC / 4; ++q)
      *reinterpret_cast<float4*>(row + seam_sidx<VEC>(c + 4 * q, D)) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  }
}
template <int VEC>
__device__ __forceinline__ void seam_row_get(const float* __restrict__ row, int c, int D, float (&v)[VEC]) {
  if constexpr (VEC == 1) v[0] = row[c];
  else {
#pragma unroll
    for (int q = 0; q < VEC / 4; ++q) {
      const float4 f = *reinterpret_cast<const float4*>(row + seam_sidx<VEC>(c + 4 * q, D));
      v[4 * q] = f.x; v[4 * q + 1] = f.y; v[4 * q + 2] = f.z; v[4 * q + 3] = f.w;
    }
  }
}

template <int VEC>
__device__ __forceinline__ void seam_store_codes(uint8_t* __restrict__ p, size_t i, const float (&v)[VEC], bool int8) {
  uint8_t c[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) c[e] = int8 ? (uint8_t)(int8_t)int8_encode(v[e]) : (uint8_t)e4m3_encode(v[e]);
  if constexpr (VEC == 8) *reinterpret_cast<uint2*>(p + i) = *reinterpret_cast<const uint2*>(c);
  else if constexpr (VEC == 4) *reinterpret_cast<uint32_t*>(p + i) = *reinterpret_cast<const uint32_t*>(c);
  else p[i] = c[0];
}
// absolute maximum and codes of the group of G elements from column c0, by one warp
template <int VEC>
__device__ __forceinline__ float seam_group_amax(const float* __restrict__ row, int c0, int G, int D, int lane) {
  float gm = 0.f;
  if constexpr (VEC > 1) {
    for (int i4 = lane; i4 < G / 4; i4 += 32) {
      const float4 f = *reinterpret_cast<const float4*>(row + seam_sidx<VEC>(c0 + 4 * i4, D));
      gm = fmaxf(fmaxf(gm, fmaxf(fabsf(f.x), fabsf(f.y))), fmaxf(fabsf(f.z), fabsf(f.w)));
    }
  } else {
    for (int i = lane; i < G; i += 32) gm = fmaxf(gm, fabsf(row[c0 + i]));
  }
  return warp_max(gm);
}
template <int VEC>
__device__ __forceinline__ void seam_group_codes(const float* __restrict__ row, int c0, uint8_t* __restrict__ dst, int G,
                                                 int D, float q_inv, bool int8, int lane) {
  if constexpr (VEC > 1) {
    for (int i4 = lane; i4 < G / 4; i4 += 32) {
      const float4 f = *reinterpret_cast<const float4*>(row + seam_sidx<VEC>(c0 + 4 * i4, D));
      const float v[4] = {f.x * q_inv, f.y * q_inv, f.z * q_inv, f.w * q_inv};
      seam_store_codes<4>(dst, (size_t)4 * i4, v, int8);
    }
  } else {
    for (int i = lane; i < G; i += 32) {
      const float v[1] = {row[c0 + i] * q_inv};
      seam_store_codes<1>(dst, (size_t)i, v, int8);
    }
  }
}

// qmode: 0 none (y in T), 1 fp8 static (inv_scale given), 2 fp8 per row, 3 int8 per row,
//        4 fp8 per group of G, 5 int8 per group of G.  scale: (rows,) or (rows, D/G).
template <typename T, int VEC>
__global__ void __launch_bounds__(SEAM_THREADS)
rms_norm_add_kernel(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ weight,
                    T* __restrict__ y, uint8_t* __restrict__ codes, T* __restrict__ res_out,
                    float* __restrict__ scale, int D, float eps, int qmode, float inv_static, int G, int pow2) {
  extern __shared__ __align__(16) float row[]; // D floats: x + residual, then the normalised row
  __shared__ float red[SEAM_THREADS / 32];
  const size_t base = (size_t)blockIdx.x * D;
  float ss = 0.f;
  for (int i = threadIdx.x * VEC; i < D; i += SEAM_THREADS * VEC) {
    float a[VEC], b[VEC], h[VEC];
    seam_load<T, VEC>(x, base + i, a);
    seam_load<T, VEC>(residual, base + i, b);
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      h[e] = a[e] + b[e];
      ss = fmaf(h[e], h[e], ss);
    }
    seam_row_put<VEC>(row, i, D, h);
    seam_store<T, VEC>(res_out, base + i, h);
  }
  const float ms = seam_block_reduce(ss, false, red) / (float)D;
  const float inv = rsqrtf(ms + eps);
  float amax = 0.f;
  for (int i = threadIdx.x * VEC; i < D; i += SEAM_THREADS * VEC) {
    float w[VEC], v[VEC];
    seam_load<T, VEC>(weight, (size_t)i, w);
    seam_row_get<VEC>(row, i, D, v);
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      v[e] = (v[e] * inv) * w[e];
      amax = fmaxf(amax, fabsf(v[e]));
    }
    seam_row_put<VEC>(row, i, D, v);
  }
  if (qmode == 0) {
    for (int i = threadIdx.x * VEC; i < D; i += SEAM_THREADS * VEC) {
      float v[VEC];
      seam_row_get<VEC>(row, i, D, v);
      seam_store<T, VEC>(y, base + i, v);
    }
    return;
  }
  if (qmode <= 3) {
    float q_inv = inv_static;
    if (qmode >= 2) {
      amax = seam_block_reduce(amax, true, red);
      const float s = amax / (qmode == 2 ? 448.0f : 127.0f);
      q_inv = s > 0.f ? 1.0f / s : 0.f;
      if (threadIdx.x == 0) scale[blockIdx.x] = s;
    }
    for (int i = threadIdx.x * VEC; i < D; i += SEAM_THREADS * VEC) {
      float v[VEC];
      seam_row_get<VEC>(row, i, D, v);
#pragma unroll
      for (int e = 0; e < VEC; ++e) v[e] *= q_inv;
      seam_store_codes<VEC>(codes, base + i, v, qmode == 3);
    }
    return;
  }
  // per group: a warp takes whole groups
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ngroups = D / G;
  const float qmax = qmode == 4 ? 448.0f : 127.0f;
  for (int g = warp; g < ngroups; g += SEAM_THREADS / 32) {
    const float gm = seam_group_amax<VEC>(row, g * G, G, D, lane);
    const float s = seam_scale(gm, qmax, qmode == 4 ? pow2 : 0);
    const float q_inv = s > 0.f ? 1.0f / s : 0.f;
    seam_group_codes<VEC>(row, g * G, codes + base + (size_t)g * G, G, D, q_inv, qmode == 5, lane);
    if (lane == 0) scale[(size_t)blockIdx.x * ngroups + g] = s;
  }
}

// act: 0 silu(x) * gate, 1 clamped: x <- min(x, limit), gate <- clamp(gate, +-limit),
// x * sigmoid(alpha x) * (1 + gate)
__device__ __forceinline__ float gated_act(int act, float x0, float x1, float alpha, float limit) {
  if (act == 1) {
    x0 = fminf(x0, limit);
    x1 = fmaxf(fminf(x1, limit), -limit);
    return (x0 / (1.0f + expf(-x0 * alpha))) * (1.0f + x1);
  }
  return (x0 / (1.0f + expf(-x0))) * x1;
}

// qmode: 2 fp8 per row, 3 int8 per row, 4 fp8 per group of G (pow2: power-of-two scales)
template <typename T, int VEC>
__global__ void __launch_bounds__(SEAM_THREADS)
silu_mul_quant_kernel(const T* __restrict__ x, const T* __restrict__ gate, uint8_t* __restrict__ codes,
                      float* __restrict__ scale, int D, int act, float alpha, float limit, int qmode, int G,
                      int pow2) {
  extern __shared__ __align__(16) float row[];
  __shared__ float red[SEAM_THREADS / 32];
  const size_t base = (size_t)blockIdx.x * D;
  float amax = 0.f;
  for (int i = threadIdx.x * VEC; i < D; i += SEAM_THREADS * VEC) {
    float a[VEC], b[VEC];
    seam_load<T, VEC>(x, base + i, a);
    seam_load<T, VEC>(gate, base + i, b);
    float v[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      v[e] = gated_act(act, a[e], b[e], alpha, limit);
      amax = fmaxf(amax, fabsf(v[e]));
    }
    seam_row_put<VEC>(row, i, D, v);
  }
  if (qmode <= 3) {
    amax = seam_block_reduce(amax, true, red);
    const float s = amax / (qmode == 2 ? 448.0f : 127.0f);
    const float q_inv = s > 0.f ? 1.0f / s : 0.f;
    if (threadIdx.x == 0) scale[blockIdx.x] = s;
    for (int i = threadIdx.x * VEC; i < D; i += SEAM_THREADS * VEC) {
      float v[VEC];
      seam_row_get<VEC>(row, i, D, v);
#pragma unroll
      for (int e = 0; e < VEC; ++e) v[e] *= q_inv;
      seam_store_codes<VEC>(codes, base + i, v, qmode == 3);
    }
    return;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ngroups = D / G;
  for (int g = warp; g < ngroups; g += SEAM_THREADS / 32) {
    const float gm = seam_group_amax<VEC>(row, g * G, G, D, lane);
    const float s = seam_scale(gm, 448.0f, pow2);
    const float q_inv = s > 0.f ? 1.0f / s : 0.f;
    seam_group_codes<VEC>(row, g * G, codes + base + (size_t)g * G, G, D, q_inv, false, lane);
    if (lane == 0) scale[(size_t)blockIdx.x * ngroups + g] = s;
  }
}

template <typename K>
static bool seam_smem(K kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return true;
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) == cudaSuccess;
}

bool launch_rms_norm_add(cudaStream_t st, qx_dtype dtype, const void* x, const void* residual, const void* weight,
                         void* y, void* codes, void* res_out, float* scale, int64_t rows, int64_t D, float eps,
                         int qmode, float inv_static, int G, int pow2) {
  const size_t smem = (size_t)D * 4;
  if (smem > 200 * 1024) return false;
#define QX_NORM(T) \
  { constexpr int V = 16 / (int)sizeof(T); \
    const bool vec = D % V == 0 && (G <= 0 || G % 4 == 0) && \
        ((((uintptr_t)x | (uintptr_t)residual | (uintptr_t)weight | (uintptr_t)y | (uintptr_t)res_out | (uintptr_t)codes) & 15) == 0); \
    if (vec) { \
      if (!seam_smem(rms_norm_add_kernel<T, V>, smem)) { cudaGetLastError(); return false; } \
      rms_norm_add_kernel<T, V><<<(unsigned)rows, SEAM_THREADS, smem, st>>>((const T*)x, (const T*)residual, (const T*)weight, \
          (T*)y, (uint8_t*)codes, (T*)res_out, scale, (int)D, eps, qmode, inv_static, G, pow2); \
    } else { \
      if (!seam_smem(rms_norm_add_kernel<T, 1>, smem)) { cudaGetLastError(); return false; } \
      rms_norm_add_kernel<T, 1><<<(unsigned)rows, SEAM_THREADS, smem, st>>>((const T*)x, (const T*)residual, (const T*)weight, \
          (T*)y, (uint8_t*)codes, (T*)res_out, scale, (int)D, eps, qmode, inv_static, G, pow2); \
    } }
  if (dtype == QX_DTYPE_F32) QX_NORM(float)
  else if (dtype == QX_DTYPE_F16) QX_NORM(__half)
  else QX_NORM(__nv_bfloat16)
#undef QX_NORM
  note_launch();
  return true;
}

bool launch_silu_mul_quant(cudaStream_t st, qx_dtype dtype, const void* x, const void* gate, void* codes, float* scale,
                           int64_t rows, int64_t D, int act, float alpha, float limit, int qmode, int G, int pow2) {
  const size_t smem = (size_t)D * 4;
  if (smem > 200 * 1024) return false;
#define QX_ACT(T) \
  { constexpr int V = 16 / (int)sizeof(T); \
    const bool vec = D % V == 0 && (G <= 0 || G % 4 == 0) && ((((uintptr_t)x | (uintptr_t)gate | (uintptr_t)codes) & 15) == 0); \
    if (vec) { \
      if (!seam_smem(silu_mul_quant_kernel<T, V>, smem)) { cudaGetLastError(); return false; } \
      silu_mul_quant_kernel<T, V><<<(unsigned)rows, SEAM_THREADS, smem, st>>>((const T*)x, (const T*)gate, (uint8_t*)codes, scale, \
          (int)D, act, alpha, limit, qmode, G, pow2); \
    } else { \
      if (!seam_smem(silu_mul_quant_kernel<T, 1>, smem)) { cudaGetLastError(); return false; } \
      silu_mul_quant_kernel<T, 1><<<(unsigned)rows, SEAM_THREADS, smem, st>>>((const T*)x, (const T*)gate, (uint8_t*)codes, scale, \
          (int)D, act, alpha, limit, qmode, G, pow2); \
    } }
  if (dtype == QX_DTYPE_F32) QX_ACT(float)
  else if (dtype == QX_DTYPE_F16) QX_ACT(__half)
  else QX_ACT(__nv_bfloat16)
#undef QX_ACT
  note_launch();
  return true;
}

}  // namespace qx
