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

// qmode: 0 none (y in T), 1 fp8 static (inv_scale given), 2 fp8 per row, 3 int8 per row,
//        4 fp8 per group of G, 5 int8 per group of G.  scale: (rows,) or (rows, D/G).
template <typename T>
__global__ void __launch_bounds__(SEAM_THREADS)
rms_norm_add_kernel(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ weight,
                    T* __restrict__ y, uint8_t* __restrict__ codes, T* __restrict__ res_out,
                    float* __restrict__ scale, int D, float eps, int qmode, float inv_static, int G, int pow2) {
  extern __shared__ float row[];               // D floats: x + residual, then the normalised row
  __shared__ float red[SEAM_THREADS / 32];
  const size_t base = (size_t)blockIdx.x * D;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += SEAM_THREADS) {
    const float h = to_f32<T>(x[base + i]) + to_f32<T>(residual[base + i]);
    row[i] = h;
    res_out[base + i] = from_f32<T>(h);
    ss = fmaf(h, h, ss);
  }
  const float ms = seam_block_reduce(ss, false, red) / (float)D;
  const float inv = rsqrtf(ms + eps);
  float amax = 0.f;
  for (int i = threadIdx.x; i < D; i += SEAM_THREADS) {
    const float v = (row[i] * inv) * to_f32<T>(weight[i]);
    row[i] = v;
    amax = fmaxf(amax, fabsf(v));
  }
  if (qmode == 0) {
    for (int i = threadIdx.x; i < D; i += SEAM_THREADS) y[base + i] = from_f32<T>(row[i]);
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
    for (int i = threadIdx.x; i < D; i += SEAM_THREADS) {
      const float v = row[i] * q_inv;
      codes[base + i] = qmode == 3 ? (uint8_t)(int8_t)int8_encode(v) : (uint8_t)e4m3_encode(v);
    }
    return;
  }
  // per group: a warp takes whole groups
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ngroups = D / G;
  const float qmax = qmode == 4 ? 448.0f : 127.0f;
  for (int g = warp; g < ngroups; g += SEAM_THREADS / 32) {
    float gm = 0.f;
    for (int i = lane; i < G; i += 32) gm = fmaxf(gm, fabsf(row[g * G + i]));
    gm = warp_max(gm);
    const float s = seam_scale(gm, qmax, qmode == 4 ? pow2 : 0);
    const float q_inv = s > 0.f ? 1.0f / s : 0.f;
    for (int i = lane; i < G; i += 32) {
      const float v = row[g * G + i] * q_inv;
      codes[base + (size_t)g * G + i] = qmode == 5 ? (uint8_t)(int8_t)int8_encode(v) : (uint8_t)e4m3_encode(v);
    }
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
template <typename T>
__global__ void __launch_bounds__(SEAM_THREADS)
silu_mul_quant_kernel(const T* __restrict__ x, const T* __restrict__ gate, uint8_t* __restrict__ codes,
                      float* __restrict__ scale, int D, int act, float alpha, float limit, int qmode, int G,
                      int pow2) {
  extern __shared__ float row[];
  __shared__ float red[SEAM_THREADS / 32];
  const size_t base = (size_t)blockIdx.x * D;
  float amax = 0.f;
  for (int i = threadIdx.x; i < D; i += SEAM_THREADS) {
    const float v = gated_act(act, to_f32<T>(x[base + i]), to_f32<T>(gate[base + i]), alpha, limit);
    row[i] = v;
    amax = fmaxf(amax, fabsf(v));
  }
  if (qmode <= 3) {
    amax = seam_block_reduce(amax, true, red);
    const float s = amax / (qmode == 2 ? 448.0f : 127.0f);
    const float q_inv = s > 0.f ? 1.0f / s : 0.f;
    if (threadIdx.x == 0) scale[blockIdx.x] = s;
    for (int i = threadIdx.x; i < D; i += SEAM_THREADS) {
      const float v = row[i] * q_inv;
      codes[base + i] = qmode == 3 ? (uint8_t)(int8_t)int8_encode(v) : (uint8_t)e4m3_encode(v);
    }
    return;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ngroups = D / G;
  for (int g = warp; g < ngroups; g += SEAM_THREADS / 32) {
    float gm = 0.f;
    for (int i = lane; i < G; i += 32) gm = fmaxf(gm, fabsf(row[g * G + i]));
    gm = warp_max(gm);
    const float s = seam_scale(gm, 448.0f, pow2);
    const float q_inv = s > 0.f ? 1.0f / s : 0.f;
    for (int i = lane; i < G; i += 32) codes[base + (size_t)g * G + i] = (uint8_t)e4m3_encode(row[g * G + i] * q_inv);
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
  if (!seam_smem(rms_norm_add_kernel<T>, smem)) { cudaGetLastError(); return false; } \
  rms_norm_add_kernel<T><<<(unsigned)rows, SEAM_THREADS, smem, st>>>((const T*)x, (const T*)residual, (const T*)weight, \
      (T*)y, (uint8_t*)codes, (T*)res_out, scale, (int)D, eps, qmode, inv_static, G, pow2)
  if (dtype == QX_DTYPE_F32) { QX_NORM(float); }
  else if (dtype == QX_DTYPE_F16) { QX_NORM(__half); }
  else { QX_NORM(__nv_bfloat16); }
#undef QX_NORM
  note_launch();
  return true;
}

bool launch_silu_mul_quant(cudaStream_t st, qx_dtype dtype, const void* x, const void* gate, void* codes, float* scale,
                           int64_t rows, int64_t D, int act, float alpha, float limit, int qmode, int G, int pow2) {
  const size_t smem = (size_t)D * 4;
  if (smem > 200 * 1024) return false;
#define QX_ACT(T) \
  if (!seam_smem(silu_mul_quant_kernel<T>, smem)) { cudaGetLastError(); return false; } \
  silu_mul_quant_kernel<T><<<(unsigned)rows, SEAM_THREADS, smem, st>>>((const T*)x, (const T*)gate, (uint8_t*)codes, scale, \
      (int)D, act, alpha, limit, qmode, G, pow2)
  if (dtype == QX_DTYPE_F32) { QX_ACT(float); }
  else if (dtype == QX_DTYPE_F16) { QX_ACT(__half); }
  else { QX_ACT(__nv_bfloat16); }
#undef QX_ACT
  note_launch();
  return true;
}

}  // namespace qx
