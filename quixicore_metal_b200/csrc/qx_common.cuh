// Shared host/device helpers for the B200 backend: element-type conversion, the epilogue math,
// the stateless RNG hash and the status / launch bookkeeping used by every translation unit.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/quixicore_cuda.h"

namespace qx {

// ---- launch bookkeeping -------------------------------------------------------------------
void note_launch(int n = 1);                       // counts kernels this library enqueued
qx_status ok(const char* op);
qx_status fail(qx_status_code code, const char* op, const char* detail);
qx_status check_launch(const char* op);            // cudaGetLastError -> status
int sm_count();                                    // SMs of the current device (cached)

// ---- formats ------------------------------------------------------------------------------
enum Format : int { F_Q4_0 = 0, F_Q8_0, F_Q6_K, F_MXFP8, F_NVFP4, F_MXFP4, F_COUNT };
int parse_format(const char* name);                // -1 if unknown
__host__ __device__ constexpr int block_k_of(int f) {
  return f == F_Q6_K ? 256 : (f == F_NVFP4 ? 16 : 32);
}
__host__ __device__ constexpr int block_bytes_of(int f) {
  return f == F_Q4_0 ? 18 : f == F_Q8_0 ? 34 : f == F_Q6_K ? 210 : f == F_MXFP8 ? 33
       : f == F_NVFP4 ? 9 : 17;
}

// ---- element types ------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// ---- epilogue math (fp32; same formulas as the reference kernels) --------------------------
// erf by the 5-term Abramowitz-Stegun polynomial, then 0.5*v*(1+erf(v/sqrt2)).
__device__ __forceinline__ float gelu_erf_as(float v) {
  const float z = v * 0.70710678118654752440f;
  const float a = fabsf(z);
  const float t = 1.0f / (1.0f + 0.3275911f * a);
  const float poly =
      (((((1.061405429f * t + -1.453152027f) * t) + 1.421413741f) * t + -0.284496736f) * t +
       0.254829592f) * t;
  const float y = 1.0f - poly * expf(-a * a);
  return 0.5f * v * (1.0f + (z < 0.0f ? -y : y));
}
__device__ __forceinline__ float silu(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float apply_act(float v, int activation) {
  if (activation == 1) return gelu_erf_as(v);
  if (activation == 2) return silu(v);
  return v;
}

// ---- RNG: stateless integer hash keyed by (seed, row, global vocab id) ----------------------
__device__ __forceinline__ float rng_uniform(uint32_t seed, uint32_t a, uint32_t b) {
  uint32_t x = seed * 0x9E3779B9u + a * 0x85EBCA77u + b * 0xC2B2AE3Du;
  x ^= x >> 16; x *= 0x7FEB352Du;
  x ^= x >> 15; x *= 0x846CA68Bu;
  x ^= x >> 16;
  return (float)(x >> 8) * (1.0f / 16777216.0f);
}
__device__ __forceinline__ float rng_gumbel(uint32_t seed, uint32_t a, uint32_t b) {
  const float u = fmaxf(rng_uniform(seed, a, b), 1e-20f);
  return -logf(-logf(u));
}

#define QX_NEG_INF (-3.4028234663852886e38f)

// (value descending, id ascending) ordering used by every selection on this path
__device__ __forceinline__ bool better(float v, int id, float bv, int bid) {
  return v > bv || (v == bv && id < bid);
}
__device__ __forceinline__ void warp_argmax(float& v, int& id) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, off);
    const int oi = __shfl_xor_sync(0xffffffffu, id, off);
    if (better(ov, oi, v, id)) { v = ov; id = oi; }
  }
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

// ---- output quantizer encoders (fp32 arithmetic on already-rounded I/O-dtype values) ---------
// e4m3: nearest with halves rounded AWAY from zero, |x| >= 448 and NaN -> 0x7E, |x| < 2^-10 ->
// signed zero.  int8: round half away, clamp to +-127.
__device__ __forceinline__ uint32_t e4m3_encode(float x) {
  const uint32_t sign = (x < 0.0f) ? 0x80u : 0u;
  const float a = fabsf(x);
  if (!(a < 448.0f)) return sign | 0x7Eu;                 // overflow and NaN saturate
  const uint32_t bits = __float_as_uint(a);
  const int E = (int)((bits >> 23) & 0xFFu) - 127;
  if (E < -6) {                                           // e4m3 subnormal range: steps of 2^-9
    const int m = (int)roundf(a * 512.0f);           // half away from zero, exact
    if (m <= 0) return sign;
    return sign | (uint32_t)(m >= 8 ? 8 : m);
  }
  int mant = (int)(((bits & 0x7FFFFFu) + 0x80000u) >> 20);
  int exp = E + 7;
  if (mant >= 8) { mant = 0; exp += 1; }
  if (exp > 15 || (exp == 15 && mant >= 7)) return sign | 0x7Eu;
  return sign | ((uint32_t)exp << 3) | (uint32_t)mant;
}

__device__ __forceinline__ int int8_encode(float x) {
  float r = roundf(x);                                    // half away from zero
  r = fminf(fmaxf(r, -127.0f), 127.0f);
  return (int)r;
}

// exact ceil(log2(q)) for a positive finite fp32 q
__device__ __forceinline__ int ceil_log2(float q) {
  const uint32_t bits = __float_as_uint(q);
  int e = (int)((bits >> 23) & 0xFFu) - 127;
  if (bits & 0x7FFFFFu) e += 1;
  return e;
}

// One MXFP8 block {e8m0 exponent; 32 e4m3 codes} from the 32 values held one per lane of a full
// warp: scale 2^ceil(log2(amax / 448)) (amax > 0), an all-zero block stores exponent 127.
__device__ __forceinline__ void mxfp8_block_store(float v, int lane, uint8_t* __restrict__ block) {
  const float amax = warp_max(fabsf(v));
  int code = 127;
  if (amax > 0.0f) {
    const int e = ceil_log2(fmaxf(amax, 1e-10f) / 448.0f);
    code = min(max(e + 127, 1), 254);
  }
  const float inv = 1.0f / __uint_as_float((uint32_t)code << 23);
  block[1 + lane] = (uint8_t)e4m3_encode(v * inv);
  if (lane == 0) block[0] = (uint8_t)code;
}

}  // namespace qx
