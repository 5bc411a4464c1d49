// Runtime output quantizers: per-token dynamic fp8 (e4m3) / int8 and per-32 MXFP8 blocks.
//
// Rules (fp32 arithmetic on the already-rounded I/O-dtype values):
//   per token : s = amax/448 (fp8) or amax/127 (int8); inv = s > 0 ? 1/s : 0; code = enc(x*inv)
//   MXFP8 rows: per group of 32, s = 2^ceil(log2(amax/448)) (amax > 0), stored as e8m0 byte,
//               followed by the 32 e4m3 codes of x/s; an all-zero group stores exponent 127.
//   e4m3 encode: nearest with halves rounded AWAY from zero, |x| >= 448 and NaN -> 0x7E,
//               |x| < 2^-10 -> signed zero.  int8 encode: round half away, clamp to +-127.
#include "qx_common.cuh"
#include "qx_kernels.h"

namespace qx {

template <typename T>
__global__ void __launch_bounds__(256)
quantize_per_token_kernel(const T* __restrict__ x, uint8_t* __restrict__ codes,
                          float* __restrict__ scale, int D, int kind) {
  __shared__ float red[8];
  const size_t base = (size_t)blockIdx.x * D;
  float amax = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) amax = fmaxf(amax, fabsf(to_f32<T>(x[base + i])));
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float s = amax / (kind == 0 ? 448.0f : 127.0f);
  const float inv = s > 0.0f ? 1.0f / s : 0.0f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float v = to_f32<T>(x[base + i]) * inv;
    codes[base + i] = kind == 0 ? (uint8_t)e4m3_encode(v) : (uint8_t)(int8_t)int8_encode(v);
  }
  if (threadIdx.x == 0) scale[blockIdx.x] = s;
}

template <typename T>
__global__ void __launch_bounds__(256)
quantize_mxfp8_rows_kernel(const T* __restrict__ x, uint8_t* __restrict__ blocks,
                           long long groups) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long g = warp; g < groups; g += nwarps) {
    mxfp8_block_store(to_f32<T>(x[g * 32 + lane]), lane, blocks + g * 33);
  }
}

void launch_quantize_per_token(cudaStream_t st, const void* x, void* codes, float* scale,
                               int64_t rows, int64_t D, qx_dtype dtype, int kind) {
  if (dtype == QX_DTYPE_F32)
    quantize_per_token_kernel<float><<<(unsigned)rows, 256, 0, st>>>((const float*)x, (uint8_t*)codes, scale, (int)D, kind);
  else if (dtype == QX_DTYPE_F16)
    quantize_per_token_kernel<__half><<<(unsigned)rows, 256, 0, st>>>((const __half*)x, (uint8_t*)codes, scale, (int)D, kind);
  else
    quantize_per_token_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)codes, scale, (int)D, kind);
  note_launch();
}

void launch_quantize_mxfp8_rows(cudaStream_t st, const void* x, void* blocks, int64_t rows,
                                int64_t D, qx_dtype dtype) {
  const long long groups = (long long)rows * (D / 32);
  long long want = (groups + 7) / 8;
  const int blocks_n = (int)(want < 1 ? 1 : (want > sm_count() * 16 ? sm_count() * 16 : want));
  if (dtype == QX_DTYPE_F32)
    quantize_mxfp8_rows_kernel<float><<<blocks_n, 256, 0, st>>>((const float*)x, (uint8_t*)blocks, groups);
  else if (dtype == QX_DTYPE_F16)
    quantize_mxfp8_rows_kernel<__half><<<blocks_n, 256, 0, st>>>((const __half*)x, (uint8_t*)blocks, groups);
  else
    quantize_mxfp8_rows_kernel<__nv_bfloat16><<<blocks_n, 256, 0, st>>>((const __nv_bfloat16*)x, (uint8_t*)blocks, groups);
  note_launch();
}

}  // namespace qx
