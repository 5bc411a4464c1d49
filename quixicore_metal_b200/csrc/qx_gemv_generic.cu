// Shape-generic decode projections: one warp per weight row, lanes stride over 32-column spans,
// fp32 FMA accumulation, up to 8 activation rows share one pass over the weights.
//
// This is the path for every (dtype, shape, alignment) the streaming tensor-core kernels do not
// take: fp32 / fp16 activations, rows whose byte pitch is not a multiple of 16, tiny problems.
// It reads each weight byte exactly once per pass and is correct for any K % block_k == 0.
#include "qx_formats.cuh"
#include "qx_kernels.h"

namespace qx {

template <typename T>
__device__ __forceinline__ void load_x32(const T* __restrict__ p, float (&x)[32]) {
#pragma unroll
  for (int i = 0; i < 32; ++i) x[i] = to_f32<T>(p[i]);
}

// MB activation rows per pass; DUAL = gate/up pair (SwiGLU) sharing the activation reads.
template <int FMT, typename T, int MB, bool DUAL>
__global__ void __launch_bounds__(256)
gemv_generic_kernel(const T* __restrict__ x, const uint8_t* __restrict__ w0,
                    const uint8_t* __restrict__ w1, const T* __restrict__ bias0,
                    const T* __restrict__ bias1, const T* __restrict__ residual,
                    T* __restrict__ y, int M, int K, int N, int activation, int use_bias,
                    int use_residual) {
  constexpr int BK = block_k_of(FMT), BB = block_bytes_of(FMT);
  const int lane = threadIdx.x & 31;
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int warps_total = (gridDim.x * blockDim.x) >> 5;
  const int m0 = blockIdx.y * MB;
  const int mcount = min(MB, M - m0);
  const size_t row_bytes = (size_t)(K / BK) * BB;
  const int spans = K / 32 + ((K % 32) ? 1 : 0);  // nvfp4 allows K % 32 == 16

  for (int n = warp_global; n < N; n += warps_total) {
    float acc0[MB], acc1[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) { acc0[m] = 0.f; acc1[m] = 0.f; }
    const uint8_t* r0 = w0 + (size_t)n * row_bytes;
    const uint8_t* r1 = DUAL ? w1 + (size_t)n * row_bytes : nullptr;
    for (int s = lane; s < spans; s += 32) {
      float wv0[32], wv1[32];
      const bool half_span = (FMT == F_NVFP4) && (s * 32 + 16 >= K);
      if (half_span) {
        // last 16 columns of an nvfp4 row whose K is 16 mod 32: decode one block by hand
        const uint8_t* b = r0 + (size_t)s * 18;
        const float sc = e4m3_to_f32(b[0]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          wv0[i] = sc * e2m1_to_f32(b[1 + i] & 15u);
          wv0[i + 8] = sc * e2m1_to_f32(b[1 + i] >> 4);
          wv0[i + 16] = 0.f; wv0[i + 24] = 0.f;
        }
        if (DUAL) {
          const uint8_t* c = r1 + (size_t)s * 18;
          const float sd = e4m3_to_f32(c[0]);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            wv1[i] = sd * e2m1_to_f32(c[1 + i] & 15u);
            wv1[i + 8] = sd * e2m1_to_f32(c[1 + i] >> 4);
            wv1[i + 16] = 0.f; wv1[i + 24] = 0.f;
          }
        }
      } else {
        decode_span32<FMT>(r0, s, wv0);
        if (DUAL) decode_span32<FMT>(r1, s, wv1);
      }
      const int ncol = half_span ? 16 : 32;
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        if (m < mcount) {
          const T* xp = x + (size_t)(m0 + m) * K + (size_t)s * 32;
          float a0 = 0.f, a1 = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (i < ncol) {
              const float xv = to_f32<T>(xp[i]);
              a0 = fmaf(xv, wv0[i], a0);
              if (DUAL) a1 = fmaf(xv, wv1[i], a1);
            }
          }
          acc0[m] += a0;
          if (DUAL) acc1[m] += a1;
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      acc0[m] = warp_sum(acc0[m]);
      if (DUAL) acc1[m] = warp_sum(acc1[m]);
    }
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        if (m < mcount) {
          const size_t o = (size_t)(m0 + m) * N + n;
          float v = acc0[m];
          if (DUAL) {
            float u = acc1[m];
            if (use_bias) { v += to_f32<T>(bias0[n]); u += to_f32<T>(bias1[n]); }
            y[o] = from_f32<T>(silu(v) * u);
          } else {
            if (use_bias) v += to_f32<T>(bias0[n]);
            v = apply_act(v, activation);
            if (use_residual) v += to_f32<T>(residual[o]);
            y[o] = from_f32<T>(v);
          }
        }
      }
    }
  }
}

template <int FMT, typename T, bool DUAL>
static void launch_fmt(cudaStream_t st, const GemvArgs& a) {
  const int warps_per_block = 8;
  int blocks = (int)((a.N + warps_per_block - 1) / warps_per_block);
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
#define QX_LAUNCH(MBV)                                                                         \
  gemv_generic_kernel<FMT, T, MBV, DUAL><<<dim3(blocks, (unsigned)((a.M + MBV - 1) / MBV)),   \
                                           warps_per_block * 32, 0, st>>>(                     \
      (const T*)a.x, (const uint8_t*)a.w0, (const uint8_t*)a.w1, (const T*)a.bias0,            \
      (const T*)a.bias1, (const T*)a.residual, (T*)a.y, (int)a.M, (int)a.K, (int)a.N,          \
      a.activation, a.use_bias, a.use_residual)
  if (a.M == 1) QX_LAUNCH(1);
  else if (a.M == 2) QX_LAUNCH(2);
  else if (a.M <= 4) QX_LAUNCH(4);
  else QX_LAUNCH(8);
#undef QX_LAUNCH
  note_launch();
}

template <typename T, bool DUAL>
static void launch_dtype(cudaStream_t st, const GemvArgs& a) {
  switch (a.format) {
    case F_Q4_0: launch_fmt<F_Q4_0, T, DUAL>(st, a); break;
    case F_Q8_0: launch_fmt<F_Q8_0, T, DUAL>(st, a); break;
    case F_Q6_K: launch_fmt<F_Q6_K, T, DUAL>(st, a); break;
    case F_MXFP8: launch_fmt<F_MXFP8, T, DUAL>(st, a); break;
    case F_NVFP4: launch_fmt<F_NVFP4, T, DUAL>(st, a); break;
    default: launch_fmt<F_MXFP4, T, DUAL>(st, a); break;
  }
}

void launch_gemv_generic(cudaStream_t st, const GemvArgs& a) {
  const bool dual = a.w1 != nullptr;
  if (a.dtype == QX_DTYPE_F32) {
    dual ? launch_dtype<float, true>(st, a) : launch_dtype<float, false>(st, a);
  } else if (a.dtype == QX_DTYPE_F16) {
    dual ? launch_dtype<__half, true>(st, a) : launch_dtype<__half, false>(st, a);
  } else {
    dual ? launch_dtype<__nv_bfloat16, true>(st, a) : launch_dtype<__nv_bfloat16, false>(st, a);
  }
}

}  // namespace qx
