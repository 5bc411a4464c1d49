// The operators either side of the decode-projection path that share its packed formats:
//   * packed embedding lookup (dequant_gather / quantized_embedding): gather rows of a packed
//     table, dequantise exactly in fp32, multiply by `scale`, optionally add an output-shaped
//     term, round ONCE to the output type; ids outside [0, rows) give all-zero rows and ignore the
//     additive term (kernels/quantization/dequant_gather/dequant_gather.metal:10-48, :62-105);
//   * qgemv / qgemm: out (N, M) = dequantise(W) (N, K) @ x (K, M) in the reference's column-major
//     activation layout (kernels/quantization/qgemv/qgemv.metal:13-45,
//     kernels/quantization/qgemm/qgemm.metal:11-50), served by the projection kernels of this
//     backend: x is transposed into their row layout, the result transposed back.  The weights are
//     dequantised exactly in fp32 here (the Metal kernels round scale * code to half first); the
//     reference's own tolerance for these two ops is 2e-2 relative.
#include "qx_formats.cuh"
#include "qx_kernels.h"

namespace qx {

// One thread per 32-column span of one output row (16 columns for the last nvfp4 span of a row
// whose width is 16 mod 32).
template <int FMT, typename T>
__global__ void __launch_bounds__(256)
quantized_embedding_kernel(const uint8_t* __restrict__ table, const int32_t* __restrict__ ids,
                           const T* __restrict__ add, T* __restrict__ out, int rows, int columns,
                           long long tokens, float scale, int use_add) {
  constexpr int BK = block_k_of(FMT), BB = block_bytes_of(FMT);
  const int spans = (columns + 31) / 32;
  const long long total = tokens * spans;
  const size_t row_bytes = (size_t)(columns / BK) * BB;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long token = i / spans;
    const int s = (int)(i - token * spans);
    const int ncol = min(32, columns - s * 32);
    T* dst = out + token * columns + (size_t)s * 32;
    const int row = ids[token];
    if (row < 0 || row >= rows) {
      for (int c = 0; c < ncol; ++c) dst[c] = from_f32<T>(0.f);
      continue;
    }
    const uint8_t* base = table + (size_t)row * row_bytes;
    float w[32];
    if (FMT == F_NVFP4 && ncol == 16) {
      const uint8_t* b = base + (size_t)s * 18;
      const float sc = e4m3_to_f32(b[0]);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        w[k] = sc * e2m1_to_f32(b[1 + k] & 15u);
        w[k + 8] = sc * e2m1_to_f32(b[1 + k] >> 4);
      }
    } else {
      decode_span32<FMT>(base, s, w);
    }
    const T* ad = add + token * columns + (size_t)s * 32;
    if (ncol == 32 && (((uintptr_t)dst | (use_add ? (uintptr_t)ad : 0)) & 15) == 0) {
      // whole span, 16-byte aligned: the additive term and the output move as 16-byte vectors
      constexpr int PER = 16 / (int)sizeof(T);            // elements per vector
#pragma unroll
      for (int q = 0; q < 32 / PER; ++q) {
        T a[PER], o[PER];
        if (use_add) *reinterpret_cast<uint4*>(a) = __ldg(reinterpret_cast<const uint4*>(ad) + q);
#pragma unroll
        for (int e = 0; e < PER; ++e) {
          float v = __fmul_rn(w[q * PER + e], scale);     // the product is rounded before the addition, as in the reference
          if (use_add) v = __fadd_rn(v, to_f32<T>(a[e]));
          o[e] = from_f32<T>(v);
        }
        reinterpret_cast<uint4*>(dst)[q] = *reinterpret_cast<const uint4*>(o);
      }
      continue;
    }
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      if (c < ncol) {
        float v = __fmul_rn(w[c], scale);                 // the product is rounded before the addition, as in the reference
        if (use_add) v = __fadd_rn(v, to_f32<T>(ad[c]));
        dst[c] = from_f32<T>(v);
      }
    }
  }
}

template <typename T>
static void launch_embedding_t(cudaStream_t st, int format, const void* table, const int32_t* ids, const void* add,
                               void* out, int64_t rows, int64_t columns, int64_t tokens, float scale, int use_add) {
  const long long total = tokens * ((columns + 31) / 32);
  long long blocks = (total + 255) / 256;
  if (blocks > sm_count() * 32) blocks = sm_count() * 32;
  if (blocks < 1) blocks = 1;
#define QX_EMB(F) quantized_embedding_kernel<F, T><<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)table, ids, (const T*)add, (T*)out, (int)rows, (int)columns, (long long)tokens, scale, use_add)
  switch (format) {
    case F_Q4_0: QX_EMB(F_Q4_0); break;
    case F_Q8_0: QX_EMB(F_Q8_0); break;
    case F_Q6_K: QX_EMB(F_Q6_K); break;
    case F_MXFP8: QX_EMB(F_MXFP8); break;
    case F_NVFP4: QX_EMB(F_NVFP4); break;
    default: QX_EMB(F_MXFP4); break;
  }
#undef QX_EMB
  note_launch();
}

void launch_quantized_embedding(cudaStream_t st, int format, qx_dtype out_dtype, const void* table, const int32_t* ids,
                                const void* add, void* out, int64_t rows, int64_t columns, int64_t tokens, float scale,
                                int use_add) {
  if (out_dtype == QX_DTYPE_F32) launch_embedding_t<float>(st, format, table, ids, add, out, rows, columns, tokens, scale, use_add);
  else if (out_dtype == QX_DTYPE_F16) launch_embedding_t<__half>(st, format, table, ids, add, out, rows, columns, tokens, scale, use_add);
  else launch_embedding_t<__nv_bfloat16>(st, format, table, ids, add, out, rows, columns, tokens, scale, use_add);
}

// out (C, R) = in (R, C)^T through a 32 x 33 shared tile.
template <typename T>
__global__ void __launch_bounds__(256)
transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int R, int C) {
  __shared__ T tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    if (r < R && c < C) tile[i][threadIdx.x] = in[(size_t)r * C + c];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int c = c0 + i, r = r0 + threadIdx.x;
    if (r < R && c < C) out[(size_t)c * R + r] = tile[threadIdx.x][i];
  }
}

void launch_transpose(cudaStream_t st, const void* in, void* out, int64_t R, int64_t C, size_t elem_bytes) {
  dim3 grid((unsigned)((C + 31) / 32), (unsigned)((R + 31) / 32)), block(32, 8);
  if (elem_bytes == 4) transpose_kernel<float><<<grid, block, 0, st>>>((const float*)in, (float*)out, (int)R, (int)C);
  else transpose_kernel<__half><<<grid, block, 0, st>>>((const __half*)in, (__half*)out, (int)R, (int)C);
  note_launch();
}

}  // namespace qx
