// Packed block formats of the QuixiCore contract and their scalar decoders.
//
// A packed weight is uint8 (N, K/block_k, block_bytes), row-major.  All six formats dequantise
// exactly in fp32 (every product has at most 24 significant bits).
//
//   q4_0   18 B / 32 w   {f16 d; u8 qs[16]}   w[i] = d*((qs[i]&15)-8), w[i+16] = d*((qs[i]>>4)-8)
//   q8_0   34 B / 32 w   {f16 d; i8 qs[32]}   w[i] = d*qs[i]
//   q6_K  210 B / 256 w  {u8 ql[128]; u8 qh[64]; i8 sc[16]; f16 d}   w = (d*sc[sub])*(code-32)
//   mxfp8  33 B / 32 w   {e8m0 e; e4m3 qs[32]}  w[i] = 2^(e-127)*e4m3(qs[i])
//   nvfp4   9 B / 16 w   {e4m3 s; u8 qs[8]}     w[i] = s*e2m1(qs[i]&15), w[i+8] = s*e2m1(qs[i]>>4)
//   mxfp4  17 B / 32 w   {e8m0 e; u8 qs[16]}    w[i] = 2^(e-127)*e2m1(qs[i]&15), w[i+16] = high nibble
//
// Codec conventions of this contract: e4m3 has no NaN/inf codes (exponent 15 decodes all eight
// mantissas, max 480); e8m0 code 0 is 2^-127 and code 255 is +inf.
#pragma once

#include "qx_common.cuh"

namespace qx {

__device__ __forceinline__ float e4m3_to_f32(uint32_t c) {
  // normal: place (e,m) in the fp32 exponent/mantissa and rebias by 2^(127-7) via one multiply
  const uint32_t mag = c & 0x7Fu;
  float v = __uint_as_float(mag << 20) * 1.329227995784916e36f;  // 2^120; exact for subnormals too
  return (c & 0x80u) ? -v : v;
}
__device__ __forceinline__ float e2m1_to_f32(uint32_t n) {
  const uint32_t mag = n & 7u;
  float v = __uint_as_float(mag << 22) * 8.507059173023462e37f;  // 2^126
  return (n & 8u) ? -v : v;
}
__device__ __forceinline__ float e8m0_to_f32(uint32_t c) {
  return __uint_as_float(c == 0 ? 0x00400000u : (c << 23));
}
__device__ __forceinline__ float f16_bits_to_f32(uint32_t lo, uint32_t hi) {
  return __half2float(__ushort_as_half((unsigned short)(lo | (hi << 8))));
}

// Decode the 32 consecutive columns [32*span, 32*span+32) of one packed row into fp32.
// `row` points at the first byte of the row.  Works for any byte alignment.
template <int FMT>
__device__ __forceinline__ void decode_span32(const uint8_t* __restrict__ row, int span,
                                              float (&w)[32]) {
  if constexpr (FMT == F_Q4_0) {
    const uint8_t* b = row + (size_t)span * 18;
    const float d = f16_bits_to_f32(b[0], b[1]);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t q = b[2 + i];
      w[i] = d * (float)((int)(q & 15u) - 8);
      w[i + 16] = d * (float)((int)(q >> 4) - 8);
    }
  } else if constexpr (FMT == F_Q8_0) {
    const uint8_t* b = row + (size_t)span * 34;
    const float d = f16_bits_to_f32(b[0], b[1]);
#pragma unroll
    for (int i = 0; i < 32; ++i) w[i] = d * (float)(int8_t)b[2 + i];
  } else if constexpr (FMT == F_Q6_K) {
    const uint8_t* b = row + (size_t)(span >> 3) * 210;
    const int j = span & 7, chunk = j >> 2, group = j & 3;
    const float d = f16_bits_to_f32(b[208], b[209]);
    const uint8_t* ql = b + chunk * 64 + 32 * (group & 1);
    const uint8_t* qh = b + 128 + chunk * 32;
    const int8_t* sc = (const int8_t*)(b + 192 + chunk * 8 + 2 * group);
    const float s0 = d * (float)sc[0], s1 = d * (float)sc[1];
#pragma unroll
    for (int l = 0; l < 32; ++l) {
      const uint32_t byte = ql[l];
      const uint32_t nib = (group & 2) ? (byte >> 4) : (byte & 15u);
      const uint32_t hb = ((uint32_t)qh[l] >> (2 * group)) & 3u;
      const int q = (int)(nib | (hb << 4)) - 32;
      w[l] = (l < 16 ? s0 : s1) * (float)q;
    }
  } else if constexpr (FMT == F_MXFP8) {
    const uint8_t* b = row + (size_t)span * 33;
    const float s = e8m0_to_f32(b[0]);
#pragma unroll
    for (int i = 0; i < 32; ++i) w[i] = s * e4m3_to_f32(b[1 + i]);
  } else if constexpr (FMT == F_NVFP4) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint8_t* b = row + ((size_t)span * 2 + h) * 9;
      const float s = e4m3_to_f32(b[0]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t q = b[1 + i];
        w[16 * h + i] = s * e2m1_to_f32(q & 15u);
        w[16 * h + i + 8] = s * e2m1_to_f32(q >> 4);
      }
    }
  } else {  // F_MXFP4
    const uint8_t* b = row + (size_t)span * 17;
    const float s = e8m0_to_f32(b[0]);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t q = b[1 + i];
      w[i] = s * e2m1_to_f32(q & 15u);
      w[i + 16] = s * e2m1_to_f32(q >> 4);
    }
  }
}

}  // namespace qx
