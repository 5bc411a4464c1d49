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

// ------------------------------------------------------------------------------------------------
// Word-based decoders: the same values as decode_span32, built from 32-bit loads and a few
// logic / FMA instructions per weight instead of one byte load and one conversion per weight.
// ------------------------------------------------------------------------------------------------
namespace qx {

// NW 32-bit words starting at byte address p (any alignment), assembled from the NW + 1 aligned
// words that enclose them.  Aligned words that start at or beyond `limit` (the end of the tensor,
// 4-byte aligned) are not read: the span of the last row may end right at the end of an allocation.
template <int NW>
__device__ __forceinline__ void load_words_any(const uint8_t* p, const uint8_t* limit, uint32_t (&r)[NW]) {
  const uint32_t* base = reinterpret_cast<const uint32_t*>((uintptr_t)p & ~(uintptr_t)3);
  const uint32_t* lim = reinterpret_cast<const uint32_t*>(limit);
  const uint32_t sh = (uint32_t)((uintptr_t)p & 3) * 8u;
  uint32_t prev = base < lim ? base[0] : 0u;
#pragma unroll
  for (int i = 0; i < NW; ++i) {
    const uint32_t next = (base + i + 1) < lim ? base[i + 1] : 0u;
    r[i] = __funnelshift_r(prev, next, sh);
    prev = next;
  }
}
// float(8388608 + byte k of w): the byte placed under the fp32 pattern of 2^23
template <int K>
__device__ __forceinline__ float magic_byte(uint32_t w) {
  return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 | K));
}
__device__ __forceinline__ float2 f16x2_to_f32(uint32_t h) {
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}
__device__ __forceinline__ uint32_t cvt_e2m1_pair(uint32_t byte_in_low_bits) {
  uint32_t r;
  asm("{ .reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0; }"
      : "=r"(r) : "r"(byte_in_low_bits));
  return r;
}
__device__ __forceinline__ uint32_t cvt_e4m3_pair(uint32_t two_bytes_in_low_bits) {
  uint32_t r;
  asm("{ .reg .b16 h0, h1;\n\t"
      "mov.b32 {h0, h1}, %1;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, h0; }"
      : "=r"(r) : "r"(two_bytes_in_low_bits));
  return r;
}

// 16 e2m1 codes of 8 bytes in the block order "low nibbles first, then high nibbles"
// (columns i and i + NB/... as the format defines) are handled by the callers; this converts the
// two codes of one byte: .x = low nibble, .y = high nibble.
__device__ __forceinline__ float2 e2m1_byte_to_f32(uint32_t w, int byte_index) {
  return f16x2_to_f32(cvt_e2m1_pair(w >> (8 * byte_index)));
}

// The raw bytes of one 32-column span held in registers: load() can be issued one step ahead of
// decode(), which hides the memory latency behind the previous span's arithmetic.
// f16 pair -> bf16 pair scaled by `mult` (a bf16 pair holding scale * 2^112): moving the f16
// exponent / mantissa bits down by three places reads, as bf16, as value * 2^-112 (zero and f16
// subnormals included), and one bf16 multiply restores value * scale.  Exact whenever value * scale
// has at most 8 significant bits and stays in the bf16 range.
__device__ __forceinline__ uint32_t f16x2_to_bf16x2_scaled(uint32_t h, uint32_t mult) {
  const uint32_t t = ((h >> 3) & 0x0FFF0FFFu) | (h & 0x80008000u);
  __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&t),
                             *reinterpret_cast<const __nv_bfloat162*>(&mult));
  return *reinterpret_cast<uint32_t*>(&r);
}
// bf16 pair (s * 2^112, s * 2^112) for an e4m3 scale byte (this contract: 0x7F decodes to 480)
__device__ __forceinline__ uint32_t e4m3_scale_mult(uint32_t sc) {
  // e4m3 bits under the bf16 exponent read as s * 2^-120 (subnormal scales included);
  // two exact multiplies (2^120, then 2^112) avoid an unrepresentable 2^232
  uint32_t t = ((sc & 0x7Fu) << 4) | ((sc & 0x80u) << 8);
  t |= t << 16;
  const uint32_t k120 = 0x7B807B80u, k112 = 0x77807780u;
  __nv_bfloat162 a = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&t), *reinterpret_cast<const __nv_bfloat162*>(&k120));
  a = __hmul2(a, *reinterpret_cast<const __nv_bfloat162*>(&k112));
  return *reinterpret_cast<uint32_t*>(&a);
}

template <int FMT> struct RawSpan {
  static constexpr int NW = FMT == F_Q8_0 ? 9 : (FMT == F_MXFP8 ? 9 : 5);
  uint32_t r[NW];
  const uint8_t* row; int span;                              // q6_K decodes from memory directly

  // limit = first byte after the packed tensor (must be 4-byte aligned)
  __device__ __forceinline__ void load(const uint8_t* __restrict__ row_, int span_,
                                       const uint8_t* __restrict__ limit) {
    row = row_; span = span_;
    if constexpr (FMT == F_Q8_0) load_words_any<9>(row_ + (size_t)span_ * 34, limit, r);
    else if constexpr (FMT == F_MXFP8) load_words_any<9>(row_ + (size_t)span_ * 33, limit, r);
    else if constexpr (FMT == F_Q4_0) load_words_any<5>(row_ + (size_t)span_ * 18, limit, r);
    else if constexpr (FMT == F_MXFP4) load_words_any<5>(row_ + (size_t)span_ * 17, limit, r);
    else if constexpr (FMT == F_NVFP4) load_words_any<5>(row_ + (size_t)span_ * 18, limit, r);
  }

  // One-term formats: the 32 weights as 16 bf16 pairs in column order, exact, without fp32.
  // Returns false when the block scale is outside the range this shortcut covers (the caller
  // then takes decode()).
  __device__ __forceinline__ bool decode_bf16(uint32_t (&pk)[16]) const {
    if constexpr (FMT == F_NVFP4) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t sc = h == 0 ? (r[0] & 0xFFu) : ((r[2] >> 8) & 0xFFu);
        const uint32_t mult = e4m3_scale_mult(sc);
        uint32_t c0, c1;
        if (h == 0) { c0 = __funnelshift_r(r[0], r[1], 8); c1 = __funnelshift_r(r[1], r[2], 8); }
        else { c0 = __funnelshift_r(r[2], r[3], 16); c1 = __funnelshift_r(r[3], r[4], 16); }
        // byte i holds columns i (low nibble) and i + 8 (high nibble) of the block
        uint32_t lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t v = f16x2_to_bf16x2_scaled(cvt_e2m1_pair((i < 4 ? c0 : c1) >> (8 * (i & 3))), mult);
          lo[i] = v & 0xFFFFu; hi[i] = v >> 16;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          pk[8 * h + i] = lo[2 * i] | (lo[2 * i + 1] << 16);
          pk[8 * h + 4 + i] = hi[2 * i] | (hi[2 * i + 1] << 16);
        }
      }
      return true;
    } else if constexpr (FMT == F_MXFP4) {
      const uint32_t e = r[0] & 0xFFu;
      if (e < 16u || e > 140u) return false;               // 2^(e-127) * 2^112 must be a normal bf16
      uint32_t mult = (e + 112u - 127u + 127u) << 7;        // bf16 bits of 2^(e - 127 + 112)
      mult |= mult << 16;
      uint32_t c[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) c[i] = __funnelshift_r(r[i], r[i + 1], 8);
      uint32_t lo[16], hi[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t v = f16x2_to_bf16x2_scaled(cvt_e2m1_pair(c[i >> 2] >> (8 * (i & 3))), mult);
        lo[i] = v & 0xFFFFu; hi[i] = v >> 16;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        pk[i] = lo[2 * i] | (lo[2 * i + 1] << 16);
        pk[8 + i] = hi[2 * i] | (hi[2 * i + 1] << 16);
      }
      return true;
    } else {
      return false;
    }
  }

  __device__ __forceinline__ void decode(float (&w)[32]) const {
    if constexpr (FMT == F_Q8_0) {
      const float d = __half2float(__ushort_as_half((unsigned short)(r[0] & 0xFFFFu)));
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int b = 2 + i;                                 // bytes 2..33, sign bit flipped: q + 128
        const uint32_t word = r[b >> 2] ^ 0x80808080u;
        float m;
        if ((b & 3) == 0) m = magic_byte<0>(word);
        else if ((b & 3) == 1) m = magic_byte<1>(word);
        else if ((b & 3) == 2) m = magic_byte<2>(word);
        else m = magic_byte<3>(word);
        w[i] = (m - 8388736.0f) * d;                         // (2^23 + q + 128) - (2^23 + 128) = q, exact
      }
    } else if constexpr (FMT == F_Q4_0) {
      const float d = __half2float(__ushort_as_half((unsigned short)(r[0] & 0xFFFFu)));
      uint32_t c[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) c[i] = __funnelshift_r(r[i], r[i + 1], 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t lo = c[i] & 0x0F0F0F0Fu, hi = (c[i] >> 4) & 0x0F0F0F0Fu;
        w[4 * i + 0] = (magic_byte<0>(lo) - 8388616.0f) * d; w[4 * i + 1] = (magic_byte<1>(lo) - 8388616.0f) * d;
        w[4 * i + 2] = (magic_byte<2>(lo) - 8388616.0f) * d; w[4 * i + 3] = (magic_byte<3>(lo) - 8388616.0f) * d;
        w[16 + 4 * i + 0] = (magic_byte<0>(hi) - 8388616.0f) * d; w[16 + 4 * i + 1] = (magic_byte<1>(hi) - 8388616.0f) * d;
        w[16 + 4 * i + 2] = (magic_byte<2>(hi) - 8388616.0f) * d; w[16 + 4 * i + 3] = (magic_byte<3>(hi) - 8388616.0f) * d;
      }
    } else if constexpr (FMT == F_MXFP4) {
      const float s = e8m0_to_f32(r[0] & 0xFFu);
      uint32_t c[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) c[i] = __funnelshift_r(r[i], r[i + 1], 8);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float2 v = e2m1_byte_to_f32(c[i >> 2], i & 3);
        w[i] = s * v.x; w[i + 16] = s * v.y;
      }
    } else if constexpr (FMT == F_NVFP4) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {                          // block h occupies bytes 9h .. 9h+8
        const uint32_t sc = h == 0 ? (r[0] & 0xFFu) : ((r[2] >> 8) & 0xFFu);
        const float s = e4m3_to_f32(sc);
        uint32_t c0, c1;
        if (h == 0) { c0 = __funnelshift_r(r[0], r[1], 8); c1 = __funnelshift_r(r[1], r[2], 8); }
        else { c0 = __funnelshift_r(r[2], r[3], 16); c1 = __funnelshift_r(r[3], r[4], 16); }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 v = e2m1_byte_to_f32(i < 4 ? c0 : c1, i & 3);
          w[16 * h + i] = s * v.x; w[16 * h + i + 8] = s * v.y;
        }
      }
    } else if constexpr (FMT == F_MXFP8) {
      const float s = e8m0_to_f32(r[0] & 0xFFu);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int b = 1 + i;
        w[i] = s * e4m3_to_f32((r[b >> 2] >> (8 * (b & 3))) & 0xFFu);
      }
    } else {
      decode_span32<FMT>(row, span, w);                      // q6_K: byte-wise form
    }
  }
};

}  // namespace qx
