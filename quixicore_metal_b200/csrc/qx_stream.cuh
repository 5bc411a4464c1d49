// Streaming small-batch core: packed weight rows -> shared memory by 2-D TMA box copies,
// in-register dequantisation straight into mma.sync A fragments, fp32 block-scaled accumulation.
//
// Why this shape.  For batch <= 16 the projection is bound by the HBM stream of packed weights
// (0.53 - 1.06 bytes per weight).  At 6.5 TB/s an SM has to retire ~40 four-bit weights per clock,
// i.e. at most ~3 issue slots per weight: fp32 FMAs plus scalar conversions do not fit, so
//   * the multiply-accumulate runs on the tensor cores (m16n8k16 f16, the batch is the n = 8
//     dimension, 16 weight rows are the m dimension) with A built in registers - the dequantised
//     weights never touch shared memory;
//   * integer / logic / half2 instructions issue at half the fp32 rate on this part, so codes are
//     turned into f16 with the cheapest exact sequence per format (magic-number OR for integers,
//     the hardware e2m1 / e4m3 converters for the float codes);
//   * every scale unit (16 or 32 columns sharing one scale) is multiplied as exact small numbers
//     and the fp16 / e8m0 scale is applied to the fp32 partial sum afterwards (nvfp4 folds its e4m3
//     scale into the f16 weight, which is exact), so the result equals fp32 dequantise-then-dot up
//     to summation order;
//   * activations are converted once per call to f16, each row scaled by a power of two so that
//     its largest magnitude sits near 2^14 (exact for every element within 2^28 of the row maximum,
//     i.e. far below the resolution of the fp32 accumulator for the rest), stored in the column
//     order the decoders produce; the epilogue multiplies the row scale back;
//   * raw rows are fetched as 2-D TMA boxes (16 rows per copy) into a per-warp ring of stages
//     (mbarrier completion), which keeps 70 - 150 KB in flight per SM with a handful of instructions.
// The k-order inside a scale unit is free (a dot product is order-blind up to rounding), so each
// thread takes the bytes that are cheapest to unpack and loads the matching activation columns.
//
// Every mbarrier wait is bounded; on expiry the warp raises the device error flag and stops computing.
#pragma once

#include <cuda.h>

#include "qx_common.cuh"

namespace qx {


// ---- PTX wrappers ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait: returns false (and records the failure) if the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err_flag) {
  for (int i = 0; i < (1 << 22); ++i)
    if (mbar_try_wait(bar, parity)) return true;
  atomicExch(err_flag, 1);
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// One 2-D TMA box (tensor map coordinates x = 32-bit word inside the row, y = row) -> shared memory.
__device__ __forceinline__ void tma_box_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Shared-memory loads by 32-bit shared-window address.  Deliberately not volatile: the compiler
// may hoist and interleave them; the mbarrier wait / __syncwarp carry the memory clobbers that
// keep them inside their pipeline stage.
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
  uint16_t v;
  asm("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
// 32 bits starting at an arbitrary shared-memory byte address (reads the two enclosing words)
__device__ __forceinline__ uint32_t lds32_any(uint32_t addr) {
  const uint32_t base = addr & ~3u;
  return __funnelshift_r(lds32(base), lds32(base + 4), (addr & 3u) * 8u);
}
// 32 bits at a 2-byte aligned address
__device__ __forceinline__ uint32_t lds32_a2(uint32_t addr) {
  return lds16(addr) | (lds16(addr + 2) << 16);
}

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// d = a * b (+ 0): the zero C operand is a constant, so no accumulator has to be cleared first
__device__ __forceinline__ void mma_f16_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ uint32_t h2sub(uint32_t a, uint32_t b) {
  uint32_t r; asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}
__device__ __forceinline__ uint32_t h2mul(uint32_t a, uint32_t b) {
  uint32_t r; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b)); return r;
}
__device__ __forceinline__ uint32_t h2fma(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c)); return r;
}
// byte `i` of w holds two e2m1 codes: low nibble -> low half, high nibble -> high half
template <int I>
__device__ __forceinline__ uint32_t cvt_e2m1x2(uint32_t w) {
  uint32_t r;
  asm("{ .reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b%2; }"
      : "=r"(r) : "r"(w), "n"(I));
  return r;
}
// half `I` (0/1) of w holds two e4m3 codes -> f16 pair (hardware rule: 0x7F / 0xFF decode to NaN)
template <int I>
__device__ __forceinline__ uint32_t cvt_e4m3x2(uint32_t w) {
  uint32_t r;
  asm("{ .reg .b16 h0, h1;\n\t"
      "mov.b32 {h0, h1}, %1;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, h%2; }"
      : "=r"(r) : "r"(w), "n"(I));
  return r;
}
__device__ __forceinline__ float f16lo_to_f32(uint32_t h) {
  return __half2float(__ushort_as_half((unsigned short)(h & 0xFFFFu)));
}

// ---- per-format geometry ----------------------------------------------------------------------
// UNIT  = columns that share one scale and are multiplied before the scale is applied;
// GROUP = columns one decode step covers (the byte-alignment pattern of the blocks repeats with
//         this period, so every shared-memory load inside a step has a static alignment);
// KC    = columns one pipeline stage holds per row (a multiple of GROUP whose byte size is a
//         multiple of 16, except q6_K whose 210-byte blocks are only 4-byte periodic);
// PERM  = column order of the prepared activations (see prep_activations_kernel).
template <int FMT> struct StreamFmt;
template <> struct StreamFmt<F_Q4_0>  { static constexpr int UNIT = 32, GROUP = 64,  KC = 512, BK = 32,  BB = 18,  PERM = 1; };
template <> struct StreamFmt<F_Q8_0>  { static constexpr int UNIT = 32, GROUP = 64,  KC = 256, BK = 32,  BB = 34,  PERM = 0; };
template <> struct StreamFmt<F_Q6_K>  { static constexpr int UNIT = 16, GROUP = 512, KC = 512, BK = 256, BB = 210, PERM = 4; };
template <> struct StreamFmt<F_MXFP8> { static constexpr int UNIT = 32, GROUP = 128, KC = 256, BK = 32,  BB = 33,  PERM = 0; };
template <> struct StreamFmt<F_NVFP4> { static constexpr int UNIT = 16, GROUP = 64,  KC = 512, BK = 16,  BB = 9,   PERM = 3; };
template <> struct StreamFmt<F_MXFP4> { static constexpr int UNIT = 32, GROUP = 128, KC = 512, BK = 32,  BB = 17,  PERM = 2; };

template <int FMT, int KCV>
struct StageGeom {
  using F = StreamFmt<FMT>;
  static constexpr int KC = KCV;
  static constexpr int CHUNK_BYTES = KC / F::BK * F::BB;          // payload bytes per row and stage
  // A stage is fetched as one TMA box of 16 rows.  The payload starts at a multiple of 4 inside
  // the row but not always of 16, so the box starts at the 16-byte boundary below and is wide
  // enough for the largest misalignment; its width (= the row pitch in shared memory) is an odd
  // multiple of 16 bytes, so the 8 rows a warp touches in one instruction start in different
  // 16-byte bank groups (no shared-memory bank conflicts).
  static constexpr int ALIGN = (CHUNK_BYTES % 16 == 0) ? 16 : ((CHUNK_BYTES % 8 == 0) ? 8 : 4);
  static constexpr int PITCH = (((CHUNK_BYTES + 16 - ALIGN + 15) / 16) | 1) * 16;
  static_assert(PITCH / 4 <= 256, "a TMA box is at most 256 elements wide");
};

// Position of column c (0 <= c < 32) of a 32-column group inside the prepared activation row.
// PERM 0: natural.  The others put the columns a thread's decode produces next to each other so
// that one 8/16-byte load yields its B fragments:
//   1 (q4_0)  thread t: 4t,4t+2,4t+1,4t+3, 16+4t,16+4t+2,16+4t+1,16+4t+3
//   2 (mxfp4) thread t: 4t,16+4t, 4t+1,16+4t+1, 4t+2,16+4t+2, 4t+3,16+4t+3
//   3 (nvfp4) per 16:   0,8,1,9,2,10,3,11,4,12,5,13,6,14,7,15
//   4 (q6_K)  per 4:    0,2,1,3
//   5 (BaseQN) per 8:   0,4,1,5,2,6,3,7
__host__ __device__ inline int perm_position(int perm, int c) {
  switch (perm) {
    case 1: { const int hi = c >> 4, r = c & 15, t = r >> 2, i = r & 3;
              return 8 * t + 4 * hi + ((i & 1) << 1 | (i >> 1)); }
    case 2: { const int hi = c >> 4, r = c & 15, t = r >> 2, i = r & 3;
              return 8 * t + 2 * i + hi; }
    case 3: { const int blk = c >> 4, r = c & 15;
              return 16 * blk + ((r & 7) << 1 | (r >> 3)); }
    case 4: { const int i = c & 3;
              return (c & ~3) | ((i & 1) << 1 | (i >> 1)); }
    case 5: { const int i = c & 7;
              return (c & ~7) | ((i & 3) << 1 | (i >> 2)); }
    default: return c;
  }
}

// ---- row decoders for the formats with a post-applied scale (unit = 32 columns) ------------------
// row<J>(s, t, a, scale): s = shared address of the block of unit J (J = position inside the
// group, which fixes the byte alignment), t = lane & 3.  a[m][0] feeds k-slots (2t, 2t+1) of MMA m,
// a[m][1] slots (2t+8, 2t+9); the matching activation order is StreamFmt::PERM.
template <int FMT> struct RowDec;

template <> struct RowDec<F_Q8_0> {
  // thread t owns code bytes 8t..8t+7 (columns 8t..8t+7); q + 1152 is built by OR-ing the byte
  // (sign bit flipped) under the f16 exponent of 1024, then 1152 is subtracted: exact.
  __device__ __forceinline__ static void word(uint32_t w, uint32_t& p01, uint32_t& p23) {
    const uint32_t u = w ^ 0x80808080u;
    p01 = h2sub(__byte_perm(u, 0x64646464u, 0x4140), 0x64806480u);
    p23 = h2sub(__byte_perm(u, 0x64646464u, 0x4342), 0x64806480u);
  }
  // load<J> / convert / scale: the two halves of row<J>, for callers that want all the shared-memory
  // loads of a stage in flight before the first conversion
  static constexpr int RAWN = 2;
  template <int J>
  __device__ __forceinline__ static void load(uint32_t s, int t, uint32_t (&raw)[2], uint32_t& sc) {
    sc = lds16(s);
    if constexpr ((J & 1) == 0) {            // block starts 4-aligned: codes at +2 straddle words
      const uint32_t p = s + 8 * t;
      const uint32_t x0 = lds32(p), x1 = lds32(p + 4), x2 = lds32(p + 8);
      raw[0] = __funnelshift_r(x0, x1, 16); raw[1] = __funnelshift_r(x1, x2, 16);
    } else {                                 // block starts at 2 mod 4: codes are word aligned
      const uint32_t p = s + 2 + 8 * t;
      raw[0] = lds32(p); raw[1] = lds32(p + 4);
    }
  }
  __device__ __forceinline__ static void convert(const uint32_t (&raw)[2], uint32_t (&a)[2][2]) {
    word(raw[0], a[0][0], a[0][1]);
    word(raw[1], a[1][0], a[1][1]);
  }
  __device__ __forceinline__ static float scale(uint32_t sc) { return f16lo_to_f32(sc); }
  template <int J>
  __device__ __forceinline__ static void row(uint32_t s, int t, uint32_t (&a)[2][2], float& sc_out) {
    uint32_t raw[2], sc;
    load<J>(s, t, raw, sc);
    convert(raw, a);
    sc_out = scale(sc);
  }
};

template <> struct RowDec<F_Q4_0> {
  // thread t owns code bytes 4t..4t+3: low nibbles = columns 4t.., high nibbles = columns 16+4t..
  // A nibble placed under the f16 exponent of 1024 (0x6400 | n) is 1024 + n; subtracting 1032 centres it.
  static constexpr int RAWN = 1;
  template <int J>
  __device__ __forceinline__ static void load(uint32_t s, int t, uint32_t (&raw)[1], uint32_t& sc) {
    sc = lds16(s);
    if constexpr ((J & 1) == 0) {
      const uint32_t p = s + 4 * t;
      raw[0] = __funnelshift_r(lds32(p), lds32(p + 4), 16);
    } else {
      raw[0] = lds32(s + 2 + 4 * t);
    }
  }
  __device__ __forceinline__ static float scale(uint32_t sc) { return f16lo_to_f32(sc); }
  template <int J>
  __device__ __forceinline__ static void row(uint32_t s, int t, uint32_t (&a)[2][2], float& sc_out) {
    uint32_t raw[1], sc;
    load<J>(s, t, raw, sc);
    convert(raw, a);
    sc_out = scale(sc);
  }
  __device__ __forceinline__ static void convert(const uint32_t (&raw)[1], uint32_t (&a)[2][2]) {
    // nibbles byte-wise, then each pair of bytes under the f16 exponent of 1024 by one byte permute
    const uint32_t lo = raw[0] & 0x0F0F0F0Fu, hi = (raw[0] >> 4) & 0x0F0F0F0Fu;
    a[0][0] = h2sub(__byte_perm(lo, 0x64646464u, 0x4240), 0x64086408u);     // bytes 0,2 low nibbles
    a[0][1] = h2sub(__byte_perm(lo, 0x64646464u, 0x4341), 0x64086408u);     // bytes 1,3 low nibbles
    a[1][0] = h2sub(__byte_perm(hi, 0x64646464u, 0x4240), 0x64086408u);     // bytes 0,2 high nibbles
    a[1][1] = h2sub(__byte_perm(hi, 0x64646464u, 0x4341), 0x64086408u);     // bytes 1,3 high nibbles
  }
};

// 2^(e - 127) for an e8m0 code: code 0 is the subnormal 2^-127, whose bit pattern 0x00400000 is
// smaller than every shifted non-zero code, so one max replaces the compare-and-select.
__device__ __forceinline__ float e8m0_scale(uint32_t e) {
  return __uint_as_float(max(e << 23, 0x00400000u));
}

template <> struct RowDec<F_MXFP4> {
  // thread t owns code bytes 4t..4t+3; byte i converts to the pair (column 4t+i, column 16+4t+i)
  static constexpr int RAWN = 1;
  template <int J>
  __device__ __forceinline__ static void load(uint32_t s, int t, uint32_t (&raw)[1], uint32_t& sc) {
    sc = lds8(s);
    constexpr int SH = (J + 1) & 3;          // (17*J + 1) mod 4
    const uint32_t p = s + 1 + 4 * t - SH;
    if constexpr (SH == 0) raw[0] = lds32(p);
    else raw[0] = __funnelshift_r(lds32(p), lds32(p + 4), 8 * SH);
  }
  __device__ __forceinline__ static void convert(const uint32_t (&raw)[1], uint32_t (&a)[2][2]) {
    const uint32_t w = raw[0];
    a[0][0] = cvt_e2m1x2<0>(w); a[0][1] = cvt_e2m1x2<1>(w);
    a[1][0] = cvt_e2m1x2<2>(w); a[1][1] = cvt_e2m1x2<3>(w);
  }
  __device__ __forceinline__ static float scale(uint32_t sc) { return e8m0_scale(sc); }
  template <int J>
  __device__ __forceinline__ static void row(uint32_t s, int t, uint32_t (&a)[2][2], float& sc_out) {
    uint32_t raw[1], sc;
    load<J>(s, t, raw, sc);
    convert(raw, a);
    sc_out = scale(sc);
  }
};

// e4m3 pair with this contract's rule for the codes 0x7F / 0xFF (+-480, no NaN): bits moved into
// the f16 exponent / mantissa decode to value * 2^-8 (subnormals included), times 2^8 is exact.
__device__ __forceinline__ uint32_t e4m3x2_exact(uint32_t h) {          // bytes at [7:0] and [23:16]
  const uint32_t bits = ((h & 0x007F007Fu) << 7) | ((h & 0x00800080u) << 8);
  return h2mul(bits, 0x5C005C00u);
}
template <> struct RowDec<F_MXFP8> {
  __device__ __forceinline__ static void word(uint32_t w, uint32_t& p01, uint32_t& p23) {
    const uint32_t t7 = w & 0x7F7F7F7Fu;
    if (((t7 + 0x01010101u) & 0x80808080u) != 0u) {    // some byte is 0x7F: the hardware would say NaN
      p01 = e4m3x2_exact(__byte_perm(w, 0u, 0x4140));
      p23 = e4m3x2_exact(__byte_perm(w, 0u, 0x4342));
    } else {
      p01 = cvt_e4m3x2<0>(w);
      p23 = cvt_e4m3x2<1>(w);
    }
  }
  static constexpr int RAWN = 2;
  template <int J>
  __device__ __forceinline__ static void load(uint32_t s, int t, uint32_t (&raw)[2], uint32_t& sc) {
    sc = lds8(s);
    constexpr int SH = (J + 1) & 3;          // (33*J + 1) mod 4
    const uint32_t p = s + 1 + 8 * t - SH;
    if constexpr (SH == 0) { raw[0] = lds32(p); raw[1] = lds32(p + 4); }
    else {
      const uint32_t x0 = lds32(p), x1 = lds32(p + 4), x2 = lds32(p + 8);
      raw[0] = __funnelshift_r(x0, x1, 8 * SH); raw[1] = __funnelshift_r(x1, x2, 8 * SH);
    }
  }
  __device__ __forceinline__ static void convert(const uint32_t (&raw)[2], uint32_t (&a)[2][2]) {
    word(raw[0], a[0][0], a[0][1]);
    word(raw[1], a[1][0], a[1][1]);
  }
  __device__ __forceinline__ static float scale(uint32_t sc) { return e8m0_scale(sc); }
  template <int J>
  __device__ __forceinline__ static void row(uint32_t s, int t, uint32_t (&a)[2][2], float& sc_out) {
    uint32_t raw[2], sc;
    load<J>(s, t, raw, sc);
    convert(raw, a);
    sc_out = scale(sc);
  }
};

// One 32-column unit of the post-scaled formats: decode 2 rows per set, one MMA pair per n-tile,
// then acc += scale * partial.  b[nt] = the thread's 8 prepared activations of this unit.
template <int FMT, int J, int NSETS, int NT>
__device__ __forceinline__ void unit32(const uint32_t (&s)[2 * NSETS], uint32_t boff, int t,
                                       const uint4 (&b)[NT], float (&acc)[NSETS][NT][4]) {
  uint32_t a[2 * NSETS][2][2];
  float sc[2 * NSETS];
#pragma unroll
  for (int r = 0; r < 2 * NSETS; ++r) RowDec<FMT>::template row<J>(s[r] + boff, t, a[r], sc[r]);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int set = 0; set < NSETS; ++set) {
      float p[4];
      mma_f16_zero(p, a[2 * set][0][0], a[2 * set + 1][0][0], a[2 * set][0][1], a[2 * set + 1][0][1], b[nt].x, b[nt].y);
      mma_f16(p, a[2 * set][1][0], a[2 * set + 1][1][0], a[2 * set][1][1], a[2 * set + 1][1][1], b[nt].z, b[nt].w);
      acc[set][nt][0] = fmaf(sc[2 * set], p[0], acc[set][nt][0]);
      acc[set][nt][1] = fmaf(sc[2 * set], p[1], acc[set][nt][1]);
      acc[set][nt][2] = fmaf(sc[2 * set + 1], p[2], acc[set][nt][2]);
      acc[set][nt][3] = fmaf(sc[2 * set + 1], p[3], acc[set][nt][3]);
    }
  }
}

__device__ __forceinline__ uint4 ldg_or_zero(const __half* row, int off) {
  return row ? __ldg(reinterpret_cast<const uint4*>(row + off)) : make_uint4(0u, 0u, 0u, 0u);
}
__device__ __forceinline__ uint2 ldg2_or_zero(const __half* row, int off) {
  return row ? __ldg(reinterpret_cast<const uint2*>(row + off)) : make_uint2(0u, 0u);
}
// A prepared activation row that lives in shared memory (batch 1, prepared by the consuming kernel
// itself): shared-window address of its first element, 0 = no row.  The group processors take the row
// pointers as a template type, so the same code reads the row from global memory or from here.
struct SmemRow { uint32_t addr; };
__device__ __forceinline__ uint4 ldg_or_zero(SmemRow row, int off) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (row.addr) asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(row.addr + 2u * (uint32_t)off));
  return v;
}
__device__ __forceinline__ uint2 ldg2_or_zero(SmemRow row, int off) {
  uint2 v = make_uint2(0u, 0u);
  if (row.addr) asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(row.addr + 2u * (uint32_t)off));
  return v;
}

// One activation row prepared by the whole CTA into shared memory, with the arithmetic of the
// preparation kernel: largest finite magnitude -> power-of-two scale 2^-S that puts it in [2^14, 2^15)
// -> xs[perm(c)] = f16(x[c] * 2^-S); *rs = 2^S.  xsrc: the raw 16-bit row (bf16 if x_bf16, else f16),
// 16-byte aligned, K % 8 == 0.  Layout at xs_base: K halves, the scale, 32 floats of scratch.
// Every thread of the CTA calls it (it contains CTA barriers).
template <int PERM>
__device__ __forceinline__ void cta_prepare_row(uint8_t* xs_base, const uint16_t* __restrict__ xsrc, int x_bf16, int K) {
  __half* xs = reinterpret_cast<__half*>(xs_base);
  float* rs_s = reinterpret_cast<float*>(xs_base + (size_t)K * 2);
  float* red = rs_s + 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const uint4* xv = reinterpret_cast<const uint4*>(xsrc);
  auto widen = [&](uint16_t b) {
    return x_bf16 ? __uint_as_float((uint32_t)b << 16) : __half2float(__ushort_as_half(b));
  };
  float amax = 0.f;
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
    const uint4 v = __ldg(xv + i);
    const uint16_t* e = reinterpret_cast<const uint16_t*>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = fabsf(widen(e[j]));
      if (a < 3.0e38f) amax = fmaxf(amax, a);          // inf / nan do not choose the scale
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  amax = 0.f;
  for (int i = 0; i < nwarps; ++i) amax = fmaxf(amax, red[i]);
  int S = 0;
  if (amax > 0.f) {
    S = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 127 - 14;
    S = max(-110, min(110, S));
  }
  const float down = __uint_as_float((uint32_t)(127 - S) << 23);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
    const uint4 v = __ldg(xv + i);
    const uint16_t* e = reinterpret_cast<const uint16_t*>(&v);
    const int c0 = 8 * i;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      xs[(c0 & ~31) + perm_position(PERM, (c0 & 31) + j)] = __float2half_rn(widen(e[j]) * down);
  }
  if (threadIdx.x == 0) *rs_s = __uint_as_float((uint32_t)(127 + S) << 23);
  __syncthreads();
}
constexpr size_t cta_prepared_row_bytes(size_t K) { return K * 2 + 4 + 32 * 4; }

// ---- group processors: one GROUP of columns for this thread's rows ---------------------------------
// s[r]: shared address of column 0 of the group in row slot r (r = 0,1: rows g, g+8 of the gate /
// only matrix; r = 2,3: the same rows of the up matrix).  The thread's prepared activations of the
// group are fetched by load_b() one group ahead of run(), which hides the L1 latency.
template <int FMT> struct GroupProc {
  using F = StreamFmt<FMT>;
  static constexpr int UNITS = F::GROUP / 32;
  static constexpr bool PIPED = true;       // has the unit-pipelined form for large batches
  static constexpr float ACC_SCALE = 1.f;   // run() accumulates dot products / ACC_SCALE
  template <int NT> struct BFrag { uint4 v[UNITS][NT]; };
  template <int NT, class XP>
  __device__ __forceinline__ static void load_b(const XP (&xr)[NT], int col, int t,
                                                BFrag<NT>& b) {
#pragma unroll
    for (int u = 0; u < UNITS; ++u)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) b.v[u][nt] = ldg_or_zero(xr[nt], col + 32 * u + 8 * t);
  }
  // PRE: the fragments were fetched one group ahead into `b` (small batches); otherwise they are
  // loaded unit by unit from xr / col (large batches, where a whole group would not fit registers).
  template <int NSETS, int NT, bool PRE, int J, class XP>
  __device__ __forceinline__ static void one(const uint32_t (&s)[2 * NSETS], int t, const BFrag<NT>& b,
                                             const XP (&xr)[NT], int col,
                                             float (&acc)[NSETS][NT][4]) {
    if constexpr (PRE) {
      unit32<FMT, J, NSETS, NT>(s, (uint32_t)(J * F::BB), t, b.v[J], acc);
    } else {
      uint4 bb[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) bb[nt] = ldg_or_zero(xr[nt], col + 32 * J + 8 * t);
      unit32<FMT, J, NSETS, NT>(s, (uint32_t)(J * F::BB), t, bb, acc);
    }
  }
  template <int NSETS, int NT, bool PRE, class XP>
  __device__ __forceinline__ static void run(const uint32_t (&s)[2 * NSETS], int t,
                                             const BFrag<NT>& b, const XP (&xr)[NT],
                                             int col, float (&acc)[NSETS][NT][4]) {
    one<NSETS, NT, PRE, 0>(s, t, b, xr, col, acc);
    if constexpr (UNITS > 1) one<NSETS, NT, PRE, 1>(s, t, b, xr, col, acc);
    if constexpr (UNITS > 2) one<NSETS, NT, PRE, 2>(s, t, b, xr, col, acc);
    if constexpr (UNITS > 3) one<NSETS, NT, PRE, 3>(s, t, b, xr, col, acc);
  }
  // Large batches: the activation fragments of one unit (NT x 16 bytes) are fetched one unit ahead.
  // `carry` holds the fragments of this group's first unit on entry and those of the next group's
  // first unit on exit (when there is a next group).
  template <int NSETS, int NT, int J, class XP>
  __device__ __forceinline__ static void piped(const uint32_t (&s)[2 * NSETS], int t,
                                               const XP (&xr)[NT], int col, bool has_next,
                                               uint4 (&cur)[NT], float (&acc)[NSETS][NT][4]) {
    uint4 nxt[NT];
    if constexpr (J + 1 < UNITS) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) nxt[nt] = ldg_or_zero(xr[nt], col + 32 * (J + 1) + 8 * t);
    } else {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) nxt[nt] = has_next ? ldg_or_zero(xr[nt], col + F::GROUP + 8 * t) : make_uint4(0u, 0u, 0u, 0u);
    }
    unit32<FMT, J, NSETS, NT>(s, (uint32_t)(J * F::BB), t, cur, acc);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) cur[nt] = nxt[nt];
    if constexpr (J + 1 < UNITS) piped<NSETS, NT, J + 1>(s, t, xr, col, has_next, cur, acc);
  }
  template <int NT, class XP>
  __device__ __forceinline__ static void load_first(const XP (&xr)[NT], int col, int t,
                                                    uint4 (&cur)[NT]) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) cur[nt] = ldg_or_zero(xr[nt], col + 8 * t);
  }
};

// nvfp4: a group is four 16-column blocks; thread t owns block t of the group outright (9 bytes),
// folds the e4m3 scale into the f16 weights (exact: 4 x 2 significant bits) and feeds its block's
// byte pair (2m, 2m+1) to MMA m; the MMAs accumulate straight into acc.
// block<false>: the scale comes from the hardware converter (codes 0x7F / 0xFF, which it reads as
// NaN and this contract as +-480, are patched).  block<true>: the scale byte's exponent and mantissa
// bits are moved under the f16 exponent instead, which is the f16 pattern of scale * 2^-8 for every
// code (subnormals and 0x7F included) in two logic operations and needs no patch; weight x scale
// stays exact (a multiple of 2^-18 with at most 6 significant bits, f16 subnormals kept), and the
// caller multiplies its accumulators by ACC_SCALE = 2^8 once per output.
template <> struct GroupProc<F_NVFP4> {
  using F = StreamFmt<F_NVFP4>;
  static constexpr bool PIPED = false;
  static constexpr float ACC_SCALE = 256.f;
  template <bool PRESCALED = false>
  __device__ __forceinline__ static void block(uint32_t s, int t, uint32_t (&a)[4][2]) {
    const uint32_t p = s + (uint32_t)(9 * t & ~3);
    const uint32_t sh = 8u * (uint32_t)t;                 // (9t mod 4) bytes
    const uint32_t w0 = lds32(p), w1 = lds32(p + 4), w2 = lds32(p + 8);
    const uint32_t x0 = __funnelshift_r(w0, w1, sh), x1 = __funnelshift_r(w1, w2, sh), x2 = w2 >> sh;
    uint32_t s2;
    if constexpr (PRESCALED) {
      const uint32_t v = __byte_perm(x0, 0u, 0x0404);     // the scale byte at [15:8] and [31:24]
      s2 = ((v >> 1) & 0x3F803F80u) | (v & 0x80008000u);
    } else {
      s2 = cvt_e4m3x2<0>(__byte_perm(x0, 0u, 0x0000));
      if ((x0 & 0x7Fu) == 0x7Fu) s2 = (x0 & 0x80u) ? 0xDF80DF80u : 0x5F805F80u;   // +-480, not NaN
    }
    a[0][0] = h2mul(cvt_e2m1x2<1>(x0), s2); a[0][1] = h2mul(cvt_e2m1x2<2>(x0), s2);
    a[1][0] = h2mul(cvt_e2m1x2<3>(x0), s2); a[1][1] = h2mul(cvt_e2m1x2<0>(x1), s2);
    a[2][0] = h2mul(cvt_e2m1x2<1>(x1), s2); a[2][1] = h2mul(cvt_e2m1x2<2>(x1), s2);
    a[3][0] = h2mul(cvt_e2m1x2<3>(x1), s2); a[3][1] = h2mul(cvt_e2m1x2<0>(x2), s2);
  }
  template <int NT> struct BFrag { uint4 v[2][NT]; };
  template <int NT, class XP>
  __device__ __forceinline__ static void load_b(const XP (&xr)[NT], int col, int t,
                                                BFrag<NT>& b) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      b.v[0][nt] = ldg_or_zero(xr[nt], col + 16 * t);
      b.v[1][nt] = ldg_or_zero(xr[nt], col + 16 * t + 8);
    }
  }
  template <int NSETS, int NT, bool PRE, class XP>
  __device__ __forceinline__ static void run(const uint32_t (&s)[2 * NSETS], int t,
                                             const BFrag<NT>& b, const XP (&xr)[NT],
                                             int col, float (&acc)[NSETS][NT][4]) {
    uint32_t a[2 * NSETS][4][2];
#pragma unroll
    for (int r = 0; r < 2 * NSETS; ++r) block<true>(s[r], t, a[r]);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      uint4 b0, b1;
      if constexpr (PRE) { b0 = b.v[0][nt]; b1 = b.v[1][nt]; }
      else { b0 = ldg_or_zero(xr[nt], col + 16 * t); b1 = ldg_or_zero(xr[nt], col + 16 * t + 8); }
#pragma unroll
      for (int set = 0; set < NSETS; ++set) {
        mma_f16(acc[set][nt], a[2 * set][0][0], a[2 * set + 1][0][0], a[2 * set][0][1], a[2 * set + 1][0][1], b0.x, b0.y);
        mma_f16(acc[set][nt], a[2 * set][1][0], a[2 * set + 1][1][0], a[2 * set][1][1], a[2 * set + 1][1][1], b0.z, b0.w);
        mma_f16(acc[set][nt], a[2 * set][2][0], a[2 * set + 1][2][0], a[2 * set][2][1], a[2 * set + 1][2][1], b1.x, b1.y);
        mma_f16(acc[set][nt], a[2 * set][3][0], a[2 * set + 1][3][0], a[2 * set][3][1], a[2 * set + 1][3][1], b1.z, b1.w);
      }
    }
  }
};

// q6_K: a group is two 256-column super-blocks (420 bytes: the first starts 4-byte aligned, the
// second at 2 mod 4).  Thread t owns columns 16*sub + 4t .. +3 of every 16-column sub-block: a ql
// word serves two sub-blocks (low / high nibbles), a qh word four (2 bits each).  6-bit codes are
// OR-ed under the f16 exponent of 1024 as 1024+c or 1024+16c; sub-scale * d is applied in fp32.
template <> struct GroupProc<F_Q6_K> {
  using F = StreamFmt<F_Q6_K>;
  static constexpr bool PIPED = false;
  static constexpr float ACC_SCALE = 1.f;
  template <int ODD>
  __device__ __forceinline__ static uint32_t ldw(uint32_t p) {    // p is 4-aligned iff !ODD
    if constexpr (ODD) return __funnelshift_r(lds32(p - 2), lds32(p + 2), 16);
    else return lds32(p);
  }
  // codes of one sub-block for one row: Q = ql word, H = qh word.  Sub-block G of the four that
  // share the words takes the low (G < 2) or high nibbles of Q and bits 2G, 2G+1 of every H byte.
  // The four 6-bit codes are assembled byte-wise (two logic ops), then each pair of bytes is
  // spread under the f16 exponent of 1024 by one byte permute and centred by one subtraction:
  // a0 <- bytes 0 and 2, a1 <- bytes 1 and 3 (the activation order is StreamFmt::PERM = 4).
  template <int G>
  __device__ __forceinline__ static void pair(uint32_t Q, uint32_t H, uint32_t& a0, uint32_t& a1) {
    const uint32_t q4 = G < 2 ? Q : (Q >> 4);
    const uint32_t h2 = G == 0 ? (H << 4) : (G == 1 ? (H << 2) : (G == 2 ? H : (H >> 2)));
    const uint32_t c = (q4 & 0x0F0F0F0Fu) | (h2 & 0x30303030u);
    a0 = h2sub(__byte_perm(c, 0x64646464u, 0x4240), 0x64206420u);
    a1 = h2sub(__byte_perm(c, 0x64646464u, 0x4341), 0x64206420u);
  }
  template <int NT> struct BFrag { int col; };   // the fragments are fetched inside run()
  template <int NT, class XP>
  __device__ __forceinline__ static void load_b(const XP (&xr)[NT], int col, int,
                                                BFrag<NT>& b) {
    b.col = col;
  }
  template <int ODD, int NSETS, int NT, class XP>
  __device__ __forceinline__ static void superblock(const uint32_t (&s)[2 * NSETS], uint32_t boff,
                                                    int t, const XP (&xr)[NT], int col,
                                                    float (&acc)[NSETS][NT][4]) {
    float d[2 * NSETS];
#pragma unroll
    for (int r = 0; r < 2 * NSETS; ++r) d[r] = f16lo_to_f32(lds16(s[r] + boff + 208));
#pragma unroll
    for (int c = 0; c < 2; ++c) {                 // 128-column chunk
#pragma unroll
      for (int l = 0; l < 2; ++l) {               // which 16 of the 32 positions
        uint32_t H[2 * NSETS], Q0[2 * NSETS], Q1[2 * NSETS], SC[2 * NSETS][2];
        uint2 bq[4][NT];                          // activations of the four sub-blocks of this step
#pragma unroll
        for (int g = 0; g < 4; ++g)
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
            bq[g][nt] = ldg2_or_zero(xr[nt], col + 128 * c + 32 * g + 16 * l + 4 * t);
#pragma unroll
        for (int r = 0; r < 2 * NSETS; ++r) {
          const uint32_t base = s[r] + boff;
          H[r] = ldw<ODD>(base + 128 + 32 * c + 16 * l + 4 * t);
          Q0[r] = ldw<ODD>(base + 64 * c + 16 * l + 4 * t);
          Q1[r] = ldw<ODD>(base + 64 * c + 32 + 16 * l + 4 * t);
          SC[r][0] = ldw<ODD>(base + 192 + 8 * c);         // sub-scales of groups 0,1 (bytes l, 2+l)
          SC[r][1] = ldw<ODD>(base + 192 + 8 * c + 4);     // groups 2,3
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {             // sub-block index sub = 8c + 2g + l
          uint32_t a[2 * NSETS][2];
          float sc[2 * NSETS];
#pragma unroll
          for (int r = 0; r < 2 * NSETS; ++r) {
            const uint32_t Q = (g & 1) ? Q1[r] : Q0[r];
            if (g == 0) pair<0>(Q, H[r], a[r][0], a[r][1]);
            else if (g == 1) pair<1>(Q, H[r], a[r][0], a[r][1]);
            else if (g == 2) pair<2>(Q, H[r], a[r][0], a[r][1]);
            else pair<3>(Q, H[r], a[r][0], a[r][1]);
            const uint32_t scw = SC[r][g >> 1];
            const int sb = (int)(int8_t)((scw >> (8 * (2 * (g & 1) + l))) & 0xFFu);
            sc[r] = d[r] * (float)sb;
          }
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint2 b = bq[g][nt];
#pragma unroll
            for (int set = 0; set < NSETS; ++set) {
              float p[4];
              mma_f16_zero(p, a[2 * set][0], a[2 * set + 1][0], a[2 * set][1], a[2 * set + 1][1], b.x, b.y);
              acc[set][nt][0] = fmaf(sc[2 * set], p[0], acc[set][nt][0]);
              acc[set][nt][1] = fmaf(sc[2 * set], p[1], acc[set][nt][1]);
              acc[set][nt][2] = fmaf(sc[2 * set + 1], p[2], acc[set][nt][2]);
              acc[set][nt][3] = fmaf(sc[2 * set + 1], p[3], acc[set][nt][3]);
            }
          }
        }
      }
    }
  }
  template <int NSETS, int NT, bool PRE, class XP>
  __device__ __forceinline__ static void run(const uint32_t (&s)[2 * NSETS], int t,
                                             const BFrag<NT>&, const XP (&xr)[NT],
                                             int col, float (&acc)[NSETS][NT][4]) {
    superblock<0, NSETS, NT>(s, 0u, t, xr, col, acc);
    superblock<1, NSETS, NT>(s, 210u, t, xr, col + 256, acc);
  }
};


// ---- the per-warp weight stream ------------------------------------------------------------------
// A warp owns a ring of STAGES stages; a stage holds ROWS row-chunks (16 rows, or 16 + 16 rows: gate
// and up rows of a SwiGLU tile, or two consecutive 16-row blocks of one matrix).  Work is a flat
// list of steps = (m-tile, chunk) pairs; step i lives in stage i % STAGES.  One lane fetches a
// 16-row block with ONE 2-D TMA box copy (a per-row bulk copy costs the issuing warp an elect loop
// of ~13 instructions per row); rows past the end of the matrix arrive as zeros.
template <int FMT, int KCV, int ROWS, int STAGES>
struct WarpStream {
  using G = StageGeom<FMT, KCV>;
  using F = StreamFmt<FMT>;
  static constexpr int STAGE_BYTES = ROWS * G::PITCH;
  static constexpr int WARP_BYTES = STAGES * STAGE_BYTES;
  static_assert((16 * G::PITCH) % 128 == 0, "the second box of a stage must start 128-byte aligned");

  uint32_t smem;             // shared address of this warp's ring (128-byte aligned)
  uint32_t bars;             // shared address of this warp's STAGES mbarriers
  const CUtensorMap* m0;     // tensor maps of the weight matrices (m1 only when ROWS == 32)
  const CUtensorMap* m1;
  int row1_off;              // rows 16..31 of a stage: m1 at row0 + row1_off
  int K, nch, lane;
  int* err_flag;             // device-global flag raised when a bounded wait expires
  bool dead;

  __device__ __forceinline__ void init(uint32_t smem_, uint32_t bars_, const CUtensorMap* m0_,
                                       const CUtensorMap* m1_, int row1_off_, int K_, int lane_,
                                       int* err_flag_) {
    smem = smem_; bars = bars_; m0 = m0_; m1 = m1_; row1_off = row1_off_; K = K_; lane = lane_;
    err_flag = err_flag_;
    nch = (K + G::KC - 1) / G::KC;
    dead = false;
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < STAGES; ++s) mbar_init(bars + 8 * s, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
  }

  // shared address at which byte 0 of (row slot r, chunk c) lands
  __device__ __forceinline__ uint32_t slot_addr(int stage, int r, int c) const {
    return smem + stage * STAGE_BYTES + r * G::PITCH + ((uint32_t)(c * G::CHUNK_BYTES) & 15u);
  }

  // lane 0 fetches the row-chunks of step (row0, c) into `stage`
  __device__ __forceinline__ void issue(int stage, int row0, int c) {
    if (lane != 0) return;
    const uint32_t bar = bars + 8 * stage;
    const uint32_t dst = smem + stage * STAGE_BYTES;
    const int x = (int)(((uint32_t)(c * G::CHUNK_BYTES) & ~15u) >> 2);
    mbar_arrive_expect_tx(bar, (uint32_t)STAGE_BYTES);
    tma_box_2d(dst, m0, x, row0, bar);
    if constexpr (ROWS == 32) tma_box_2d(dst + 16 * G::PITCH, m1, x, row0 + row1_off, bar);
  }

  __device__ __forceinline__ bool wait(int stage, uint32_t parity) {
    if (dead) return false;
    if (!mbar_wait(bars + 8 * stage, parity, err_flag)) dead = true;
    return !dead;
  }
};

}  // namespace qx
