// BaseQN consumers: weights stored as three planes - packed codes (rows, K * bits / 8), one scale
// and (asymmetric tensors) one bias per `group` columns.  bits in {2,3,4,5,6,8}; lane c of a row
// occupies bits [c * bits, (c + 1) * bits) of the row's little-endian bit string; scales / biases are
// bf16, f16, e8m0 or e4m3.  w = fl(fl(code * scale) + bias), symmetric tensors (code - 2^(bits-1)) * scale.
// Follows kernels/quantization/base_q/README.md:8-47 and base_q.metal:8-41 of the reference.
//
// Two device paths:
//  * base_q_stream_kernel: 16-bit activations, K % 128 == 0, 16-byte aligned code rows.  Code rows
//    arrive in shared memory as 2-D TMA boxes (16 rows x 512 columns per stage, per-warp rings);
//    codes become exact f16 integers by a magic-number OR and feed mma.sync m16n8k16 against the
//    row-scaled f16 activations; each 32-column partial is scaled in fp32 and the bias enters as
//    bias * sum(x) of the chunk.  The warps of a CTA share the stages of one 16-row tile and add
//    their partial sums in shared memory; the last one to arrive runs the epilogue.
//  * base_q_generic_kernel: any dtype / alignment, one warp per row.
#include <cuda.h>

#include "qx_common.cuh"
#include "qx_formats.cuh"
#include "qx_kernels.h"
#include "qx_stream.cuh"
#include "qx_tmap.h"

namespace qx {

namespace {

// ---- plane access -------------------------------------------------------------------------------
// stype: 0 bf16, 1 f16, 2 e8m0, 3 e4m3 (base_q_descriptor.h:9-14 of the reference)
__device__ __forceinline__ float bq_scale_at(const uint8_t* __restrict__ plane, long long index, int stype) {
  if (stype == 0) return __uint_as_float((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(plane) + index) << 16);
  if (stype == 1) return __half2float(__ushort_as_half(__ldg(reinterpret_cast<const uint16_t*>(plane) + index)));
  if (stype == 2) return e8m0_to_f32(__ldg(plane + index));
  return e4m3_to_f32(__ldg(plane + index));
}
__host__ __device__ inline int bq_scale_bytes(int stype) { return stype < 2 ? 2 : 1; }

// the 8 codes that start at column c8 * 8 (bits bytes, byte aligned) as one 64-bit string
__device__ __forceinline__ uint64_t bq_load8(const uint8_t* __restrict__ row, int c8, int bits) {
  const uint8_t* p = row + (size_t)c8 * bits;
  uint64_t v = 0;
  for (int i = 0; i < bits; ++i) v |= (uint64_t)__ldg(p + i) << (8 * i);
  return v;
}

// ---- dequantise / embedding: one thread per 8 columns ---------------------------------------------
// ids == nullptr: out row r = weight row r.  Otherwise out row r = weight row ids[r], zeros when the
// id is outside [0, rows).
template <typename T>
__global__ void __launch_bounds__(256)
base_q_rows_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                   const uint8_t* __restrict__ biases, const int32_t* __restrict__ ids, T* __restrict__ out,
                   long long out_rows, long long rows, int K, int bits, int group, int stype, int symmetric) {
  const int per_row = K / 8;
  const long long total = out_rows * per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row;
    const int c8 = (int)(i - r * per_row);
    long long src = r;
    if (ids) src = ids[r];
    T* o = out + r * K + (size_t)c8 * 8;
    if (src < 0 || src >= rows) {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = from_f32<T>(0.f);
      continue;
    }
    const uint64_t v = bq_load8(codes + (size_t)src * ((size_t)K * bits / 8), c8, bits);
    const long long g = src * (K / group) + (c8 * 8) / group;
    const float sc = bq_scale_at(scales, g, stype);
    const float bi = symmetric ? 0.f : bq_scale_at(biases, g, stype);
    const uint32_t mask = (1u << bits) - 1u;
    const int off = 1 << (bits - 1);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int code = (int)((uint32_t)(v >> (j * bits)) & mask);
      const float w = symmetric ? (float)(code - off) * sc : __fadd_rn(__fmul_rn((float)code, sc), bi);
      o[j] = from_f32<T>(w);
    }
  }
}

// ---- generic matmul: one warp per weight row, up to 8 activation columns per pass --------------------
// x element (k, m) at x[k * xk + m * xm]; out element (row, m) at out[row * orow + m * ocol].
// mats == 2: out = silu(W0 x) * (W1 x).
struct BQPlanes { const uint8_t* codes; const uint8_t* scales; const uint8_t* biases; };

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
base_q_generic_kernel(BQPlanes w0, BQPlanes w1, int mats, const T* __restrict__ x, long long xk, long long xm,
                      TO* __restrict__ out, long long orow, long long ocol, long long rows, int K, int M,
                      int bits, int group, int stype, int symmetric) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int m0 = blockIdx.y * 8;
  const int mb = min(8, M - m0);
  const size_t row_bytes = (size_t)K * bits / 8;
  const uint32_t mask = (1u << bits) - 1u;
  const int off = 1 << (bits - 1);
  float acc[2][8];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[a][j] = 0.f;
  for (int c8 = lane; c8 < K / 8; c8 += 32) {
    float xv[8][8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int m = 0; m < 8; ++m)
        xv[j][m] = m < mb ? to_f32<T>(x[(long long)(c8 * 8 + j) * xk + (long long)(m0 + m) * xm]) : 0.f;
    for (int a = 0; a < mats; ++a) {
      const BQPlanes& w = a ? w1 : w0;
      const uint64_t v = bq_load8(w.codes + (size_t)row * row_bytes, c8, bits);
      const long long g = row * (K / group) + (c8 * 8) / group;
      const float sc = bq_scale_at(w.scales, g, stype);
      const float bi = symmetric ? 0.f : bq_scale_at(w.biases, g, stype);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int code = (int)((uint32_t)(v >> (j * bits)) & mask);
        const float wt = symmetric ? (float)(code - off) * sc : __fadd_rn(__fmul_rn((float)code, sc), bi);
#pragma unroll
        for (int m = 0; m < 8; ++m) acc[a][m] = fmaf(wt, xv[j][m], acc[a][m]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    float g = warp_sum(acc[0][m]);
    float u = mats == 2 ? warp_sum(acc[1][m]) : 0.f;
    if (lane == 0 && m < mb) {
      const float r = mats == 2 ? silu(g) * u : g;
      out[row * orow + (long long)(m0 + m) * ocol] = from_f32<TO>(r);
    }
  }
}

}  // namespace

namespace {

// ---- streaming tensor-core kernel ---------------------------------------------------------------
constexpr int BQ_KC = 512;            // columns per stage
constexpr int BQ_SLOTS = 16;          // tiles whose partial sums can be open at once in a CTA
constexpr int BQ_MAX_WARPS = 16;      // mbarrier slots reserved per CTA
// Warps launched per code width.  Up to 4 bits: 16 warps of at most 128 registers.  Wider codes move
// more bytes per stage, gain from deeper rings and from fetching the scales one item ahead, which
// needs more registers: 12 warps of up to 168.
__host__ __device__ constexpr int bq_warps(int bits) { return bits <= 4 ? 16 : 12; }

template <int BITS> struct BQGeom {
  static constexpr int STAGE_BYTES = BQ_KC * BITS / 8;       // payload per row
  // Row pitch in shared memory = box width: the payload plus 16 bytes, an odd multiple of 16 bytes,
  // so the 8 rows one instruction touches start in different 16-byte bank groups.
  static constexpr int PITCH = STAGE_BYTES + 16;
  static constexpr int BOX_BYTES = 16 * PITCH;
  static_assert((PITCH / 16) % 2 == 1 && BOX_BYTES % 128 == 0, "stage geometry");
};

struct BQSeg {
  const uint8_t* scales; const uint8_t* biases;   // plane bases of this matrix
  void* out;
  long long rows;       // weight rows (per expert for an expert stack)
  int tile0;            // first 16-row tile of this matrix in the launch's tile numbering
  int map;              // which tensor map covers its codes
};

struct BQStreamParams {
  BQSeg seg[3];
  int nseg;
  int mode;             // 0: every segment is its own projection; 1: seg 0 = gate, seg 1 = up, out = silu(g) * u
  int tiles;            // 16-row tiles of the launch (mode 1: of one matrix)
  int K, M, group, stype, symmetric;
  const __half* x16;    // prepared activations (M, K): f16, row-scaled, column order 5 of perm_position
  const float* rowscale;
  long long orow, ocol; // out element (row, m) at out[row * orow + m * ocol]
  int out_dtype;        // qx_dtype
  // expert stacks: activation column m belongs to expert expert_of_tile[m / 32]; its rows start at
  // expert * expert_rows in the planes (mode 1: gate rows first, up rows expert_up_off later)
  const int32_t* expert_of_tile;
  long long expert_rows, expert_up_off;
  int experts;
  int nst;              // ring depth per warp
  int* err;
  // XS instantiation (one activation column): the raw 16-bit activations, prepared by every CTA itself
  // into shared memory at byte offset xs_off of the dynamic window (x16 / rowscale unused)
  const uint16_t* xsrc;
  int x_bf16;
  unsigned xs_off;
};

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
  return v;
}

// The 8 codes of one lane (bits [0, 8 * BITS) of the string that starts at shared byte address a)
// as four f16 pairs: pair j = (code j, code j + 4).  A code sits in the low mantissa bits of its
// half, i.e. it is the f16 subnormal code * 2^-24: exact, and no conversion instruction is needed.
template <int BITS>
__device__ __forceinline__ void bq_pairs(uint32_t a, uint32_t (&pr)[4]) {
  constexpr uint32_t M2 = ((1u << BITS) - 1u) * 0x00010001u;
  uint32_t u[4];
  if constexpr (BITS == 2) {
    const uint32_t lo = lds16(a);
    const uint32_t w = __byte_perm(lo, 0u, 0x1110);
#pragma unroll
    for (int j = 0; j < 4; ++j) u[j] = w >> (2 * j);
  } else if constexpr (BITS == 4) {
    const uint32_t lo = lds32(a);
#pragma unroll
    for (int j = 0; j < 4; ++j) u[j] = lo >> (4 * j);
  } else if constexpr (BITS == 8) {
    const uint2 v = lds64(a);
    u[0] = __byte_perm(v.x, v.y, 0x4400); u[1] = __byte_perm(v.x, v.y, 0x5511);
    u[2] = __byte_perm(v.x, v.y, 0x6622); u[3] = __byte_perm(v.x, v.y, 0x7733);
  } else {
    const uint32_t a0 = a & ~3u, sh = (a & 3u) * 8u;
    const uint32_t w0 = lds32(a0), w1 = lds32(a0 + 4);
    const uint32_t lo = __funnelshift_r(w0, w1, sh), hi = w1 >> sh;
    if constexpr (BITS == 3) {
      const uint32_t w = __byte_perm(lo, lo >> 12, 0x5410);
#pragma unroll
      for (int j = 0; j < 4; ++j) u[j] = w >> (3 * j);
    } else if constexpr (BITS == 5) {
      const uint32_t f = __funnelshift_r(lo, hi, 20);
      const uint32_t w = __byte_perm(lo, f, 0x5410);
      u[0] = w; u[1] = w >> 5; u[2] = w >> 10;
      u[3] = __byte_perm(lo >> 15, f >> 15, 0x5410);
    } else {   // 6
      const uint32_t f = __funnelshift_r(lo, hi, 24);
      const uint32_t w = __byte_perm(lo, f, 0x5410);
      const uint32_t w2 = __byte_perm(lo >> 12, f >> 12, 0x5410);
      u[0] = w; u[1] = w >> 6; u[2] = w2; u[3] = w2 >> 6;
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) pr[j] = u[j] & M2;
}

// element e of a lane's scale vector (2-byte elements: 4 in raw.x / raw.y; 1-byte: 4 in raw.x)
__device__ __forceinline__ uint32_t bq_elem(uint2 raw, int e, int sb) {
  if (sb == 2) return (((e & 2) ? raw.y : raw.x) >> ((e & 1) * 16)) & 0xFFFFu;
  return (raw.x >> (8 * e)) & 0xFFu;
}
__device__ __forceinline__ uint2 bq_load_vec(const uint8_t* p, int nbytes) {
  uint2 r = make_uint2(0u, 0u);
  if (nbytes == 8) r = __ldg(reinterpret_cast<const uint2*>(p));
  else if (nbytes == 4) r.x = __ldg(reinterpret_cast<const uint32_t*>(p));
  else if (nbytes == 2) r.x = __ldg(reinterpret_cast<const uint16_t*>(p));
  else r.x = __ldg(p);
  return r;
}

__device__ __forceinline__ void bq_store(void* out, long long idx, float v, int dtype) {
  if (dtype == QX_DTYPE_F32) reinterpret_cast<float*>(out)[idx] = v;
  else if (dtype == QX_DTYPE_F16) reinterpret_cast<__half*>(out)[idx] = __float2half_rn(v);
  else reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
}

// Position in a CTA's flat list of (local tile, stage) pairs; a warp's next item is W pairs later.
struct BQCursor {
  int tl, s;
  __device__ __forceinline__ void advance(int by, int spt) {
    s += by;
    while (s >= spt) { s -= spt; ++tl; }
  }
};

// NC = activation columns a CTA serves (1, 4 or 8): the width of the bias-path accumulators.
// Arithmetic per weight row r and column n:
//   out = rowscale[n] * ( 2^24 * sum_c scale[r,c] * P[r,c,n]  +  sum_c beta[r,c] * S[c,n] )
// with c the 32-column chunks, P the tensor-core partial over the subnormal codes (= 2^-24 * sum
// code * x), S[c,n] the sum of the 32 prepared activations, beta = bias (asymmetric) or
// -2^(BITS-1) * scale (symmetric).
template <int BITS, int NC, bool XS>
__global__ void __launch_bounds__(bq_warps(BITS) * 32, 1)
base_q_stream_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                     const __grid_constant__ CUtensorMap map2, const BQStreamParams p) {
  using G = BQGeom<BITS>;
  extern __shared__ __align__(128) uint8_t bq_smem[];
  // a programmatic dependent of the kernel before it: nothing of its output is touched before this point
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;");
  const int W = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int K = p.K, nchunks = K / 32, nst = p.nst;
  // prepared activations and row scales: global (preparation kernel), or with XS this CTA's own copy of
  // the single column in shared memory (read through generic addresses)
  const __half* x16 = p.x16;
  const float* rowscale = p.rowscale;
  if constexpr (XS) {
    static_assert(NC == 1, "in-kernel preparation: one activation column");
    cta_prepare_row<5>(bq_smem + p.xs_off, p.xsrc, p.x_bf16, K);
    x16 = reinterpret_cast<const __half*>(bq_smem + p.xs_off);
    rowscale = reinterpret_cast<const float*>(bq_smem + p.xs_off + (size_t)K * 2);
  }
  auto ldx = [](const uint4* q) { if constexpr (XS) return *q; else return __ldg(q); };
  const int spt1 = (K + BQ_KC - 1) / BQ_KC;
  const int mats = p.mode == 1 ? 2 : 1;
  const int spt = mats * spt1;
  const int col0 = blockIdx.y * 8;
  const int ncol = min(NC, p.M - col0);
  long long rowoff = 0;
  if (p.expert_of_tile) {
    const int e = p.expert_of_tile[col0 / 32];
    if (e < 0 || e >= p.experts) return;          // a padding tile: its output rows stay as they are
    rowoff = (long long)e * p.expert_rows;
  }

  // shared memory: chunk sums | partial-sum slots | counters | epochs | mbarriers | rings
  float* S = reinterpret_cast<float*>(bq_smem);                       // [nchunks + 16][8], the tail zero
  float* red = S + (size_t)(nchunks + 16) * 8;                        // [SLOTS][2][128]
  int* cnt = reinterpret_cast<int*>(red + BQ_SLOTS * 256);
  int* epoch = cnt + BQ_SLOTS;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epoch + BQ_SLOTS);
  const uint32_t ring0 = (smem_u32(bars + BQ_MAX_WARPS * 8) + 127u) & ~127u;

  for (int i = threadIdx.x; i < (nchunks + 16) * 8; i += blockDim.x) {
    const int c = i >> 3, n = i & 7;
    float s = 0.f;
    if (n < ncol && c < nchunks) {
      const uint4* xp = reinterpret_cast<const uint4*>(x16 + (size_t)(col0 + n) * K + (size_t)c * 32);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 v = ldx(xp + q);
        const float2 a = f16x2_to_f32(v.x), b = f16x2_to_f32(v.y), c2 = f16x2_to_f32(v.z), d = f16x2_to_f32(v.w);
        s += ((a.x + a.y) + (b.x + b.y)) + ((c2.x + c2.y) + (d.x + d.y));
      }
    }
    S[i] = s;
  }
  for (int i = threadIdx.x; i < BQ_SLOTS * 256; i += blockDim.x) red[i] = 0.f;
  if (threadIdx.x < BQ_SLOTS) { cnt[threadIdx.x] = 0; epoch[threadIdx.x] = threadIdx.x; }
  const uint32_t mybars = smem_u32(bars) + (uint32_t)warp * 64u;      // up to 8 stages per warp
  if (lane == 0)
    for (int s = 0; s < nst; ++s) mbar_init(mybars + 8 * s, 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();

  const int b = blockIdx.x, Gx = gridDim.x;
  const int my_tiles = b < p.tiles ? (p.tiles - b + Gx - 1) / Gx : 0;
  const int J = my_tiles * spt;                                       // fits: tiles * stages < 2^31
  // every warp takes a contiguous range of the CTA's (tile, stage) list: its accumulators live across
  // the stages of a tile, and a tile costs it one update of the shared slot
  const int per = (J + W - 1) / W;
  const int first = warp * per;
  const int n_items = first < J ? min(per, J - first) : 0;
  const uint32_t myring = ring0 + (uint32_t)warp * (uint32_t)(nst * G::BOX_BYTES);
  const int gshift = p.group == 32 ? 0 : (p.group == 64 ? 1 : 2);
  const int sb = bq_scale_bytes(p.stype);
  const int vec_bytes = (128 / p.group) * sb;
  const int groups_per_row = K / p.group;
  const float sym_off = -(float)(1 << (BITS - 1));
  bool dead = false;

  // (tile, matrix, stage, segment) of a cursor position
  auto locate = [&](const BQCursor& c, int& mat, int& stage, int& sidx, int& trow0) {
    mat = c.s >= spt1 ? 1 : 0;
    stage = c.s - mat * spt1;
    const int tile = b + c.tl * Gx;
    sidx = mats == 2 ? mat : 0;
    if (mats == 1) {
      if (p.nseg > 1 && tile >= p.seg[1].tile0) sidx = 1;
      if (p.nseg > 2 && tile >= p.seg[2].tile0) sidx = 2;
    }
    trow0 = (tile - p.seg[sidx].tile0) * 16;
  };
  BQCursor icur{first / spt, first % spt};                            // next item to fetch (lane 0 uses it)
  auto issue = [&](int i) {
    if (lane == 0) {
      int mat, stage, sidx, trow0;
      locate(icur, mat, stage, sidx, trow0);
      const int slot = i % nst;
      const uint32_t bar = mybars + 8 * slot;
      const CUtensorMap* m = p.seg[sidx].map == 0 ? &map0 : (p.seg[sidx].map == 1 ? &map1 : &map2);
      const long long y = rowoff + (mat == 1 ? p.expert_up_off : 0) + trow0;
      mbar_arrive_expect_tx(bar, (uint32_t)G::BOX_BYTES);
      tma_box_2d(myring + slot * G::BOX_BYTES, m, stage * (G::STAGE_BYTES / 4), (int)y, bar);
    }
    icur.advance(1, spt);
  };

  int issued = 0;
  for (; issued < n_items && issued < nst; ++issued) issue(issued);

  float acc[4] = {0.f, 0.f, 0.f, 0.f};        // scale path, D-fragment layout: rows g / g+8, columns 2t / 2t+1
  float bacc[2][NC];                          // bias path: rows g / g+8, this lane's chunks, every column
#pragma unroll
  for (int rr = 0; rr < 2; ++rr)
#pragma unroll
    for (int n = 0; n < NC; ++n) bacc[rr][n] = 0.f;
  int consumed = 0;
  BQCursor cur{first / spt, first % spt};
  // raw scale / bias vectors of an item (this lane's 128 columns of rows g and g + 8), fetched one
  // item ahead so that their latency hides behind the arithmetic of the current item
  struct RawScales { uint2 s[2], b[2]; bool ok[2]; };
  auto fetch_scales = [&](const BQCursor& c, RawScales& r) {
    int mat, stage, sidx, trow0;
    locate(c, mat, stage, sidx, trow0);
    const BQSeg& sg = p.seg[sidx];
    const int colb = stage * BQ_KC + t * 128;
    const long long prow = rowoff + (mat == 1 ? p.expert_up_off : 0) + trow0 + g;
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      r.ok[rr] = colb < K && trow0 + g + 8 * rr < sg.rows;
      r.s[rr] = make_uint2(0u, 0u); r.b[rr] = make_uint2(0u, 0u);
      if (r.ok[rr]) {
        const size_t off = ((size_t)(prow + 8 * rr) * groups_per_row + colb / p.group) * sb;
        r.s[rr] = bq_load_vec(sg.scales + off, vec_bytes);
        if (!p.symmetric) r.b[rr] = bq_load_vec(sg.biases + off, vec_bytes);
      }
    }
  };
  constexpr bool AHEAD = BITS > 4;                 // one-item-ahead fetch where the register budget allows
  RawScales raw_cur, raw_next;
  if (AHEAD && n_items > 0) fetch_scales(cur, raw_next);
  for (int i = 0; i < n_items && !dead; ++i) {
    int mat, stage, sidx, trow0;
    locate(cur, mat, stage, sidx, trow0);
    const int tl = cur.tl;
    if constexpr (AHEAD) {
      raw_cur = raw_next;
      if (i + 1 < n_items) {
        BQCursor nx = cur;
        nx.advance(1, spt);
        fetch_scales(nx, raw_next);
      }
    } else {
      fetch_scales(cur, raw_cur);
    }
    float sfc[2][4];
    {
      const float* Sq = S + (size_t)(stage * 16 + 4 * t) * 8;          // rows past nchunks are zero
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const bool ok = raw_cur.ok[rr];
        const uint2 rs = raw_cur.s[rr], rb = raw_cur.b[rr];
        // storage -> fp32, the storage type tested once per row (not once per element)
        float scv[4], bev[4];
        auto convert = [&](auto conv) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            scv[q] = conv(bq_elem(rs, q >> gshift, sb));
            bev[q] = p.symmetric ? sym_off * scv[q] : conv(bq_elem(rb, q >> gshift, sb));
          }
        };
        if (p.stype == 0) convert([](uint32_t r) { return __uint_as_float(r << 16); });
        else if (p.stype == 1) convert([](uint32_t r) { return __half2float(__ushort_as_half((unsigned short)r)); });
        else if (p.stype == 2) convert([](uint32_t r) { return e8m0_to_f32(r); });
        else convert([](uint32_t r) { return e4m3_to_f32(r); });
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          sfc[rr][q] = ok ? scv[q] : 0.f;
          const float beta = ok ? bev[q] : 0.f;
#pragma unroll
          for (int n = 0; n < NC; ++n) bacc[rr][n] = fmaf(beta, Sq[q * 8 + n], bacc[rr][n]);
        }
      }
    }
    const int slot = i % nst;
    if (!mbar_wait(mybars + 8 * slot, (uint32_t)((i / nst) & 1), p.err)) { dead = true; break; }
    consumed = i + 1;
    const uint32_t base = myring + slot * G::BOX_BYTES;
    const uint32_t rowA = base + g * G::PITCH + t * BITS, rowB = rowA + 8 * G::PITCH;
    // lanes whose column does not exist read column 0: their D columns are never written out
    const __half* xr = x16 + (size_t)(col0 + (g < ncol ? g : 0)) * K + (size_t)stage * BQ_KC + 8 * t;
    const int nch = min(16, nchunks - stage * 16);
    auto chunk = [&](int c, const uint4& bv) {
      uint32_t pa[4], pb[4];
      bq_pairs<BITS>(rowA + c * 4 * BITS, pa);
      bq_pairs<BITS>(rowB + c * 4 * BITS, pb);
      float d[4];
      mma_f16_zero(d, pa[0], pb[0], pa[1], pb[1], bv.x, bv.y);
      mma_f16(d, pa[2], pb[2], pa[3], pb[3], bv.z, bv.w);
      const int src = (lane & ~3) | (c >> 2);
      const float sA = __shfl_sync(0xffffffffu, sfc[0][c & 3], src);
      const float sB = __shfl_sync(0xffffffffu, sfc[1][c & 3], src);
      acc[0] = fmaf(sA, d[0], acc[0]); acc[1] = fmaf(sA, d[1], acc[1]);
      acc[2] = fmaf(sB, d[2], acc[2]); acc[3] = fmaf(sB, d[3], acc[3]);
    };
    if (nch == 16) {                               // a whole stage: no branches, the activation loads 4 chunks ahead
      uint4 bq[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) bq[c] = ldx(reinterpret_cast<const uint4*>(xr + c * 32));
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const uint4 bv = bq[c & 3];
        if (c + 4 < 16) bq[c & 3] = ldx(reinterpret_cast<const uint4*>(xr + (c + 4) * 32));
        chunk(c, bv);
      }
    } else {
#pragma unroll
      for (int c = 0; c < 16; ++c)
        if (c < nch) chunk(c, ldx(reinterpret_cast<const uint4*>(xr + c * 32)));
    }
    __syncwarp();
    if (issued < n_items) { issue(issued); ++issued; }

    // last item of this warp for (tile, matrix): add the partial sums to the tile's slot
    cur.advance(1, spt);
    if (i + 1 < n_items && cur.tl == tl && (cur.s >= spt1 ? 1 : 0) == mat) continue;
    const int rs = tl % BQ_SLOTS;
    {
      volatile int* ep = epoch + rs;
      int spins = 0;
      while (*ep != tl) {
        if (++spins > (1 << 22)) { atomicExch(p.err, 1); dead = true; break; }
      }
      if (dead) break;
    }
    float* slotp = red + rs * 256 + mat * 128;
    if (2 * t < ncol) {
      atomicAdd(slotp + g * 8 + 2 * t, acc[0] * 16777216.f);
      atomicAdd(slotp + (g + 8) * 8 + 2 * t, acc[2] * 16777216.f);
    }
    if (2 * t + 1 < ncol) {
      atomicAdd(slotp + g * 8 + 2 * t + 1, acc[1] * 16777216.f);
      atomicAdd(slotp + (g + 8) * 8 + 2 * t + 1, acc[3] * 16777216.f);
    }
    acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
#pragma unroll
    for (int rr = 0; rr < 2; ++rr)
#pragma unroll
      for (int n = 0; n < NC; ++n) {
        float v = bacc[rr][n];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        if ((n & 3) == t && n < ncol) atomicAdd(slotp + (g + 8 * rr) * 8 + n, v);
        bacc[rr][n] = 0.f;
      }
    __syncwarp();
    int old = 0;
    if (lane == 0) { __threadfence_block(); old = atomicAdd(cnt + rs, 1); }
    old = __shfl_sync(0xffffffffu, old, 0);
    int need = 0;                                  // warps whose ranges meet this tile, per matrix
    for (int m = 0; m < mats; ++m) {
      const int a = tl * spt + m * spt1;
      need += (a + spt1 - 1) / per - a / per + 1;
    }
    if (old != need - 1) continue;
    // every contribution is in: epilogue of the tile by this warp
    __threadfence_block();
    const BQSeg& so = p.seg[mats == 2 ? 0 : sidx];
    for (int idx = lane; idx < 128; idx += 32) {
      const int r = idx >> 3, n = idx & 7;
      const float gsum = atomicExch(red + rs * 256 + idx, 0.f);
      const float usum = mats == 2 ? atomicExch(red + rs * 256 + 128 + idx, 0.f) : 0.f;
      if (n < ncol && trow0 + r < so.rows) {
        const float sc = rowscale[col0 + n];
        const float v = mats == 2 ? silu(gsum * sc) * (usum * sc) : gsum * sc;
        bq_store(so.out, (long long)(trow0 + r) * p.orow + (long long)(col0 + n) * p.ocol, v, p.out_dtype);
      }
    }
    __syncwarp();
    if (lane == 0) { cnt[rs] = 0; __threadfence_block(); atomicExch(epoch + rs, tl + BQ_SLOTS); }
  }
  // a warp that gave up still owns copies in flight: wait for them (bounded) before the CTA may exit
  if (dead)
    for (int i = consumed; i < issued; ++i) mbar_wait(mybars + 8 * (i % nst), (uint32_t)((i / nst) & 1), p.err);
}

}  // namespace

// ---- host side ------------------------------------------------------------------------------------
static inline size_t bq_align256(size_t n) { return (n + 255) & ~(size_t)255; }

static bool bq_stream_fits(int bits, int64_t K, int* warps, int* nst, size_t* smem) {
  const int pitch = BQ_KC * bits / 8 + 16, box = 16 * pitch;
  const size_t fixed = (size_t)(K / 32 + 16) * 32 + BQ_SLOTS * 256 * 4 + BQ_SLOTS * 8 + BQ_MAX_WARPS * 64 + 128;
  // the rest of the SM's 256 KB stays L1: every warp re-reads the activations
  const size_t budget = (bits <= 4 ? 168 : 200) * 1024;
  for (int w : {bq_warps(bits), 8}) {
    if (fixed + (size_t)w * 2 * box > budget) continue;
    int n = (int)((budget - fixed) / ((size_t)w * box));
    if (n > 6) n = 6;
    *warps = w; *nst = n; *smem = fixed + (size_t)w * n * box;
    return true;
  }
  return false;
}

size_t base_q_scratch_bytes(int64_t K, int64_t M, qx_dtype dtype, bool x_is_km) {
  if (dtype == QX_DTYPE_F32) return 0;                       // fp32 activations run on the generic kernel
  size_t n = bq_align256((size_t)M * K * 2) + bq_align256((size_t)M * 4);
  if (x_is_km && M > 1) n += bq_align256((size_t)M * K * 2);
  return n;
}

template <int BITS, int NC, bool XS>
static bool bq_launch_stream_nc(cudaStream_t st, const CUtensorMap* maps, const BQStreamParams& p, int gx, int gy,
                                int warps, size_t smem) {
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(base_q_stream_kernel<BITS, NC, XS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    attr_set[dev] = true;
  }
  // a programmatic dependent of the kernel before it (see griddepcontrol.wait in the kernel)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(gx, gy);
  cfg.blockDim = dim3(warps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, base_q_stream_kernel<BITS, NC, XS>, maps[0], maps[1], maps[2], p) != cudaSuccess) {
    cudaGetLastError();
    base_q_stream_kernel<BITS, NC, XS><<<dim3(gx, gy), warps * 32, smem, st>>>(maps[0], maps[1], maps[2], p);
  }
  note_launch();
  return true;
}

template <int BITS>
static bool bq_launch_stream(cudaStream_t st, const CUtensorMap* maps, const BQStreamParams& p, int gx, int gy,
                             int warps, size_t smem) {
  if (p.M == 1 && p.xsrc) return bq_launch_stream_nc<BITS, 1, true>(st, maps, p, gx, gy, warps, smem);
  if (p.M == 1) return bq_launch_stream_nc<BITS, 1, false>(st, maps, p, gx, gy, warps, smem);
  if (p.M <= 4) return bq_launch_stream_nc<BITS, 4, false>(st, maps, p, gx, gy, warps, smem);
  return bq_launch_stream_nc<BITS, 8, false>(st, maps, p, gx, gy, warps, smem);
}

// One launch over up to three weight matrices (mode 0) or a gate / up pair (mode 1).  x: (K, M) when
// x_is_km, else (M, K).  Output element (row, m) of matrix i at out_i[row * orow + m * ocol].
// Returns false when no device path could be configured.
bool launch_base_q_matmul(cudaStream_t st, const BaseQDesc& d, const BaseQMat* mats, int nmat, int mode,
                          const void* x, bool x_is_km, int64_t K, int64_t M, qx_dtype dtype, int64_t orow,
                          int64_t ocol, void* scratch, size_t scratch_bytes, const BaseQExperts* ex) {
  const size_t row_bytes = (size_t)K * d.bits / 8;
  int warps = 0, nst = 0;
  size_t smem = 0;
  bool fast = !options().force_generic && dtype != QX_DTYPE_F32 && K % 128 == 0 && K >= BQ_KC &&
              ((uintptr_t)x & 15) == 0 && scratch && scratch_bytes >= base_q_scratch_bytes(K, M, dtype, x_is_km) &&
              bq_stream_fits(d.bits, K, &warps, &nst, &smem) && device_error_flag() != nullptr;
  for (int i = 0; i < nmat && fast; ++i)
    fast = ((uintptr_t)mats[i].codes & 15) == 0 && ((uintptr_t)mats[i].scales & 7) == 0 &&
           (d.symmetric || ((uintptr_t)mats[i].biases & 7) == 0);
  if (fast) {
    char* ws = (char*)scratch;
    const void* xr = x;
    if (x_is_km && M > 1) {
      launch_transpose(st, x, ws, K, M, 2);
      xr = ws;
      ws += bq_align256((size_t)M * K * 2);
    }
    __half* x16 = (__half*)ws;
    float* rowscale = (float*)(ws + bq_align256((size_t)M * K * 2));
    BQStreamParams p{};
    // one activation column whose prepared copy fits behind the rings: every CTA prepares it itself
    const size_t xs_off = (smem + 15) & ~(size_t)15;
    if (M == 1 && !ex && xs_off + cta_prepared_row_bytes((size_t)K) <= 227 * 1024) {
      p.xsrc = (const uint16_t*)xr;
      p.x_bf16 = dtype == QX_DTYPE_BF16;
      p.xs_off = (unsigned)xs_off;
      smem = xs_off + cta_prepared_row_bytes((size_t)K);
    } else {
      launch_prep_activations(st, xr, dtype, x16, rowscale, (int)M, (int)K, 5);
      note_launch();
    }
    CUtensorMap maps[3];
    const int pitch = BQ_KC * d.bits / 8 + 16;
    int tiles = 0;
    const int64_t stack = ex ? ex->experts : 1;
    for (int i = 0; i < nmat && fast; ++i) {
      const int64_t map_rows = ex ? stack * ex->expert_rows : mats[i].rows;
      fast = cached_weight_map(&maps[i], mats[i].codes, map_rows, row_bytes, pitch, 16);
      p.seg[i] = BQSeg{(const uint8_t*)mats[i].scales, (const uint8_t*)mats[i].biases, mats[i].out, mats[i].rows,
                       mode == 1 ? 0 : tiles, i};
      if (mode != 1 || i == 0) tiles += (int)((mats[i].rows + 15) / 16);
    }
    for (int i = nmat; i < 3; ++i) maps[i] = maps[0];
    if (fast) {
      p.nseg = nmat; p.mode = mode; p.tiles = tiles;
      p.K = (int)K; p.M = (int)M; p.group = d.group; p.stype = d.stype; p.symmetric = d.symmetric;
      p.x16 = x16; p.rowscale = rowscale; p.orow = orow; p.ocol = ocol; p.out_dtype = (int)dtype;
      p.expert_of_tile = ex ? ex->expert_of_tile : nullptr;
      p.expert_rows = ex ? ex->expert_rows : 0;
      p.expert_up_off = ex ? ex->up_offset : 0;
      p.experts = ex ? (int)ex->experts : 0;
      p.nst = nst; p.err = device_error_flag();
      const int gy = (int)((M + 7) / 8);
      int gx = sm_count() / (gy < sm_count() ? gy : sm_count());
      if (gx < 1) gx = 1;
      if (gx > tiles) gx = tiles;
      switch (d.bits) {
        case 2: fast = bq_launch_stream<2>(st, maps, p, gx, gy, warps, smem); break;
        case 3: fast = bq_launch_stream<3>(st, maps, p, gx, gy, warps, smem); break;
        case 4: fast = bq_launch_stream<4>(st, maps, p, gx, gy, warps, smem); break;
        case 5: fast = bq_launch_stream<5>(st, maps, p, gx, gy, warps, smem); break;
        case 6: fast = bq_launch_stream<6>(st, maps, p, gx, gy, warps, smem); break;
        default: fast = bq_launch_stream<8>(st, maps, p, gx, gy, warps, smem); break;
      }
      if (fast) return true;
    }
  }
  if (ex) return false;                                       // expert stacks have no generic form
  // generic: one launch per projection (mode 1: one launch computes both matrices)
  const long long xk = x_is_km ? M : 1, xm = x_is_km ? 1 : K;
  const int launches = mode == 1 ? 1 : nmat;
  for (int i = 0; i < launches; ++i) {
    BQPlanes w0{(const uint8_t*)mats[i].codes, (const uint8_t*)mats[i].scales, (const uint8_t*)mats[i].biases};
    BQPlanes w1 = w0;
    if (mode == 1) w1 = BQPlanes{(const uint8_t*)mats[1].codes, (const uint8_t*)mats[1].scales, (const uint8_t*)mats[1].biases};
    const dim3 grid((unsigned)((mats[i].rows + 7) / 8), (unsigned)((M + 7) / 8));
    const int nm = mode == 1 ? 2 : 1;
#define QX_BQ_GENERIC(T)                                                                                         \
    base_q_generic_kernel<T, T><<<grid, 256, 0, st>>>(w0, w1, nm, (const T*)x, xk, xm, (T*)mats[i].out, orow, ocol, \
                                                      mats[i].rows, (int)K, (int)M, d.bits, d.group, d.stype, d.symmetric)
    if (dtype == QX_DTYPE_F32) QX_BQ_GENERIC(float);
    else if (dtype == QX_DTYPE_F16) QX_BQ_GENERIC(__half);
    else QX_BQ_GENERIC(__nv_bfloat16);
#undef QX_BQ_GENERIC
    note_launch();
  }
  return true;
}

// out (out_rows, K) = dequantised rows (ids == nullptr: all rows in order; else gathered, zero rows
// for ids outside [0, rows)).
void launch_base_q_rows(cudaStream_t st, const BaseQDesc& d, const void* codes, const void* scales,
                        const void* biases, const int32_t* ids, void* out, int64_t out_rows, int64_t rows,
                        int64_t K, qx_dtype out_dtype) {
  const long long total = out_rows * (K / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  if (blocks < 1) blocks = 1;
#define QX_BQ_ROWS(T)                                                                                             \
  base_q_rows_kernel<T><<<(unsigned)blocks, 256, 0, st>>>((const uint8_t*)codes, (const uint8_t*)scales,          \
                                                          (const uint8_t*)biases, ids, (T*)out, out_rows, rows,   \
                                                          (int)K, d.bits, d.group, d.stype, d.symmetric)
  if (out_dtype == QX_DTYPE_F32) QX_BQ_ROWS(float);
  else if (out_dtype == QX_DTYPE_F16) QX_BQ_ROWS(__half);
  else QX_BQ_ROWS(__nv_bfloat16);
#undef QX_BQ_ROWS
  note_launch();
}

}  // namespace qx
