// Fused LM head + sampling over packed weights: logits live only in shared memory.
//
// Stage 1 (partials): one CTA per 256-row vocabulary tile and per group of up to 8 hidden rows.
// The CTA projects its tile, keeps the (tokens x 256) logits in shared memory and reduces them to
// per-tile partials: the running (max, id) for argmax / categorical, the tile's top-k for top-k /
// top-p, plus the tile's tempered log-sum-exp for top-p.  Tiles start at multiples of 256 of the
// GLOBAL vocabulary id, which is what the top-p pool semantics are defined on.
//
// Stage 2 (reduce): one CTA per hidden row merges the partials of all tiles (and, for a sharded
// vocabulary, of all shards): max with lowest-id tie break; exact top-k by a radix select on the
// candidate values; nucleus threshold by 32 bisection steps against the full-vocabulary
// normalizer; Gumbel-max with the stateless (seed, row, global id) noise stream.
//
// Ordering everywhere: value descending, ties to the smaller id.
#include <atomic>

#include "qx_block.cuh"
#include "qx_formats.cuh"
#include "qx_kernels.h"
#include "qx_stream.cuh"
#include "qx_tmap.h"

namespace qx {

constexpr int LMH_TILE = 256;
constexpr int LMH_TB = 8;        // hidden rows per stage-1 CTA
constexpr int LMH_RED_THREADS = 1024;
constexpr int LMH_RED_COMPACT = 4096;   // candidates the stage-2 top-k search keeps in shared memory after its prefilter

// Reduce one hidden row's 256 tile logits (shared memory) to the tile partials of its mode.
// Executed by one warp.  nvalid <= 0 marks a padding tile: absent partials are written.
// Mode 4 (lm_head_masked, kernels/quantization/lm_head/lm_head.metal:1152-1262): the tile's top-k
// among the tokens whose bit is set in the row's allow mask, and the log-sum-exp of the raw logits
// over the allowed tokens (norm_allowed) or over every token of the tile.
__device__ __forceinline__ void lmh_select_token(const float* __restrict__ logit, int nvalid, int v0,
                                                 long long vocab_offset,
                                                 const float* __restrict__ bias, int t, int tile,
                                                 long long tiles_stride, int mode, int topk,
                                                 float invtemp, uint32_t seed,
                                                 float* __restrict__ part_val,
                                                 int32_t* __restrict__ part_id,
                                                 float* __restrict__ part_lse, int lane,
                                                 const LmhMask mask = LmhMask{nullptr, 0, 1}) {
  if (mode <= 1) {
    float best = QX_NEG_INF;
    int bid = 0x7fffffff;
    for (int lr = lane; lr < nvalid; lr += 32) {
      const int gid = (int)(vocab_offset + v0 + lr);
      float ls = logit[lr] * invtemp;
      if (bias) ls += bias[v0 + lr];
      if (mode == 1) ls += rng_gumbel(seed, (uint32_t)t, (uint32_t)gid);
      if (better(ls, gid, best, bid)) { best = ls; bid = gid; }
    }
    warp_argmax(best, bid);
    if (lane == 0) {
      part_val[(size_t)t * tiles_stride + tile] = best;
      part_id[(size_t)t * tiles_stride + tile] = bid == 0x7fffffff ? -1 : bid;
    }
    return;
  }
  // modes 2/3/4: tile top-k of the raw logits (+bias); modes 3/4 also the (tempered) log-sum-exp
  float mv[8];
  int mi[8];
  unsigned in_lse = 0u;          // bit j: element j counts towards the tile's log-sum-exp
  unsigned ncand_l = 0u;         // this lane's candidates
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int lr = lane + 32 * j;
    if (lr < nvalid) {
      float ls = logit[lr];
      if (bias) ls += bias[v0 + lr];
      mv[j] = ls;
      const long long gid = vocab_offset + v0 + lr;
      bool cand = true;
      if (mode == 4) cand = (mask.bits[(size_t)t * mask.words + (gid >> 5)] >> (gid & 31)) & 1u;
      mi[j] = cand ? (int)gid : -1;
      ncand_l += cand ? 1u : 0u;
      if (cand || (mode == 4 && !mask.norm_allowed)) in_lse |= 1u << j;
    } else {
      mv[j] = QX_NEG_INF;
      mi[j] = -1;
    }
  }
  if (mode >= 3) {
    // (tempered) log-sum-exp of the tile: maximum first, then one exponential per element
    float lmax = QX_NEG_INF;
#pragma unroll
    for (int j = 0; j < 8; ++j) lmax = fmaxf(lmax, ((in_lse >> j) & 1u) ? mv[j] * invtemp : QX_NEG_INF);
    const float gmax = warp_max(lmax);
    float lsum = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) lsum += ((in_lse >> j) & 1u) ? expf(mv[j] * invtemp - gmax) : 0.f;
    const float gsum = warp_sum(lsum);
    if (lane == 0)
      part_lse[(size_t)t * tiles_stride + tile] = gsum > 0.f ? gmax + logf(gsum) : QX_NEG_INF;
  }
  // Tile top-k as an unordered set: find the k-th largest key by a bitwise binary search on the
  // order-preserving keys (one warp-wide count per step), then emit every element above it and, of
  // the elements equal to it, the ones with the smallest ids.
  const size_t pbase = ((size_t)t * tiles_stride + tile) * topk;
  const int k_eff = min(topk, mode == 4 ? (int)__reduce_add_sync(0xffffffffu, ncand_l) : max(nvalid, 0));
  uint32_t key[8];
  uint32_t kmax = 0u, kmin = 0xFFFFFFFFu;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    key[j] = mi[j] >= 0 ? float_key(mv[j]) : 0u;
    kmax = max(kmax, key[j]);
    if (mi[j] >= 0) kmin = min(kmin, key[j]);
  }
  uint32_t out_pos = 0u;
  if (k_eff > 0) {
    const uint32_t hi = __reduce_max_sync(0xffffffffu, kmax);
    uint32_t lo = __reduce_min_sync(0xffffffffu, kmin);
    // with a full tile and k <= 32, every lane's largest element is among at least 32 elements
    // that are >= the smallest such maximum
    if (k_eff <= 32 && nvalid >= LMH_TILE && mode != 4) lo = max(lo, __reduce_min_sync(0xffffffffu, kmax));
    const int nb = 32 - __clz(hi ^ lo);                 // bits below the common prefix of lo and hi
    uint32_t ans = nb >= 32 ? 0u : (lo >> nb) << nb;
    for (int b = nb - 1; b >= 0; --b) {
      const uint32_t cand = ans | (1u << b);
      unsigned c = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) c += key[j] >= cand ? 1u : 0u;
      c = __reduce_add_sync(0xffffffffu, c);
      if (c >= (unsigned)k_eff) ans = cand;
      if (c == (unsigned)k_eff) break;      // exactly k elements lie at or above cand: that is the set
    }
    unsigned cg = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) cg += key[j] > ans ? 1u : 0u;
    const unsigned need = (unsigned)k_eff - __reduce_add_sync(0xffffffffu, cg);   // ties to take, >= 1
    const uint32_t lt_mask = (1u << lane) - 1u;
    unsigned ties_before = 0u;
#pragma unroll
    for (int j = 0; j < 8; ++j) {                       // id order = (j, lane) lexicographic
      const bool valid = mi[j] >= 0;
      const bool eq = valid && key[j] == ans;
      const uint32_t bal_eq = __ballot_sync(0xffffffffu, eq);
      const bool sel = valid && (key[j] > ans || (eq && ties_before + __popc(bal_eq & lt_mask) < need));
      const uint32_t bal = __ballot_sync(0xffffffffu, sel);
      if (sel) {
        const uint32_t pos = out_pos + __popc(bal & lt_mask);
        part_val[pbase + pos] = mv[j];
        part_id[pbase + pos] = mi[j];
      }
      out_pos += __popc(bal);
      ties_before += __popc(bal_eq);
    }
  }
  for (int kk = (int)out_pos + lane; kk < topk; kk += 32) {
    part_val[pbase + kk] = QX_NEG_INF;
    part_id[pbase + kk] = -1;
  }
}

// The same reduction for up to R hidden rows at once, one warp.  The threshold search is a chain of
// dependent warp-wide counts (about 25 steps of ~40 cycles each); running R rows through the chain
// together hides that latency, which is what the per-tile selection of many hidden rows is bound
// by.  logit[r] = the row's 256 tile logits in shared memory, trow[r] = its row index in the call
// (< 0: slot unused).  Same results as lmh_select_token row by row.
template <int R>
__device__ __forceinline__ void lmh_select_rows(const float* const (&logit)[R], const int (&trow)[R],
                                                int nvalid, int v0, long long vocab_offset,
                                                const float* __restrict__ bias, int tile,
                                                long long tiles_stride, int mode, int topk, float invtemp,
                                                uint32_t seed, float* __restrict__ part_val,
                                                int32_t* __restrict__ part_id,
                                                float* __restrict__ part_lse, int lane,
                                                const LmhMask mask = LmhMask{nullptr, 0, 1}) {
  if (mode <= 1 || mode == 4 || nvalid < LMH_TILE) {   // cheap modes, masked rows and ragged last tiles: row by row
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (trow[r] >= 0)
        lmh_select_token(logit[r], nvalid, v0, vocab_offset, bias, trow[r], tile, tiles_stride, mode, topk,
                         invtemp, seed, part_val, part_id, part_lse, lane, mask);
    return;
  }
  // full tile: every lane holds 8 valid elements per row
  uint32_t key[R][8];
  uint32_t hi[R], lo[R], ans[R];
  int nb[R];
  int maxnb = 0;
  const int k_eff = min(topk, LMH_TILE);
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float mv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float ls = trow[r] >= 0 ? logit[r][lane + 32 * j] : 0.f;
      if (bias) ls += bias[v0 + lane + 32 * j];
      mv[j] = ls;
    }
    if (mode == 3 && trow[r] >= 0) {
      float lmax = QX_NEG_INF;
#pragma unroll
      for (int j = 0; j < 8; ++j) lmax = fmaxf(lmax, mv[j] * invtemp);
      const float gmax = warp_max(lmax);
      float lsum = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) lsum += expf(mv[j] * invtemp - gmax);
      const float gsum = warp_sum(lsum);
      if (lane == 0)
        part_lse[(size_t)trow[r] * tiles_stride + tile] = gsum > 0.f ? gmax + logf(gsum) : QX_NEG_INF;
    }
    uint32_t kmax = 0u, kmin = 0xFFFFFFFFu;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      key[r][j] = float_key(mv[j]);
      kmax = max(kmax, key[r][j]);
      kmin = min(kmin, key[r][j]);
    }
    hi[r] = __reduce_max_sync(0xffffffffu, kmax);
    lo[r] = __reduce_min_sync(0xffffffffu, kmin);
    // k <= 32: every lane's largest element is among at least 32 elements >= the smallest such maximum
    if (k_eff <= 32) lo[r] = max(lo[r], __reduce_min_sync(0xffffffffu, kmax));
    nb[r] = 32 - __clz(hi[r] ^ lo[r]);
    ans[r] = nb[r] >= 32 ? 0u : (lo[r] >> nb[r]) << nb[r];
    maxnb = max(maxnb, nb[r]);
  }
  for (int b = maxnb - 1; b >= 0; --b) {
    unsigned c[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint32_t cand = ans[r] | (1u << b);
      unsigned cc = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) cc += key[r][j] >= cand ? 1u : 0u;
      c[r] = cc;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) c[r] = __reduce_add_sync(0xffffffffu, c[r]);
    int pending = 0;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (b < nb[r] && c[r] >= (unsigned)k_eff) {
        ans[r] |= 1u << b;
        if (c[r] == (unsigned)k_eff) nb[r] = 0;   // exactly k elements lie at or above ans: that is the set
      }
      pending |= nb[r];
    }
    if (pending == 0) break;
  }
  const uint32_t lt_mask = (1u << lane) - 1u;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (trow[r] < 0) continue;
    const size_t pbase = ((size_t)trow[r] * tiles_stride + tile) * topk;
    unsigned cg = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) cg += key[r][j] > ans[r] ? 1u : 0u;
    const unsigned need = (unsigned)k_eff - __reduce_add_sync(0xffffffffu, cg);   // ties to take, >= 1
    unsigned ties_before = 0u, out_pos = 0u;
#pragma unroll
    for (int j = 0; j < 8; ++j) {                       // id order = (j, lane) lexicographic
      const bool eq = key[r][j] == ans[r];
      const uint32_t bal_eq = __ballot_sync(0xffffffffu, eq);
      const bool sel = key[r][j] > ans[r] || (eq && ties_before + __popc(bal_eq & lt_mask) < need);
      const uint32_t bal = __ballot_sync(0xffffffffu, sel);
      if (sel) {
        const uint32_t pos = out_pos + __popc(bal & lt_mask);
        float ls = logit[r][lane + 32 * j];
        if (bias) ls += bias[v0 + lane + 32 * j];
        part_val[pbase + pos] = ls;
        part_id[pbase + pos] = (int)(vocab_offset + v0 + lane + 32 * j);
      }
      out_pos += __popc(bal);
      ties_before += __popc(bal_eq);
    }
    for (int kk = (int)out_pos + lane; kk < topk; kk += 32) {
      part_val[pbase + kk] = QX_NEG_INF;
      part_id[pbase + kk] = -1;
    }
  }
}

template <int FMT, typename T>
__global__ void __launch_bounds__(256)
lmh_partials_kernel(const T* __restrict__ h, const uint8_t* __restrict__ wq,
                    const float* __restrict__ bias, float* __restrict__ part_val,
                    int32_t* __restrict__ part_id, float* __restrict__ part_lse, int T_rows, int V,
                    int K, long long vocab_offset, long long tiles_stride, int mode, int topk,
                    float invtemp, uint32_t seed, const LmhMask mask) {
  constexpr int BK = block_k_of(FMT), BB = block_bytes_of(FMT);
  __shared__ float logit[LMH_TB][LMH_TILE];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tile = blockIdx.x;
  const int t0 = blockIdx.y * LMH_TB;
  const int tcount = min(LMH_TB, T_rows - t0);
  const int v0 = tile * LMH_TILE;   // tiles at or beyond V hold no rows and emit absent partials
  const size_t row_bytes = (size_t)(K / BK) * BB;
  const int spans = (K + 31) / 32;

  // ---- projection: warp w owns local rows [32w, 32w+32) ----
  for (int r = 0; r < 32; ++r) {
    const int lr = warp * 32 + r;
    const int v = v0 + lr;
    if (v >= V || v0 >= V) {
      if (lane < LMH_TB) logit[lane][lr] = QX_NEG_INF;
      continue;
    }
    const uint8_t* row = wq + (size_t)v * row_bytes;
    float acc[LMH_TB];
#pragma unroll
    for (int m = 0; m < LMH_TB; ++m) acc[m] = 0.f;
    for (int s = lane; s < spans; s += 32) {
      float w[32];
      int ncol = 32;
      if (FMT == F_NVFP4 && s * 32 + 16 >= K) {
        const uint8_t* b = row + (size_t)s * 18;
        const float sc = e4m3_to_f32(b[0]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          w[i] = sc * e2m1_to_f32(b[1 + i] & 15u);
          w[i + 8] = sc * e2m1_to_f32(b[1 + i] >> 4);
          w[i + 16] = 0.f; w[i + 24] = 0.f;
        }
        ncol = 16;
      } else {
        decode_span32<FMT>(row, s, w);
      }
#pragma unroll
      for (int m = 0; m < LMH_TB; ++m) {
        if (m < tcount) {
          const T* hp = h + (size_t)(t0 + m) * K + (size_t)s * 32;
          float a = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < ncol) a = fmaf(to_f32<T>(hp[i]), w[i], a);
          acc[m] += a;
        }
      }
    }
#pragma unroll
    for (int m = 0; m < LMH_TB; ++m) {
      const float s = warp_sum(acc[m]);
      if (lane == 0) logit[m][lr] = s;
    }
  }
  __syncthreads();

  // ---- per-token selection: warp w handles token t0 + w ----
  if (warp >= tcount) return;
  lmh_select_token(logit[warp], min(LMH_TILE, V - v0), v0, vocab_offset, bias, t0 + warp, tile,
                   tiles_stride, mode, topk, invtemp, seed, part_val, part_id, part_lse, lane, mask);
}


// Stage 1 over a dense (V, K) head in the dtype of h (the reference's unquantized lm_head_sample,
// kernels/quantization/lm_head/lm_head.metal:175-217, :400-441): same tiles, same partials, same
// score formulas as the packed form; a warp walks a vocabulary row with 16-byte loads and keeps
// fp32 sums for up to 8 hidden rows.
template <typename T>
__global__ void __launch_bounds__(256)
lmh_dense_partials_kernel(const T* __restrict__ h, const T* __restrict__ W,
                          const float* __restrict__ bias, float* __restrict__ part_val,
                          int32_t* __restrict__ part_id, float* __restrict__ part_lse, int T_rows, int V,
                          int K, long long tiles_stride, int mode, int topk, float invtemp, uint32_t seed,
                          const LmhMask mask) {
  __shared__ float logit[LMH_TB][LMH_TILE];
  constexpr int VEC = 16 / (int)sizeof(T);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tile = blockIdx.x;
  const int t0 = blockIdx.y * LMH_TB;
  const int tcount = min(LMH_TB, T_rows - t0);
  const int v0 = tile * LMH_TILE;
  const bool vec_ok = (K % VEC) == 0 && (((uintptr_t)W | (uintptr_t)h) & 15) == 0;
  for (int r = 0; r < 32; ++r) {
    const int lr = warp * 32 + r;
    const int v = v0 + lr;
    if (v >= V) {
      if (lane < LMH_TB) logit[lane][lr] = QX_NEG_INF;
      continue;
    }
    const T* row = W + (size_t)v * K;
    float acc[LMH_TB];
#pragma unroll
    for (int m = 0; m < LMH_TB; ++m) acc[m] = 0.f;
    if (vec_ok) {
      for (int c = lane * VEC; c < K; c += 32 * VEC) {
        const uint4 wv = __ldg(reinterpret_cast<const uint4*>(row + c));
        const T* we = reinterpret_cast<const T*>(&wv);
#pragma unroll
        for (int m = 0; m < LMH_TB; ++m) {
          if (m < tcount) {
            const uint4 hv = __ldg(reinterpret_cast<const uint4*>(h + (size_t)(t0 + m) * K + c));
            const T* he = reinterpret_cast<const T*>(&hv);
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[m] = fmaf(to_f32<T>(we[i]), to_f32<T>(he[i]), acc[m]);
          }
        }
      }
    } else {
      for (int c = lane; c < K; c += 32) {
        const float wv = to_f32<T>(row[c]);
#pragma unroll
        for (int m = 0; m < LMH_TB; ++m)
          if (m < tcount) acc[m] = fmaf(wv, to_f32<T>(h[(size_t)(t0 + m) * K + c]), acc[m]);
      }
    }
#pragma unroll
    for (int m = 0; m < LMH_TB; ++m) {
      const float s = warp_sum(acc[m]);
      if (lane == 0) logit[m][lr] = s;
    }
  }
  __syncthreads();
  if (warp >= tcount) return;
  lmh_select_token(logit[warp], min(LMH_TILE, V - v0), v0, 0, bias, t0 + warp, tile, tiles_stride, mode,
                   topk, invtemp, seed, part_val, part_id, part_lse, lane, mask);
}

void launch_lm_head_dense_partials(cudaStream_t st, const void* h, const void* W, const float* bias,
                                   float* part_val, int32_t* part_id, int64_t T, int64_t V, int64_t K,
                                   qx_dtype dtype, int mode, int topk, float invtemp, uint32_t seed,
                                   float* part_lse, const LmhMask mask) {
  const long long tiles = (V + LMH_TILE - 1) / LMH_TILE;
  dim3 grid((unsigned)tiles, (unsigned)((T + LMH_TB - 1) / LMH_TB));
  if (dtype == QX_DTYPE_F32)
    lmh_dense_partials_kernel<float><<<grid, 256, 0, st>>>((const float*)h, (const float*)W, bias, part_val, part_id, part_lse,
                                                            (int)T, (int)V, (int)K, tiles, mode, topk, invtemp, seed, mask);
  else if (dtype == QX_DTYPE_F16)
    lmh_dense_partials_kernel<__half><<<grid, 256, 0, st>>>((const __half*)h, (const __half*)W, bias, part_val, part_id, part_lse,
                                                             (int)T, (int)V, (int)K, tiles, mode, topk, invtemp, seed, mask);
  else
    lmh_dense_partials_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)h, (const __nv_bfloat16*)W, bias,
                                                                    part_val, part_id, part_lse, (int)T, (int)V, (int)K, tiles,
                                                                    mode, topk, invtemp, seed, mask);
  note_launch();
}

// ------------------------------------------------------------------------------------------
// Stage 1, streaming tensor-core form (bf16 / f16 hidden rows, aligned shapes): the projection
// runs on the per-warp weight stream of qx_stream.cuh.  A CTA is 8 warps and owns one 256-row
// vocabulary tile at a time; warp w streams rows [32w, 32w+32) of the tile over the full K
// (two 16-row m-tiles sharing every activation fragment) for up to 64 hidden rows at once, so the
// packed weights are read exactly once per pass.  The logits stay in the accumulator registers
// and visit shared memory 16 hidden rows at a time for the per-tile selection.
// ------------------------------------------------------------------------------------------
template <int FMT> struct LmhCfg;      // columns per stage and ring depth that fit 8 warps x 32 rows
template <> struct LmhCfg<F_Q8_0>  { static constexpr int KC = 256, STAGES = 2; };
template <> struct LmhCfg<F_Q4_0>  { static constexpr int KC = 256, STAGES = 4; };
template <> struct LmhCfg<F_NVFP4> { static constexpr int KC = 256, STAGES = 4; };
template <> struct LmhCfg<F_MXFP4> { static constexpr int KC = 512, STAGES = 2; };
template <> struct LmhCfg<F_MXFP8> { static constexpr int KC = 128, STAGES = 2; };

// QX_LMH_UNROLL: whole stages run fully unrolled for up to this many 8-row n-tiles.
// QX_LMH_WROWS16_MIN_NT: n-tiles from which a CTA is 16 warps of 16 rows instead of 8 warps of 32.
#ifndef QX_LMH_WROWS16_MIN_NT
#define QX_LMH_WROWS16_MIN_NT 2
#endif
#ifndef QX_LMH_UNROLL
#define QX_LMH_UNROLL 2
#endif
constexpr int LMH_LOGIT_PITCH = 257;
constexpr int LMH_TOK_CHUNK = 16;

// WROWS = vocabulary rows per warp: 32 (8 warps, two m-tiles share every activation fragment) or
// 16 (16 warps: more loads in flight; used from 9 hidden rows per pass).
// XS: a single hidden row, prepared by every CTA itself into shared memory (xsrc = the raw 16-bit row,
// bf16 if x_bf16 else f16; x16 / rowscale unused) instead of by the preparation kernel.
template <int FMT, int NT, int WROWS, bool XS>
__global__ void __launch_bounds__(256 / WROWS * 32, 1)
lmh_stream_kernel(const __grid_constant__ CUtensorMap wmap, const __half* __restrict__ x16,
                  const float* __restrict__ rowscale, const uint16_t* __restrict__ xsrc, int x_bf16,
                  const float* __restrict__ bias,
                  float* __restrict__ part_val, int32_t* __restrict__ part_id,
                  float* __restrict__ part_lse, int T_total, int tokens_per_group, int V, int K,
                  long long vocab_offset, long long tiles_stride, int mode, int topk, float invtemp,
                  uint32_t seed, const LmhMask mask, int* __restrict__ err_flag) {
  using F = StreamFmt<FMT>;
  using C = LmhCfg<FMT>;
  asm volatile("griddepcontrol.launch_dependents;");   // the merge stage may be scheduled; it waits for this grid's end
  constexpr int NW = 256 / WROWS;             // warps per CTA
  constexpr int NSETS = WROWS / 16;
  using WS = WarpStream<FMT, C::KC, WROWS, C::STAGES>;
  using GP = GroupProc<FMT>;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  // Work items are (vocabulary tile, group of hidden rows) pairs, the group index running fastest
  // so that the CTAs that stream the same tile for different row groups run at the same time and
  // share the tile through L2.
  const int groups = (T_total + tokens_per_group - 1) / tokens_per_group;

  uint8_t* ring = smem_raw + (size_t)warp * WS::WARP_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)NW * WS::WARP_BYTES) + warp * C::STAGES;
  float* logit = reinterpret_cast<float*>(smem_raw + (size_t)NW * WS::WARP_BYTES + (size_t)NW * C::STAGES * 8);

  WS ws;
  ws.init(smem_u32(ring), smem_u32(bars), &wmap, &wmap, 16, K, lane, err_flag);   // rows 16..31: same matrix

  const int real_tiles = (V + LMH_TILE - 1) / LMH_TILE;
  const int items = real_tiles * groups;
  const int my_tiles = (int)blockIdx.x < items ? (items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int nch = ws.nch;
  const int steps = my_tiles * nch;
  auto step_row0 = [&](int i) { return (((int)blockIdx.x + (i / nch) * (int)gridDim.x) / groups) * LMH_TILE + warp * WROWS; };

#pragma unroll
  for (int p = 0; p < C::STAGES - 1; ++p)
    if (p < steps) ws.issue(p, step_row0(p), p % nch);
  // Programmatic dependent launch: the weight boxes above do not depend on the kernel before this one
  // (the preparation kernel, or with XS whatever produced the hidden row); everything below does.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  using XP = typename std::conditional<XS, SmemRow, const __half*>::type;
  uint8_t* xs_base = reinterpret_cast<uint8_t*>(logit + LMH_TOK_CHUNK * LMH_LOGIT_PITCH);   // XS: behind the logit buffer
  const float* rs_ptr = rowscale;
  if constexpr (XS) {
    static_assert(NT == 1, "in-kernel preparation: one row");
    cta_prepare_row<F::PERM>(xs_base, xsrc, x_bf16, K);
    rs_ptr = reinterpret_cast<const float*>(xs_base + (size_t)K * 2);
  }

  float acc[NSETS][NT][4];
  for (int j = 0; j < my_tiles; ++j) {
    const int item = (int)blockIdx.x + j * (int)gridDim.x;
    const int tile = item / groups;
    const int t_base = (item % groups) * tokens_per_group;
    const int T_pass = min(tokens_per_group, T_total - t_base);
    const int row0 = tile * LMH_TILE + warp * WROWS;
    XP xr[NT];
    if constexpr (XS) {
      xr[0] = SmemRow{g == 0 ? smem_u32(xs_base) : 0u};
    } else {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int m = nt * 8 + g;
        xr[nt] = m < T_pass ? x16 + (size_t)(t_base + m) * K : nullptr;
      }
    }
#pragma unroll
    for (int a = 0; a < NSETS; ++a)
#pragma unroll
      for (int b = 0; b < NT; ++b)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;

    for (int c = 0; c < nch; ++c) {
      const int i = j * nch + c;
      const int stage = i % C::STAGES;
      const int nxt = i + C::STAGES - 1;
      if (nxt < steps) ws.issue(nxt % C::STAGES, step_row0(nxt), nxt % nch);
      const bool ready = ws.wait(stage, (uint32_t)((i / C::STAGES) & 1));
      const int col_base = c * C::KC;
      const int ngroups = ready ? min(C::KC, K - col_base) / F::GROUP : 0;
      uint32_t s[2 * NSETS];
      s[0] = ws.slot_addr(stage, g, c);
      s[1] = ws.slot_addr(stage, g + 8, c);
      if constexpr (NSETS == 2) {
        s[2] = ws.slot_addr(stage, 16 + g, c);
        s[3] = ws.slot_addr(stage, 24 + g, c);
      }
      constexpr uint32_t GROUP_BYTES = F::GROUP / F::BK * F::BB;
      if constexpr (NT > 2 && GP::PIPED) {
        uint4 bcar[NT];                              // fragments of the next unit, fetched one unit ahead
        if (ngroups > 0) GP::template load_first<NT>(xr, col_base, t, bcar);
        for (int gi = 0; gi < ngroups; ++gi) {
          GP::template piped<NSETS, NT, 0>(s, t, xr, col_base + gi * F::GROUP, gi + 1 < ngroups, bcar, acc);
#pragma unroll
          for (int r = 0; r < 2 * NSETS; ++r) s[r] += GROUP_BYTES;
        }
      } else {
        constexpr bool PRE = NT <= 2;               // prefetch activations one group ahead
        typename GP::template BFrag<NT> bcur, bnext;
        if (PRE && ngroups > 0) GP::template load_b<NT>(xr, col_base, t, bcur);
        constexpr int FULL = C::KC / F::GROUP;
        if (QX_LMH_UNROLL >= NT && ngroups == FULL) {
          // a whole stage: fully unrolled (immediate shared-memory offsets, no fragment moves)
#pragma unroll
          for (int gi = 0; gi < FULL; ++gi) {
            if (PRE && gi + 1 < FULL) GP::template load_b<NT>(xr, col_base + (gi + 1) * F::GROUP, t, bnext);
            GP::template run<NSETS, NT, PRE>(s, t, bcur, xr, col_base + gi * F::GROUP, acc);
            if (PRE) bcur = bnext;
#pragma unroll
            for (int r = 0; r < 2 * NSETS; ++r) s[r] += GROUP_BYTES;
          }
        } else {
          for (int gi = 0; gi < ngroups; ++gi) {
            if (PRE && gi + 1 < ngroups) GP::template load_b<NT>(xr, col_base + (gi + 1) * F::GROUP, t, bnext);
            GP::template run<NSETS, NT, PRE>(s, t, bcur, xr, col_base + gi * F::GROUP, acc);
            if (PRE) bcur = bnext;
#pragma unroll
            for (int r = 0; r < 2 * NSETS; ++r) s[r] += GROUP_BYTES;
          }
        }
      }
      __syncwarp();
    }

    // ---- selection, 16 hidden rows (two n-tiles) at a time ----
    const int v0 = tile * LMH_TILE;
    const int nvalid = min(LMH_TILE, V - v0);
#pragma unroll
    for (int tc = 0; tc < (NT + 1) / 2; ++tc) {
      __syncthreads();                              // previous chunk's readers are done
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int nt = 2 * tc + h;
        if (nt < NT) {
#pragma unroll
          for (int set = 0; set < NSETS; ++set)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int ml = h * 8 + 2 * t + (e & 1);
              const int m = nt * 8 + 2 * t + (e & 1);
              const float rs = m < T_pass ? rs_ptr[t_base + m] * GP::ACC_SCALE : 0.f;
              logit[ml * LMH_LOGIT_PITCH + warp * WROWS + set * 16 + g + (e >> 1) * 8] = acc[set][nt][e] * rs;
            }
        }
      }
      __syncthreads();
#pragma unroll
      for (int ml = warp; ml < LMH_TOK_CHUNK; ml += NW) {   // each warp reduces some of the 16 rows
        const int m = tc * LMH_TOK_CHUNK + ml;
        if (m < T_pass)
          lmh_select_token(logit + ml * LMH_LOGIT_PITCH, nvalid, v0, vocab_offset, bias, t_base + m,
                           tile, tiles_stride, mode, topk, invtemp, seed, part_val, part_id, part_lse,
                           lane, mask);
      }
    }
  }

  // padding tiles of a short shard carry absent partials
  for (long long tile = real_tiles + blockIdx.x; tile < tiles_stride; tile += gridDim.x) {
    for (int m = warp; m < T_total; m += NW)
      lmh_select_token(logit, 0, 0, vocab_offset, nullptr, m, (int)tile, tiles_stride, mode,
                       topk, invtemp, seed, part_val, part_id, part_lse, lane);
  }
}

}  // namespace qx
#include "qx_tc_pipeline.cuh"
namespace qx {

// Epilogue of the tensor-core pipeline for LM-head stage 1: the worker warps move the logits of the
// item's 256 vocabulary rows to shared memory ([hidden row][256]), then every warp reduces hidden
// rows to their tile partials.
template <int BN>
struct LmhEpi {
  struct Args {
    const float* bias;
    float* part_val; int32_t* part_id; float* part_lse;
    int T_total, V;
    long long vocab_offset, tiles_stride;
    int mode, topk;
    float invtemp;
    uint32_t seed;
    // items shared by several CTAs (each took a slice of K): where the other CTAs leave their partial
    // logits ([shared item][part - 1][BN * 256] floats), the flags that say so, and the value that
    // means "written during this launch"
    float* xchg; unsigned* flags; unsigned epoch;
    int* err_flag;
    LmhMask mask;
  };
  static constexpr bool DUAL = false;
  __device__ __forceinline__ static void run(const Args& a, const TcItem& it) {
    constexpr int CW = BN / 4;
    if (it.warp < LTC_DQW) {
      const uint32_t lane_sel = (uint32_t)((it.warp & 3) * 32) << 16;
      const int RS = (it.warp & 3) * 32 + it.lane;
      const int cg = it.warp >> 2;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t v[CW];
        tmem_ld_nowait<CW>(it.tmem_base + lane_sel + (uint32_t)(h * BN + cg * CW), v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < CW; ++i) {
          const int m = cg * CW + i;
          const float rs = m < it.m_count ? it.rowscale[it.m_base + m] : 0.f;
          it.smem_f32[m * LMH_TILE + h * 128 + RS] = __uint_as_float(v[i]) * rs;
        }
      }
    }
    tc_fence_before();
    __syncthreads();
    if (it.kparts > 1) {
      // the logits above are this CTA's slice of K; part 0 collects the others and selects
      constexpr int N4 = BN * LMH_TILE / 4;
      const int tid = it.warp * 32 + it.lane;
      float4* mine = reinterpret_cast<float4*>(it.smem_f32);
      float* slots = a.xchg + (size_t)it.split_index * (it.kparts - 1) * (BN * LMH_TILE);
      unsigned* fl = a.flags + it.split_index * (it.kparts - 1);
      if (it.kpart != 0) {
        float4* dst = reinterpret_cast<float4*>(slots + (size_t)(it.kpart - 1) * (BN * LMH_TILE));
        for (int i = tid; i < N4; i += LTC_WARPS * 32) dst[i] = mine[i];
        __threadfence();
        __syncthreads();
        if (tid == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(fl + it.kpart - 1), "r"(a.epoch) : "memory");
        return;
      }
      if (tid == 0) {
        for (int p = 1; p < it.kparts; ++p) {
          bool seen = false;
          for (int k = 0; k < (1 << 22) && !seen; ++k) {      // bounded: about a second
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(fl + p - 1) : "memory");
            seen = v == a.epoch;
            if (!seen) __nanosleep(200);
          }
          if (!seen) atomicExch(a.err_flag, 4);
        }
      }
      __syncthreads();
      for (int p = 1; p < it.kparts; ++p) {
        const float4* src = reinterpret_cast<const float4*>(slots + (size_t)(p - 1) * (BN * LMH_TILE));
        for (int i = tid; i < N4; i += LTC_WARPS * 32) {
          const float4 o = __ldcg(src + i);
          float4 v = mine[i];
          v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
          mine[i] = v;
        }
      }
      __syncthreads();
    }
    const int v0 = it.tile * LMH_TILE;
    const int nvalid = min(LMH_TILE, a.V - v0);
    // every warp takes up to four hidden rows (warp, warp + 18, ...) and reduces them together
    constexpr int RPW = (BN + LTC_WARPS - 1) / LTC_WARPS;
    const float* rows[RPW];
    int trow[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int m = it.warp + r * LTC_WARPS;
      rows[r] = it.smem_f32 + (m < it.m_count ? m : 0) * LMH_TILE;
      trow[r] = m < it.m_count ? it.m_base + m : -1;
    }
    lmh_select_rows<RPW>(rows, trow, nvalid, v0, a.vocab_offset, a.bias, it.tile, a.tiles_stride, a.mode, a.topk,
                         a.invtemp, a.seed, a.part_val, a.part_id, a.part_lse, it.lane, a.mask);
  }
  // padding tiles of a short shard carry absent partials
  __device__ __forceinline__ static void tail(const Args& a, const float* scratch, int real_tiles, int warp, int lane) {
    for (long long tile = real_tiles + blockIdx.x; tile < a.tiles_stride; tile += gridDim.x)
      for (int m = warp; m < a.T_total; m += LTC_WARPS)
        lmh_select_token(scratch, 0, 0, a.vocab_offset, nullptr, m, (int)tile, a.tiles_stride, a.mode,
                         a.topk, a.invtemp, a.seed, a.part_val, a.part_id, a.part_lse, lane);
  }
};

template <int FMT>
static bool lmh_stream_ok(const LmHeadArgs& a) {
  using F = StreamFmt<FMT>;
  const size_t row_bytes = (size_t)(a.K / F::BK) * F::BB;
  return (a.dtype == QX_DTYPE_BF16 || a.dtype == QX_DTYPE_F16) && a.K % LmhCfg<FMT>::KC == 0 &&
         row_bytes % 16 == 0 && ((uintptr_t)a.wq & 15) == 0 && a.V >= 32;
}

template <int FMT, int NT, bool XS>
static void launch_lmh_stream_nt(cudaStream_t st, const LmHeadArgs& a, const __half* x16,
                                 const float* rowscale, float* pv, int32_t* pi, float* pl,
                                 int64_t tiles_stride, int* err, const CUtensorMap& wmap) {
  using C = LmhCfg<FMT>;
  constexpr int WROWS = NT >= QX_LMH_WROWS16_MIN_NT ? 16 : 32;
  constexpr int NW = 256 / WROWS;
  using WS = WarpStream<FMT, C::KC, WROWS, C::STAGES>;
  const size_t smem = (size_t)NW * WS::WARP_BYTES + (size_t)NW * C::STAGES * 8 +
                      (size_t)LMH_TOK_CHUNK * LMH_LOGIT_PITCH * 4 + (XS ? cta_prepared_row_bytes((size_t)a.K) : 0);
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaFuncSetAttribute(lmh_stream_kernel<FMT, NT, WROWS, XS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    attr_set[dev] = true;
  }
  const int real_tiles = (int)((a.V + LMH_TILE - 1) / LMH_TILE);
  const int tpg = NT * 8;
  const long long items = (long long)real_tiles * ((a.T + tpg - 1) / tpg);
  const unsigned blocks = (unsigned)(items < sm_count() ? items : sm_count());
  // a programmatic dependent of the kernel before it (see griddepcontrol.wait in the kernel)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(NW * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, lmh_stream_kernel<FMT, NT, WROWS, XS>, wmap, x16, rowscale, (const uint16_t*)a.h,
                         (int)(a.dtype == QX_DTYPE_BF16), a.bias, pv, pi, pl, (int)a.T, tpg, (int)a.V, (int)a.K,
                         (long long)a.vocab_offset, (long long)tiles_stride, a.mode, a.topk, a.invtemp, a.seed,
                         a.mask, err) != cudaSuccess) {
    cudaGetLastError();
    lmh_stream_kernel<FMT, NT, WROWS, XS><<<blocks, NW * 32, smem, st>>>(
        wmap, x16, rowscale, (const uint16_t*)a.h, (int)(a.dtype == QX_DTYPE_BF16), a.bias, pv, pi, pl, (int)a.T, tpg,
        (int)a.V, (int)a.K, (long long)a.vocab_offset, (long long)tiles_stride, a.mode, a.topk, a.invtemp, a.seed,
        a.mask, err);
  }
  note_launch();
}

// ---- stage-1 scratch ----------------------------------------------------------------------------
// [0, 1 KB)  release flags of K-split items (cleared before every launch that shares items)
// [1 KB, ..) prepared activations (row-major, or the operand-tile image in groups of 32 / 64 rows)
// then       one fp32 row scale per hidden row
// then       exchange slots of K-split items, as far as the scratch reaches
constexpr size_t LMH_FLAG_BYTES = 1024;
static size_t lmh_round256(size_t n) { return (n + 255) & ~(size_t)255; }
static size_t lmh_act_bytes(int64_t T, int64_t K) { return lmh_round256((size_t)((T + 63) / 64 * 64) * K * 2); }
size_t lm_head_scratch_min_bytes(int64_t T, int64_t K) {
  return LMH_FLAG_BYTES + lmh_act_bytes(T, K) + lmh_round256((size_t)T * 4);
}
size_t lm_head_scratch_full_bytes(int64_t T, int64_t K) {
  // at most 3/4 of the SMs hold a partner slot of 64 x 256 floats
  return lm_head_scratch_min_bytes(T, K) + (T > 16 ? (size_t)(3 * sm_count() / 4) * 64 * LMH_TILE * 4 : 0);
}
struct LmhScratch {
  unsigned* flags; __half* act; float* rowscale; float* xchg; size_t xchg_bytes;
};
static bool lmh_carve(const LmHeadArgs& a, LmhScratch* out) {
  const size_t need = lm_head_scratch_min_bytes(a.T, a.K);
  if (!a.scratch || a.scratch_bytes < need) return false;
  char* p = (char*)a.scratch;
  out->flags = (unsigned*)p;
  out->act = (__half*)(p + LMH_FLAG_BYTES);
  out->rowscale = (float*)(p + LMH_FLAG_BYTES + lmh_act_bytes(a.T, a.K));
  out->xchg = (float*)(p + need);
  out->xchg_bytes = a.scratch_bytes - need;
  return true;
}

// tcgen05 form of stage 1 for more than 16 hidden rows.
template <int FMT, int BN>
static bool launch_lmh_tc_bn(cudaStream_t st, const LmHeadArgs& a, float* pv, int32_t* pi, float* pl,
                             int64_t tiles_stride, int* err) {
  using S = TcSmem<FMT, BN>;
  using C = TcCfg<FMT>;
  using Epi = LmhEpi<BN>;
  static_assert(S::TOTAL <= 227 * 1024, "stage-1 tensor-core configuration exceeds shared memory");
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute(tc_pipeline_kernel<FMT, BN, Epi>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    attr_set[dev] = true;
  }
  LmhScratch sc;
  if (!lmh_carve(a, &sc)) return false;
  const size_t row_bytes = (size_t)(a.K / StreamFmt<FMT>::BK) * StreamFmt<FMT>::BB;
  CUtensorMap wmap;
  if (!cached_weight_map(&wmap, a.wq, a.V, row_bytes, C::BOX)) return false;
  const int groups = (int)((a.T + BN - 1) / BN);
  const int real_tiles = (int)((a.V + LMH_TILE - 1) / LMH_TILE);
  const long long items = (long long)real_tiles * groups;
  // The last, partial round of items (all items, when there are fewer than SMs - a small vocabulary
  // shard): when it would leave at least half of the SMs idle, each of its items is shared by 2 or
  // 4 CTAs that take a slice of K each, as far as the exchange slots fit the scratch.
  const int nks = (int)(a.K / LTC_KS);
  const long long sms = sm_count();
  const long long leftover = items % sms;
  int ksplit = 1;
  // not while the stream is being captured: a cooperative launch that fails there would
  // invalidate the capture, and there is no second attempt inside one
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  cudaStreamIsCapturing(st, &cap);
  const size_t slot_bytes = (size_t)BN * LMH_TILE * 4;
  auto fits = [&](int ks) {
    return (size_t)leftover * (ks - 1) * slot_bytes <= sc.xchg_bytes && (size_t)leftover * (ks - 1) * 4 <= LMH_FLAG_BYTES;
  };
  if (options().lm_head_ksplit && leftover > 0 && cap == cudaStreamCaptureStatusNone) {
    if (leftover * 4 <= sms && nks % 4 == 0 && fits(4)) ksplit = 4;
    else if (leftover * 2 <= sms && nks % 2 == 0 && fits(2)) ksplit = 2;
  }
  const unsigned grid = (unsigned)(items >= sms ? sms : items * ksplit);
  static std::atomic<unsigned> epoch_counter{1};
  const unsigned epoch = epoch_counter.fetch_add(1) | 0x40000000u;     // never 0
  launch_prep_activations(st, a.h, a.dtype, sc.act, sc.rowscale, (int)a.T, (int)a.K, StreamFmt<FMT>::PERM, BN);
  note_launch();
  const typename Epi::Args ea{a.bias, pv, pi, pl, (int)a.T, (int)a.V, (long long)a.vocab_offset,
                              (long long)tiles_stride, a.mode, a.topk, a.invtemp, a.seed,
                              sc.xchg, sc.flags, epoch, err, a.mask};
  bool launched = false;
  if (ksplit > 1) {
    // the flags start every launch at zero, whatever an earlier user of the scratch left there
    if (cudaMemsetAsync(sc.flags, 0, LMH_FLAG_BYTES, st) != cudaSuccess) { cudaGetLastError(); ksplit = 1; }
  }
  if (ksplit > 1) {
    // CTAs of this launch wait for one another: ask for a cooperative launch, which only starts
    // when the whole grid is resident
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(LTC_WARPS * 32);
    cfg.dynamicSmemBytes = S::TOTAL;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    launched = cudaLaunchKernelEx(&cfg, tc_pipeline_kernel<FMT, BN, Epi>, wmap, wmap, (const __half*)sc.act,
                                  (const float*)sc.rowscale, (int)a.T, (int)a.V, (int)a.K, ksplit, err, ea) == cudaSuccess;
    if (!launched) { cudaGetLastError(); ksplit = 1; }
  }
  if (!launched) {
    const unsigned grid1 = (unsigned)(items >= sms ? sms : items);
    tc_pipeline_kernel<FMT, BN, Epi><<<grid1, LTC_WARPS * 32, S::TOTAL, st>>>(
        wmap, wmap, sc.act, sc.rowscale, (int)a.T, (int)a.V, (int)a.K, 1, err, ea);
  }
  note_launch();
  return true;
}

template <int FMT>
static bool launch_lmh_tc(cudaStream_t st, const LmHeadArgs& a, float* pv, int32_t* pi, float* pl,
                          int64_t tiles_stride, int* err) {
  if (a.T <= 16 || a.K % LTC_KS != 0 || a.V < 128) return false;
  if (a.T <= 32) return launch_lmh_tc_bn<FMT, 32>(st, a, pv, pi, pl, tiles_stride, err);
  return launch_lmh_tc_bn<FMT, 64>(st, a, pv, pi, pl, tiles_stride, err);
}

template <int FMT>
static bool launch_lmh_stream(cudaStream_t st, const LmHeadArgs& a, float* pv, int32_t* pi, float* pl,
                              int64_t tiles_stride) {
  if (!lmh_stream_ok<FMT>(a)) return false;
  int* err = device_error_flag();
  if (!err) return false;
  if (launch_lmh_tc<FMT>(st, a, pv, pi, pl, tiles_stride, err)) return true;
  LmhScratch sc;
  if (!lmh_carve(a, &sc)) return false;
  CUtensorMap wmap;
  {
    const size_t row_bytes = (size_t)(a.K / StreamFmt<FMT>::BK) * StreamFmt<FMT>::BB;
    if (!cached_weight_map(&wmap, a.wq, a.V, row_bytes, StageGeom<FMT, LmhCfg<FMT>::KC>::PITCH, 16)) return false;
  }
  __half* x16 = sc.act;
  float* rowscale = sc.rowscale;
  // a single hidden row is prepared by the stage-1 CTAs themselves (one launch less per decoded token)
  using WS1 = WarpStream<FMT, LmhCfg<FMT>::KC, 32, LmhCfg<FMT>::STAGES>;
  if (a.T == 1 && ((uintptr_t)a.h & 15) == 0 && a.K % 8 == 0 &&
      (size_t)8 * WS1::WARP_BYTES + (size_t)8 * LmhCfg<FMT>::STAGES * 8 + (size_t)LMH_TOK_CHUNK * LMH_LOGIT_PITCH * 4 +
              cta_prepared_row_bytes((size_t)a.K) <= 227 * 1024) {
    launch_lmh_stream_nt<FMT, 1, true>(st, a, nullptr, nullptr, pv, pi, pl, tiles_stride, err, wmap);
    return true;
  }
  launch_prep_activations(st, a.h, a.dtype, x16, rowscale, (int)a.T, (int)a.K, StreamFmt<FMT>::PERM);
  note_launch();
  // hidden rows per CTA: 64 when there are enough vocabulary tiles to fill the GPU; fewer rows
  // per CTA (more CTAs, each re-reading the weights from L2) when the vocabulary shard is small
  const int real_tiles = (int)((a.V + LMH_TILE - 1) / LMH_TILE);
  int tpg = 64;
  while (tpg > 8 && (long long)real_tiles * ((a.T + tpg - 1) / tpg) < sm_count() && a.T > tpg / 2) tpg >>= 1;
  while (tpg > 8 && a.T <= tpg / 2) tpg >>= 1;
  if (tpg <= 8) launch_lmh_stream_nt<FMT, 1, false>(st, a, x16, rowscale, pv, pi, pl, tiles_stride, err, wmap);
  else if (tpg <= 16) launch_lmh_stream_nt<FMT, 2, false>(st, a, x16, rowscale, pv, pi, pl, tiles_stride, err, wmap);
  else if (tpg <= 32) launch_lmh_stream_nt<FMT, 4, false>(st, a, x16, rowscale, pv, pi, pl, tiles_stride, err, wmap);
  else launch_lmh_stream_nt<FMT, 8, false>(st, a, x16, rowscale, pv, pi, pl, tiles_stride, err, wmap);
  return true;
}

static bool launch_lmh_stream_any(cudaStream_t st, const LmHeadArgs& a, float* pv, int32_t* pi,
                                  float* pl, int64_t ts) {
  if (options().force_generic) return false;
  switch (a.format) {
    case F_Q8_0: return launch_lmh_stream<F_Q8_0>(st, a, pv, pi, pl, ts);
    case F_Q4_0: return launch_lmh_stream<F_Q4_0>(st, a, pv, pi, pl, ts);
    case F_NVFP4: return launch_lmh_stream<F_NVFP4>(st, a, pv, pi, pl, ts);
    case F_MXFP4: return launch_lmh_stream<F_MXFP4>(st, a, pv, pi, pl, ts);
    case F_MXFP8: return launch_lmh_stream<F_MXFP8>(st, a, pv, pi, pl, ts);
    default: return false;    // q6_K heads take the generic kernel
  }
}

// ------------------------------------------------------------------------------------------
// Stage 2
// ------------------------------------------------------------------------------------------

__global__ void __launch_bounds__(LMH_RED_THREADS)
lmh_reduce_kernel(const float* __restrict__ cand_val, const int32_t* __restrict__ cand_id,
                  const float* __restrict__ cand_lse, int shards, int T_rows, long long ncand_s,
                  long long nlse_s, long long shard_stride, long long lse_stride,
                  int cache_elems, int mode,
                  int topk, float invtemp, uint32_t seed, float top_p, int32_t* __restrict__ ids,
                  int emit_set, float* __restrict__ out_val, int32_t* __restrict__ out_id) {
  __shared__ BlockScratch S;
  // Programmatic dependent launch: this grid may be scheduled while the kernel before it (stage 1, or the
  // exchange) still runs; nothing is read or written before that kernel has completed.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int t = blockIdx.x;
  const int tid = threadIdx.x, nth = blockDim.x;
  // candidates of row t: shard s contributes ncand_s entries at (s*shard_stride + t*ncand_s + j)
  // (tile lses: s*shard_stride + t*nlse_s + j)
  extern __shared__ float cache[];                // mode 3: tempered logits + their exponentials
  const long long ncand = ncand_s * shards;
  const long long nlse = nlse_s * shards;
  struct View {
    const float* v; const int32_t* i; long long per, hop;
    __device__ __forceinline__ long long at(long long j) const {
      return per == 0 ? j : (j / per) * hop + (j % per);
    }
  };
  const View vw{cand_val + (size_t)t * ncand_s, cand_id + (size_t)t * ncand_s,
                shards > 1 ? ncand_s : 0, shard_stride};
#define cv(j) vw.v[vw.at(j)]
#define ci(j) vw.i[vw.at(j)]

  if (mode <= 1) {
    float best = QX_NEG_INF;
    int bid = 0x7fffffff;
    for (long long j = tid; j < ncand; j += nth) {
      const int id = ci(j);
      if (id >= 0 && better(cv(j), id, best, bid)) { best = cv(j); bid = id; }
    }
    block_argmax(best, bid, S);
    if (tid == 0) {
      if (emit_set) { out_val[t] = best; out_id[t] = bid == 0x7fffffff ? -1 : bid; }
      else ids[t] = bid;
    }
    return;
  }

  if (mode == 2) {
    // ---- exact top-k membership by radix select over candidate keys ----
    // `finish` selects among n candidates given by accessors and emits the result.
    auto finish = [&](long long n, auto val, auto idf) {
      unsigned nvalid_l = 0;
      for (long long j = tid; j < n; j += nth) nvalid_l += idf(j) >= 0 ? 1u : 0u;
      const unsigned nvalid = block_sum_u(nvalid_l, S);
      uint32_t tau = 0u;
      int id_cut = 0x7fffffff;
      if (nvalid > (unsigned)topk) {
        unsigned remaining = (unsigned)topk, count_eq = 0;
        block_radix_select(n, [&](long long j, uint32_t& kx) {
          if (idf(j) < 0) return false;
          kx = float_key(val(j));
          return true;
        }, (unsigned)topk, S, tau, remaining, count_eq);
        if (count_eq > remaining) {
          // several candidates share the threshold value: keep the `remaining` smallest ids
          int cut = -1;
          for (unsigned r = 0; r < remaining; ++r) {
            int mine = 0x7fffffff;
            for (long long j = tid; j < n; j += nth) {
              const int id = idf(j);
              if (id > cut && float_key(val(j)) == tau) mine = min(mine, id);
            }
            cut = block_min_int(mine, S);
          }
          id_cut = cut;
        }
      }
      if (emit_set) {
        if (tid == 0) S.u[3] = 0u;
        __syncthreads();
        for (long long j = tid; j < n; j += nth) {
          const int id = idf(j);
          if (id < 0) continue;
          const uint32_t key = float_key(val(j));
          if (key > tau || (key == tau && id <= id_cut)) {
            const unsigned slot = atomicAdd(&S.u[3], 1u);
            if (slot < (unsigned)topk) {
              out_val[(size_t)t * topk + slot] = val(j);
              out_id[(size_t)t * topk + slot] = id;
            }
          }
        }
        __syncthreads();
        for (unsigned slot = S.u[3] + tid; slot < (unsigned)topk; slot += nth) {
          out_val[(size_t)t * topk + slot] = QX_NEG_INF;
          out_id[(size_t)t * topk + slot] = -1;
        }
        return;
      }
      float best = QX_NEG_INF;
      int bid = 0x7fffffff;
      constexpr int U = 8;                           // candidates fetched per thread before any is judged
      for (long long j0 = tid; j0 < n; j0 += (long long)nth * U) {
        int idu[U];
        float vu[U];
  #pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long j = j0 + (long long)u * nth;
          idu[u] = j < n ? idf(j) : -1;
          vu[u] = j < n ? val(j) : 0.f;
        }
  #pragma unroll
        for (int u = 0; u < U; ++u) {
          if (idu[u] < 0) continue;
          const uint32_t key = float_key(vu[u]);
          if (key > tau || (key == tau && idu[u] <= id_cut)) {
            const float p = vu[u] * invtemp + rng_gumbel(seed, (uint32_t)t, (uint32_t)idu[u]);
            if (better(p, idu[u], best, bid)) { best = p; bid = idu[u]; }
          }
        }
      }
      block_argmax(best, bid, S);
      if (tid == 0) ids[t] = bid == 0x7fffffff ? -1 : bid;
      return;
    };
    // Candidates arrive in groups of topk (one group per vocabulary tile): the topk-th largest of the
    // group maxima is a lower bound of the topk-th largest candidate, so only the candidates at or
    // above it - a few hundred of tens of thousands - are copied to shared memory and searched
    // exactly.  Without the group structure (already merged sets, few groups) or when more than
    // LMH_RED_COMPACT candidates pass (massive ties), every candidate is searched as it lies.
    const int ngroups = cache_elems;
    if (ngroups >= topk && (long long)ngroups * topk == ncand) {
      uint32_t* g_key = reinterpret_cast<uint32_t*>(cache);
      float* l_val = cache + ngroups;
      int* l_id = reinterpret_cast<int*>(l_val + LMH_RED_COMPACT);
      const int lane = tid & 31, warp = tid >> 5, nwarps = nth >> 5;
      unsigned present_l = 0;
      for (int grp = warp; grp < ngroups; grp += nwarps) {
        uint32_t best = 0u;
        for (int e = lane; e < topk; e += 32) {
          const long long j = (long long)grp * topk + e;
          if (ci(j) >= 0) best = max(best, max(float_key(cv(j)), 1u));
        }
        best = __reduce_max_sync(0xffffffffu, best);
        if (lane == 0) { g_key[grp] = best; present_l += best != 0u ? 1u : 0u; }
      }
      __syncthreads();
      const unsigned present = block_sum_u(present_l, S);
      if (present >= (unsigned)topk) {
        uint32_t tau0 = 0u;
        unsigned rem0 = 0, ceq0 = 0;
        block_radix_select(ngroups, [&](long long gi, uint32_t& kx) {
          kx = g_key[gi];
          return kx != 0u;
        }, (unsigned)topk, S, tau0, rem0, ceq0);
        if (tid == 0) S.u[4] = 0u;
        __syncthreads();
        constexpr int U = 8;
        for (long long j0 = tid; j0 < ncand; j0 += (long long)nth * U) {
          int idu[U];
          float vu[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const long long j = j0 + (long long)u * nth;
            idu[u] = j < ncand ? ci(j) : -1;
            vu[u] = j < ncand ? cv(j) : 0.f;
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (idu[u] < 0 || max(float_key(vu[u]), 1u) < tau0) continue;
            const unsigned slot = atomicAdd(&S.u[4], 1u);
            if (slot < (unsigned)LMH_RED_COMPACT) { l_val[slot] = vu[u]; l_id[slot] = idu[u]; }
          }
        }
        __syncthreads();
        const unsigned m = S.u[4];
        if (m <= (unsigned)LMH_RED_COMPACT) {
          finish((long long)m, [&](long long j) { return l_val[j]; }, [&](long long j) { return l_id[j]; });
          return;
        }
      }
    }
    finish(ncand, [&](long long j) { return cv(j); }, [&](long long j) { return ci(j); });
    return;
  }

  // ---- mode 3: nucleus over the pooled candidates against the full-vocabulary normalizer ----
  // the bisection steps re-scan every candidate: keep ls and exp(ls - mx) in shared memory when they
  // fit (absent candidates are stored as -inf / 0 and never pass a threshold); then the candidates
  // are read from global memory once
  const bool cached = cache_elems >= ncand;
  float* c_ls = cache;
  float* c_ex = cache + cache_elems;
  float mx = QX_NEG_INF;
  if (cached) {
    constexpr int U = 8;                           // candidates fetched per thread before any is used
    for (long long j0 = tid; j0 < ncand; j0 += (long long)nth * U) {
      int idu[U];
      float vu[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long j = j0 + (long long)u * nth;
        idu[u] = j < ncand ? ci(j) : -1;
        vu[u] = j < ncand ? cv(j) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long j = j0 + (long long)u * nth;
        if (j < ncand) {
          const float ls = idu[u] >= 0 ? vu[u] * invtemp : QX_NEG_INF;
          c_ls[j] = ls;
          mx = fmaxf(mx, ls);
        }
      }
    }
  } else {
    for (long long j = tid; j < ncand; j += nth)
      if (ci(j) >= 0) mx = fmaxf(mx, cv(j) * invtemp);
  }
  mx = block_max(mx, S);
  float Z = 0.f;
  for (long long j = tid; j < nlse; j += nth) {
    const float pl = cand_lse[(j / nlse_s) * lse_stride + (long long)t * nlse_s + (j % nlse_s)];
    if (pl > QX_NEG_INF) Z += expf(pl - mx);
  }
  Z = block_sum(Z, S);
  if (cached) {
    const int n = (int)ncand;
    for (int j = tid; j < n; j += nth) {
      const float ls = c_ls[j];
      c_ex[j] = ls > QX_NEG_INF ? expf(ls - mx) : 0.f;
    }
    __syncthreads();
  }
  float lo = mx - 40.0f, hi = mx;
  for (int it = 0; it < 32; ++it) {
    const float mid = 0.5f * (lo + hi);
    float sm = 0.f;
    if (cached) {
      // Also note whether any candidate lies in each half of [lo, hi): once the half that is kept
      // holds none, further halvings cannot change the set {ls >= lo}, and the search stops.
      unsigned fl = 0u;
      const int n = (int)ncand;
      for (int j = tid; j < n; j += nth) {
        const float ls = c_ls[j];
        if (ls >= mid) { sm += c_ex[j]; fl |= ls < hi ? 2u : 0u; }
        else fl |= ls >= lo ? 1u : 0u;
      }
      block_sum_or(sm, fl, S);
      if (sm / Z >= top_p) { lo = mid; if (!(fl & 2u)) break; }
      else { hi = mid; if (!(fl & 1u)) break; }
      continue;
    } else {
      for (long long j = tid; j < ncand; j += nth) {
        const float ls = cv(j) * invtemp;
        if (ci(j) >= 0 && ls >= mid) sm += expf(ls - mx);
      }
    }
    sm = block_sum(sm, S) / Z;
    if (sm >= top_p) lo = mid; else hi = mid;
  }
  float best = QX_NEG_INF;
  int bid = 0x7fffffff;
  {
    constexpr int U = 8;                           // ids of a batch are fetched together (selected or not)
    for (long long j0 = tid; j0 < ncand; j0 += (long long)nth * U) {
      int idu[U];
      float lsu[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long j = j0 + (long long)u * nth;
        idu[u] = j < ncand ? ci(j) : -1;
        lsu[u] = j < ncand ? (cached ? c_ls[j] : cv(j) * invtemp) : QX_NEG_INF;
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (idu[u] < 0 || lsu[u] < lo) continue;
        const float p = lsu[u] + rng_gumbel(seed, (uint32_t)t, (uint32_t)idu[u]);
        if (better(p, idu[u], best, bid)) { best = p; bid = idu[u]; }
      }
    }
  }
  block_argmax(best, bid, S);
  if (tid == 0) ids[t] = (best == QX_NEG_INF || bid == 0x7fffffff) ? -1 : bid;
}
#undef cv
#undef ci

template <int FMT, typename T>
static void launch_partials_t(cudaStream_t st, const LmHeadArgs& a, float* pv, int32_t* pi,
                              float* pl, int64_t tiles_stride) {
  // the grid covers tiles_stride tiles so that padding tiles of a short shard are written too
  dim3 grid((unsigned)tiles_stride, (unsigned)((a.T + LMH_TB - 1) / LMH_TB));
  lmh_partials_kernel<FMT, T><<<grid, 256, 0, st>>>(
      (const T*)a.h, (const uint8_t*)a.wq, a.bias, pv, pi, pl, (int)a.T, (int)a.V, (int)a.K,
      (long long)a.vocab_offset, (long long)tiles_stride, a.mode, a.topk, a.invtemp, a.seed, a.mask);
  note_launch();
}

template <typename T>
static void launch_partials_f(cudaStream_t st, const LmHeadArgs& a, float* pv, int32_t* pi,
                              float* pl, int64_t ts) {
  switch (a.format) {
    case F_Q4_0: launch_partials_t<F_Q4_0, T>(st, a, pv, pi, pl, ts); break;
    case F_Q8_0: launch_partials_t<F_Q8_0, T>(st, a, pv, pi, pl, ts); break;
    case F_Q6_K: launch_partials_t<F_Q6_K, T>(st, a, pv, pi, pl, ts); break;
    case F_MXFP8: launch_partials_t<F_MXFP8, T>(st, a, pv, pi, pl, ts); break;
    case F_NVFP4: launch_partials_t<F_NVFP4, T>(st, a, pv, pi, pl, ts); break;
    default: launch_partials_t<F_MXFP4, T>(st, a, pv, pi, pl, ts); break;
  }
}

void launch_lm_head_partials(cudaStream_t st, const LmHeadArgs& a, float* part_val,
                             int32_t* part_id, float* part_lse, int64_t tiles_stride) {
  if (launch_lmh_stream_any(st, a, part_val, part_id, part_lse, tiles_stride)) return;
  if (a.dtype == QX_DTYPE_F32) launch_partials_f<float>(st, a, part_val, part_id, part_lse, tiles_stride);
  else if (a.dtype == QX_DTYPE_F16) launch_partials_f<__half>(st, a, part_val, part_id, part_lse, tiles_stride);
  else launch_partials_f<__nv_bfloat16>(st, a, part_val, part_id, part_lse, tiles_stride);
}

void launch_lm_head_reduce(cudaStream_t st, const float* cand_val, const int32_t* cand_id,
                           const float* cand_lse, int shards, int64_t T, int64_t ncand,
                           int64_t nlse, int64_t shard_stride, int mode, int topk, float invtemp,
                           uint32_t seed, float top_p, int32_t* ids, int emit_set, float* out_val,
                           int32_t* out_id) {
  // shard_stride = elements between consecutive shards in all three arrays (0: dense (S,T,C))
  const long long stride_c = shard_stride > 0 ? shard_stride : (long long)T * ncand;
  int cache_elems = 0;
  size_t smem = 0;
  if (mode == 3 && (size_t)ncand * shards * 8 <= 200 * 1024) {
    cache_elems = (int)(ncand * shards);
    smem = (size_t)cache_elems * 8;
  }
  if (mode == 2 && topk > 0 && (ncand * shards) % topk == 0) {
    const long long groups = ncand * shards / topk;             // one group of topk candidates per tile
    if (groups >= topk && groups <= 8192) {
      cache_elems = (int)groups;
      smem = (size_t)groups * 4 + (size_t)LMH_RED_COMPACT * 8;
    }
  }
  if (smem > 48 * 1024) {                                       // once per device
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
      cudaFuncSetAttribute(lmh_reduce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      attr_set[dev] = true;
    }
  }
  const long long stride_l = shard_stride > 0 ? shard_stride : (long long)T * (nlse > 0 ? nlse : 1);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)T);
  cfg.blockDim = dim3(LMH_RED_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const long long ncand_a = (long long)ncand, nlse_a = (long long)(nlse > 0 ? nlse : 1);
  if (cudaLaunchKernelEx(&cfg, lmh_reduce_kernel, cand_val, cand_id, cand_lse, shards, (int)T, ncand_a, nlse_a,
                         (long long)stride_c, (long long)stride_l, cache_elems, mode, topk, invtemp, seed, top_p, ids,
                         emit_set, out_val, out_id) != cudaSuccess) {
    cudaGetLastError();
    lmh_reduce_kernel<<<(unsigned)T, LMH_RED_THREADS, smem, st>>>(
        cand_val, cand_id, cand_lse, shards, (int)T, ncand_a, nlse_a, stride_c, stride_l, cache_elems, mode, topk,
        invtemp, seed, top_p, ids, emit_set, out_val, out_id);
  }
  note_launch();
}

}  // namespace qx
