// decode_linear_epilogue / decode_swiglu for bf16 / f16 activations, batch <= 16: the streaming
// tensor-core path (see qx_stream.cuh for the design).
//
// Two launches per call: prep_activations_kernel turns the activations into row-scaled f16 in the
// decoder's column order (stream-ordered scratch of M*K*2 + M*4 bytes), then gemv_stream_kernel
// streams the weights.  Work split of the main kernel: an m-tile is 16 weight rows (16 gate + 16 up
// rows for SwiGLU); a step is one pipeline stage (KC columns) of one m-tile.  One CTA per SM takes a
// contiguous share of the m-tiles, balanced to within one tile, and its warps cut the flat list of
// the share's (tile, chunk) steps into equal contiguous ranges, each streamed through the warp's
// private ring.  A tile that lies inside one range is finished by that warp.  A tile cut by range
// boundaries is finished after a CTA barrier by the warp that holds its chunk 0, which adds the
// other warps' partial accumulators from shared memory in warp order (deterministic).  Every SM
// therefore streams the same number of bytes whatever N is.

#include "qx_kernels.h"
#include "qx_stream.cuh"
#include "qx_tmap.h"

namespace qx {

// Raised by any kernel of this library whose bounded wait expired; read by qx_cuda_device_error().
static __device__ int g_qx_device_error = 0;

int* device_error_flag() {
  static int* ptr[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_qx_device_error) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    ptr[dev] = (int*)p;
  }
  return ptr[dev];
}

int read_device_error_flag() {
  int v = -1;
  if (cudaMemcpyFromSymbol(&v, g_qx_device_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

// ---- activation preparation ----------------------------------------------------------------------
// Grid (slices, rows).  Every CTA first finds the row's largest finite magnitude by reading the
// whole row (a few KB from L2; cheaper than a second launch or a grid-wide reduction), derives the
// power-of-two scale 2^-S that puts it in [2^14, 2^15), then converts its slice:
// x16[m][perm(c)] = f16(x[m][c] * 2^-S); rowscale[m] = 2^S.
// img_rows > 0 selects the operand-tile image the tcgen05 kernels copy in bulk instead of the plain
// row-major layout: rows are taken in groups of img_rows; a group is stored k-stage by k-stage
// (64 columns = 128 bytes per row), each stage as img_rows consecutive 128-byte rows whose 16-byte
// chunks are XOR-swizzled with the row index (the 128-byte swizzle of a K-major operand tile);
// rows past M are zero.
template <typename T>
__global__ void __launch_bounds__(256)
prep_activations_kernel(const T* __restrict__ x, __half* __restrict__ x16,
                        float* __restrict__ rowscale, int M, int K, int perm, int img_rows) {
  __shared__ float red[8];
  asm volatile("griddepcontrol.launch_dependents;");   // a dependent grid may be scheduled from now on
  const int m = blockIdx.y;
  if (m >= M) {                                     // zero padding row of the last image group
    const int per = (((K + gridDim.x - 1) / gridDim.x) + 31) & ~31;
    const int c0 = blockIdx.x * per, c1 = min(K, c0 + per);
    const int grp = m / img_rows, ml = m % img_rows;
    __half* out = x16 + (size_t)grp * img_rows * K;
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x)
      out[((size_t)(c >> 6) * img_rows + ml) * 64 + ((((c >> 3) & 7) ^ (ml & 7)) << 3) + (c & 7)] = __float2half_rn(0.f);
    return;
  }
  const T* xr = x + (size_t)m * K;
  float amax = 0.f;
  if constexpr (sizeof(T) == 2) {
    const uint4* xv = reinterpret_cast<const uint4*>(xr);          // 8 elements per load (K % 8 == 0)
    const int nv = K / 8;
    auto fold = [&](const uint4& v) {
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float a = fabsf(to_f32<T>(e[j]));
        if (a < 3.0e38f) amax = fmaxf(amax, a);                    // inf / nan do not choose the scale
      }
    };
    int i = threadIdx.x;
    for (; i + 3 * (int)blockDim.x < nv; i += 4 * blockDim.x) {    // four loads in flight per thread
      const uint4 v0 = __ldg(xv + i), v1 = __ldg(xv + i + blockDim.x), v2 = __ldg(xv + i + 2 * blockDim.x),
                  v3 = __ldg(xv + i + 3 * blockDim.x);
      fold(v0); fold(v1); fold(v2); fold(v3);
    }
    for (; i < nv; i += blockDim.x) fold(__ldg(xv + i));
  } else {
    for (int c = threadIdx.x; c < K; c += blockDim.x) {
      const float a = fabsf(to_f32<T>(xr[c]));
      if (a < 3.0e38f) amax = fmaxf(amax, a);
    }
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  int S = 0;
  if (amax > 0.f) {
    S = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 127 - 14;
    S = max(-110, min(110, S));
  }
  const float down = __uint_as_float((uint32_t)(127 - S) << 23);   // 2^-S
  const int per = (((K + gridDim.x - 1) / gridDim.x) + 31) & ~31;  // slice: whole 32-column groups
  const int c0 = blockIdx.x * per, c1 = min(K, c0 + per);
  if (img_rows > 0) {
    const int grp = m / img_rows, ml = m % img_rows;
    __half* out = x16 + (size_t)grp * img_rows * K;
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
      const int pos = (c & ~31) + perm_position(perm, c & 31);
      out[((size_t)(pos >> 6) * img_rows + ml) * 64 + ((((pos >> 3) & 7) ^ (ml & 7)) << 3) + (pos & 7)] =
          __float2half_rn(to_f32<T>(xr[c]) * down);
    }
  } else if (sizeof(T) == 2) {
    __half* out = x16 + (size_t)m * K;                             // slices are whole 32-column groups: 8 per load
    const uint4* xv = reinterpret_cast<const uint4*>(xr);
    for (int i = c0 / 8 + threadIdx.x; i < c1 / 8; i += blockDim.x) {
      const uint4 v = __ldg(xv + i);
      const T* e = reinterpret_cast<const T*>(&v);
      const int c = 8 * i;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        out[(c & ~31) + perm_position(perm, (c & 31) + j)] = __float2half_rn(to_f32<T>(e[j]) * down);
    }
  } else {
    __half* out = x16 + (size_t)m * K;
    for (int c = c0 + threadIdx.x; c < c1; c += blockDim.x) {
      const int pos = (c & ~31) + perm_position(perm, c & 31);
      out[pos] = __float2half_rn(to_f32<T>(xr[c]) * down);
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) rowscale[m] = __uint_as_float((uint32_t)(127 + S) << 23);
}

void launch_prep_activations(cudaStream_t st, const void* x, qx_dtype dtype, __half* x16,
                             float* rowscale, int M, int K, int perm, int img_rows) {
  int slices = (K + 1023) / 1024;
  if (slices > 32) slices = 32;
  const int rows = img_rows > 0 ? (M + img_rows - 1) / img_rows * img_rows : M;
  dim3 grid(slices, rows);
  if (dtype == QX_DTYPE_F16)
    prep_activations_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, x16, rowscale, M, K, perm, img_rows);
  else
    prep_activations_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, x16, rowscale, M, K, perm, img_rows);
}

// Whole stages run fully unrolled in the instantiations with up to this many 8-row n-tiles (0 = never).
#ifndef QX_STREAM_UNROLL
#define QX_STREAM_UNROLL 2
#endif
constexpr int STREAM_STAGES = 2;      // per-warp ring depth; latency is hidden by the number of warps

// HALF = stages of half the format's column count.
//  * single matrix, 1 - 2 rows: full-width stages and 20 warps (102 registers each);
//  * more rows, or a SwiGLU pair: half-width stages.  The prepared activations (2*K bytes per row)
//    are re-read from L1 by every warp; the smaller rings leave the L1 side of the SM's memory large
//    enough to hold them, and a SwiGLU stage of 32 rows fits 16 warps instead of 10.
//    q6_K cannot halve (a stage is one decode group).
template <int FMT, bool DUAL, bool HALF>
struct StreamCfg {
  static_assert(!(HALF && FMT == F_Q6_K), "q6_K stages cannot be halved");
  static constexpr int KC = HALF ? StreamFmt<FMT>::KC / 2 : StreamFmt<FMT>::KC;
  static constexpr int ROWS = DUAL ? 32 : 16;
  using WS = WarpStream<FMT, KC, ROWS, STREAM_STAGES>;
  // shared memory per warp: ring, mbarriers, one partial-sum slot (NACC x 32 f32)
  static constexpr int warp_smem(int nt) { return WS::WARP_BYTES + STREAM_STAGES * 8 + 32 * nt * 4 * (DUAL ? 2 : 1) * 4; }
  static constexpr int warp_cap(int nt) { return (!DUAL && !HALF && nt == 1) ? 20 : 16; }
  // warps per CTA: as many as 220 KB of shared memory hold, at most warp_cap
  static constexpr int max_warps(int nt) {
    return 220 * 1024 / warp_smem(nt) < warp_cap(nt) ? 220 * 1024 / warp_smem(nt) : warp_cap(nt);
  }
};

// XS: batch 1 with the activation row prepared by every CTA itself into shared memory (xsrc = the raw
// 16-bit row, bf16 if x_bf16 else f16; x16 / rowscale unused) instead of by a preparation kernel: one launch less in front of a
// projection whose own run takes 5 - 50 us.  Same arithmetic, same results.
template <int FMT, int NT, bool DUAL, bool HALF, typename T, bool XS>
__global__ void __launch_bounds__(StreamCfg<FMT, DUAL, HALF>::max_warps(NT) * 32, 1)
gemv_stream_kernel(const __grid_constant__ CUtensorMap wmap0, const __grid_constant__ CUtensorMap wmap1,
                   const __half* __restrict__ x16, const float* __restrict__ rowscale, const uint16_t* __restrict__ xsrc, int x_bf16,
                   const T* __restrict__ bias0, const T* __restrict__ bias1,
                   const T* __restrict__ residual, T* __restrict__ y, int M, int K, int N,
                   int activation, int use_bias, int use_residual, uint8_t* __restrict__ mx_blocks,
                   int* __restrict__ err_flag) {
  using Cfg = StreamCfg<FMT, DUAL, HALF>;
  using WS = typename Cfg::WS;
  using F = StreamFmt<FMT>;
  constexpr int NSETS = DUAL ? 2 : 1;
  constexpr int NACC = NSETS * NT * 4;

  extern __shared__ __align__(128) uint8_t smem_raw[];
  asm volatile("griddepcontrol.launch_dependents;");   // a programmatic dependent may be scheduled; it waits for this grid's end
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;

  // shared memory: [per-warp rings][mbarriers][one partial-sum slot per warp (NACC x 32 f32)]
  uint8_t* ring = smem_raw + (size_t)warp * WS::WARP_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)nwarps * WS::WARP_BYTES) + warp * STREAM_STAGES;
  float* slots = reinterpret_cast<float*>(smem_raw + (size_t)nwarps * WS::WARP_BYTES + (size_t)nwarps * STREAM_STAGES * 8);

  WS ws;
  ws.init(smem_u32(ring), smem_u32(bars), &wmap0, &wmap1, 0, K, lane, err_flag);

  // This CTA's m-tiles [T0, T1) and the flat list of their (tile, chunk) steps; this warp's share
  // of the list is [sb, se).
  // With the fused MXFP8 output (mx_blocks) the shares are cut at even tiles, so that every block
  // of 32 output channels is produced by one CTA, which packs it once its tiles are stored.
  const int ntiles = (N + 15) >> 4;
  const int nch = ws.nch;
  const int tunit = mx_blocks ? 2 : 1;
  const int nunits = (ntiles + tunit - 1) / tunit;
  const int T0 = min(ntiles, tunit * (int)((long long)nunits * blockIdx.x / gridDim.x));
  const int T1 = min(ntiles, tunit * (int)((long long)nunits * (blockIdx.x + 1) / gridDim.x));
  const unsigned S = (unsigned)((T1 - T0) * nch);          // the host keeps S * (nwarps + 1) below 2^31
  auto range_begin = [&](int w) { return (int)(S * (unsigned)w / (unsigned)nwarps); };
  const int sb = range_begin(warp), se = range_begin(warp + 1);

  using XP = typename std::conditional<XS, SmemRow, const __half*>::type;
  XP xr[NT];
  // XS: [prepared row: K halves][row scale][32 floats of reduction scratch] behind the partial-sum slots
  uint8_t* xs_base = smem_raw + (((size_t)nwarps * Cfg::warp_smem(NT) + 15) & ~(size_t)15);
  const float* rs_ptr = rowscale;
  if constexpr (XS) {
    rs_ptr = reinterpret_cast<const float*>(xs_base + (size_t)K * 2);
    xr[0] = SmemRow{g == 0 ? smem_u32(xs_base) : 0u};
  } else {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int m = nt * 8 + g;
      xr[nt] = m < M ? x16 + (size_t)m * K : nullptr;
    }
  }

  // (tile, chunk) of the next step to fetch
  int f_tile = T0 + sb / nch, f_c = sb % nch, fetched = sb;
  auto fetch_next = [&](int stage) {
    ws.issue(stage, f_tile * 16, f_c);
    if (++f_c == nch) { f_c = 0; ++f_tile; }
    ++fetched;
  };
#pragma unroll
  for (int p = 0; p < STREAM_STAGES - 1; ++p)
    if (fetched < se) fetch_next(p);
  // Programmatic dependent launch: this grid may start while the activation-preparation kernel is
  // still running (the weight boxes above do not depend on it); everything below reads its output.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if constexpr (XS) {
    static_assert(NT == 1, "in-kernel preparation: one row");
    cta_prepare_row<F::PERM>(xs_base, xsrc, x_bf16, K);
  }

  float acc[NSETS][NT][4];
  auto clear_acc = [&]() {
#pragma unroll
    for (int a = 0; a < NSETS; ++a)
#pragma unroll
      for (int b = 0; b < NT; ++b)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;
  };
  clear_acc();

  // row scale back, bias, activation, residual, one rounding
  auto epilogue = [&](int row0) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int n = row0 + g + (e >> 1) * 8;
        const int m = nt * 8 + 2 * t + (e & 1);
        if (n < N && m < M) {
          const float rs = rs_ptr[m] * GroupProc<FMT>::ACC_SCALE;
          float v = acc[0][nt][e] * rs;
          const size_t o = (size_t)m * N + n;
          if constexpr (DUAL) {
            float up = acc[NSETS - 1][nt][e] * rs;
            if (use_bias) { v += to_f32<T>(bias0[n]); up += to_f32<T>(bias1[n]); }
            y[o] = from_f32<T>(silu(v) * up);
          } else {
            if (use_bias) v += to_f32<T>(bias0[n]);
            v = apply_act(v, activation);
            if (use_residual) v += to_f32<T>(residual[o]);
            y[o] = from_f32<T>(v);
          }
        }
      }
    }
  };

  int tile = T0 + sb / nch, c = sb % nch;
  int seg_c0 = c;            // chunk at which the running partial sum of `tile` started
  int pending_tile = -1;     // tile whose first chunks this warp summed but whose end lies in later warps
  for (int i = sb; i < se; ++i) {
    const int k = i - sb;
    const int stage = k % STREAM_STAGES;
    if (fetched < se) fetch_next((k + STREAM_STAGES - 1) % STREAM_STAGES);
    const bool ready = ws.wait(stage, (uint32_t)((k / STREAM_STAGES) & 1));

    const int col_base = c * Cfg::KC;
    const int ngroups = ready ? min(Cfg::KC, K - col_base) / F::GROUP : 0;
    uint32_t s[2 * NSETS];
    s[0] = ws.slot_addr(stage, g, c);
    s[1] = ws.slot_addr(stage, g + 8, c);
    if constexpr (DUAL) {
      s[2] = ws.slot_addr(stage, 16 + g, c);
      s[3] = ws.slot_addr(stage, 24 + g, c);
    }
    constexpr uint32_t GROUP_BYTES = F::GROUP / F::BK * F::BB;
    using GP = GroupProc<FMT>;
    constexpr bool PRE = NT <= 2;                 // prefetch activations one group ahead
    typename GP::template BFrag<NT> bcur, bnext;
    if (PRE && ngroups > 0) GP::template load_b<NT>(xr, col_base, t, bcur);
    constexpr int FULL = Cfg::KC / F::GROUP;
    if constexpr (NT > 2 && GP::PIPED) {
      uint4 bcar[NT];                             // 32 rows: the fragments of the next unit, fetched one unit ahead
      if (ngroups > 0) GP::template load_first<NT>(xr, col_base, t, bcar);
      for (int gi = 0; gi < ngroups; ++gi) {
        GP::template piped<NSETS, NT, 0>(s, t, xr, col_base + gi * F::GROUP, gi + 1 < ngroups, bcar, acc);
#pragma unroll
        for (int r = 0; r < 2 * NSETS; ++r) s[r] += GROUP_BYTES;
      }
    } else if (QX_STREAM_UNROLL >= NT && ngroups == FULL) {
      // a whole stage (every stage but the last of a ragged K): fully unrolled, so the shared-memory
      // offsets are immediates and the prefetched fragments need no register moves
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
    __syncwarp();

    ++c;
    const bool tile_done = c == nch;
    if (tile_done || i + 1 == se) {
      if (seg_c0 != 0) {
        // the tile began in an earlier warp, which adds this partial sum after the CTA barrier
        float* slot = slots + (size_t)warp * NACC * 32;
        const float* flat = &acc[0][0][0];
#pragma unroll
        for (int q = 0; q < NACC; ++q) slot[q * 32 + lane] = flat[q];
        clear_acc();
      } else if (tile_done) {
        epilogue(tile * 16);
        clear_acc();
      } else {
        pending_tile = tile;
      }
      if (tile_done) { c = 0; ++tile; seg_c0 = 0; }
    }
  }

  // ---- tiles split over several warps: the warp that holds chunk 0 adds the others' partial sums
  //      in warp order (deterministic) and finishes the tile ----
  __syncthreads();
  if (pending_tile >= 0) {
    const int tile_end = (pending_tile - T0 + 1) * nch;
    float* flat = &acc[0][0][0];
    int b2 = se;                                   // first step of the tile held by another warp
    while (b2 < tile_end) {
      // step i belongs to warp floor(((i + 1) * nwarps - 1) / S); warps with empty ranges are skipped
      const int w2 = (int)(((unsigned)(b2 + 1) * (unsigned)nwarps - 1u) / S);
      const float* slot = slots + (size_t)w2 * NACC * 32;
#pragma unroll
      for (int q = 0; q < NACC; ++q) flat[q] += slot[q * 32 + lane];
      b2 = range_begin(w2 + 1);
    }
    epilogue(pending_tile * 16);
  }

  // ---- fused output requantisation: the rounded outputs of this CTA's channels -> MXFP8 blocks ----
  if constexpr (sizeof(T) == 2) {
    if (mx_blocks) {
      __syncthreads();                               // this CTA's stores to y are visible to the CTA
      const int nb0 = T0 >> 1, nb = (T1 >> 1) - nb0;
      const int nblk_row = N >> 5;
      for (int idx = warp; idx < nb * M; idx += nwarps) {
        const int blk = nb0 + idx / M, m = idx - (idx / M) * M;
        const float v = to_f32<T>(y[(size_t)m * N + blk * 32 + lane]);
        mxfp8_block_store(v, lane, mx_blocks + ((size_t)m * nblk_row + blk) * 33);
      }
    }
  }
}

template <int FMT, int NT, bool DUAL, bool HALF, typename T, bool XS>
static bool launch_stream_x(cudaStream_t st, const GemvArgs& a, int nwarps, size_t smem, int blocks, const __half* x16,
                            const float* rowscale, int* err) {
  using Cfg = StreamCfg<FMT, DUAL, HALF>;
  static bool attr_set[64] = {};                    // per instantiation and device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return false;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(gemv_stream_kernel<FMT, NT, DUAL, HALF, T, XS>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    attr_set[dev] = true;
  }
  using WSG = typename Cfg::WS::G;
  const size_t row_bytes = (size_t)(a.K / StreamFmt<FMT>::BK) * StreamFmt<FMT>::BB;
  CUtensorMap map0, map1;
  bool maps_ok = cached_weight_map(&map0, a.w0, a.N, row_bytes, WSG::PITCH, 16);
  if (maps_ok && DUAL) maps_ok = cached_weight_map(&map1, a.w1, a.N, row_bytes, WSG::PITCH, 16);
  if (!DUAL) map1 = map0;
  if (!maps_ok) return false;
  // MXFP8 output rows are packed by the same kernel (needs whole 32-channel blocks)
  uint8_t* mx = (a.out_quant == OQ_MXFP8 && !a.out_f32 && a.N % 32 == 0) ? (uint8_t*)a.q_codes : nullptr;
  // launched as a programmatic dependent of the kernel before it (see griddepcontrol.wait): the
  // preparation kernel, or with XS whatever produced the activations
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3((unsigned)(nwarps * 32));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, gemv_stream_kernel<FMT, NT, DUAL, HALF, T, XS>, map0, map1, x16, rowscale, (const uint16_t*)a.x,
                         (int)(a.dtype == QX_DTYPE_BF16),
                         (const T*)a.bias0, (const T*)a.bias1, (const T*)a.residual, (T*)a.y, (int)a.M, (int)a.K,
                         (int)a.N, a.activation, a.use_bias, a.use_residual, mx, err) != cudaSuccess) {
    cudaGetLastError();
    gemv_stream_kernel<FMT, NT, DUAL, HALF, T, XS><<<blocks, nwarps * 32, smem, st>>>(
        map0, map1, x16, rowscale, (const uint16_t*)a.x, (int)(a.dtype == QX_DTYPE_BF16), (const T*)a.bias0, (const T*)a.bias1, (const T*)a.residual,
        (T*)a.y, (int)a.M, (int)a.K, (int)a.N, a.activation, a.use_bias, a.use_residual, mx, err);
  }
  return true;
}

template <int FMT, int NT, bool DUAL, bool HALF, typename T>
static bool launch_stream_t(cudaStream_t st, const GemvArgs& a) {
  const int sms = sm_count();
  const int ntiles = (int)((a.N + 15) / 16);
  using Cfg = StreamCfg<FMT, DUAL, HALF>;
  int nwarps = Cfg::max_warps(NT);
  // one CTA per SM; a CTA takes a contiguous, balanced share of the m-tiles and its warps split the
  // (tile, chunk) steps of that share evenly
  const int units = (a.out_quant == OQ_MXFP8 && !a.out_f32 && a.N % 32 == 0) ? (ntiles + 1) / 2 : ntiles;
  const int blocks = units < sms ? units : sms;
  const long long nch = (a.K + Cfg::KC - 1) / Cfg::KC;
  if ((long long)((ntiles + blocks - 1) / blocks + 2) * nch * (nwarps + 1) >= (1LL << 31)) return false;
  int* err = device_error_flag();
  if (!err) return false;

  // Batch 1 with a row that fits beside the rings (giving up at most two of the warps): every CTA
  // prepares the row itself, no preparation kernel.
  if constexpr (NT == 1) {
    if (a.M == 1 && ((uintptr_t)a.x & 15) == 0 && a.K % 8 == 0 && (a.dtype == QX_DTYPE_BF16 || a.dtype == QX_DTYPE_F16)) {
      const size_t extra = cta_prepared_row_bytes((size_t)a.K);
      for (int w = nwarps; w >= nwarps - 2 && w >= 8; --w) {
        const size_t smem = (((size_t)w * Cfg::warp_smem(NT) + 15) & ~(size_t)15) + extra;
        if (smem <= 227 * 1024) {
          if (!launch_stream_x<FMT, NT, DUAL, HALF, T, true>(st, a, w, smem, blocks, nullptr, nullptr, err)) return false;
          note_launch(1);
          return true;
        }
      }
    }
  }
  // prepared activations and row scales live in the call's scratch
  const size_t x16_bytes = ((size_t)a.M * a.K * 2 + 255) & ~(size_t)255;
  if (!a.scratch || a.scratch_bytes < x16_bytes + (((size_t)a.M * 4 + 255) & ~(size_t)255)) return false;
  __half* x16 = (__half*)a.scratch;
  float* rowscale = (float*)((char*)a.scratch + x16_bytes);
  const size_t smem = (size_t)nwarps * Cfg::warp_smem(NT);
  launch_prep_activations(st, a.x, a.dtype, x16, rowscale, (int)a.M, (int)a.K, StreamFmt<FMT>::PERM);
  if (!launch_stream_x<FMT, NT, DUAL, HALF, T, false>(st, a, nwarps, smem, blocks, x16, rowscale, err)) return false;
  note_launch(2);
  return true;
}

template <int FMT, typename T>
static bool launch_stream_f(cudaStream_t st, const GemvArgs& a) {
  const bool dual = a.w1 != nullptr;
  constexpr bool H = FMT != F_Q6_K;                 // half-width stages where the format allows
  if (a.M <= 2 && !dual) return launch_stream_t<FMT, 1, false, false, T>(st, a);
  if (a.M <= 8) return dual ? launch_stream_t<FMT, 1, true, H, T>(st, a) : launch_stream_t<FMT, 1, false, H, T>(st, a);
  // 17 - 32 rows of a single matrix in one pass (reached through the pass form below)
  if (a.M > 16 && !dual) return launch_stream_t<FMT, 4, false, H, T>(st, a);
  // 9 - 16 rows, single matrix: full-width stages (the rings of fewer, wider stages keep more bytes in flight)
  return dual ? launch_stream_t<FMT, 2, true, H, T>(st, a) : launch_stream_t<FMT, 2, false, false, T>(st, a);
}

template <int FMT>
static bool stream_shape_ok(const GemvArgs& a) {
  using F = StreamFmt<FMT>;
  const size_t row_bytes = (size_t)(a.K / F::BK) * F::BB;
  // every decode step covers GROUP columns; rows and stages must start on 16-byte boundaries
  // (q6_K stages start on 4-byte boundaries, which its decoder expects)
  return a.K % F::GROUP == 0 && row_bytes % 16 == 0;
}

// Preconditions of the streaming path; anything else takes the generic kernel.
bool stream_path_ok(const GemvArgs& a) {
  if ((a.dtype != QX_DTYPE_BF16 && a.dtype != QX_DTYPE_F16) || a.M > 16 || a.N < 1) return false;
  if (((uintptr_t)a.w0 & 15) != 0 || (a.w1 && ((uintptr_t)a.w1 & 15) != 0)) return false;
  switch (a.format) {
    case F_Q4_0: return stream_shape_ok<F_Q4_0>(a);
    case F_Q8_0: return stream_shape_ok<F_Q8_0>(a);
    case F_Q6_K: return stream_shape_ok<F_Q6_K>(a);
    case F_MXFP8: return stream_shape_ok<F_MXFP8>(a);
    case F_NVFP4: return stream_shape_ok<F_NVFP4>(a);
    default: return stream_shape_ok<F_MXFP4>(a);
  }
}

template <typename T>
static bool launch_stream_dt(cudaStream_t st, const GemvArgs& a) {
  switch (a.format) {
    case F_Q4_0: return launch_stream_f<F_Q4_0, T>(st, a);
    case F_Q8_0: return launch_stream_f<F_Q8_0, T>(st, a);
    case F_Q6_K: return launch_stream_f<F_Q6_K, T>(st, a);
    case F_MXFP8: return launch_stream_f<F_MXFP8, T>(st, a);
    case F_NVFP4: return launch_stream_f<F_NVFP4, T>(st, a);
    default: return launch_stream_f<F_MXFP4, T>(st, a);
  }
}

bool launch_gemv_stream(cudaStream_t st, const GemvArgs& a) {
  if (a.out_f32) return launch_stream_dt<float>(st, a);      // raw fp32 dot products
  if (a.dtype == QX_DTYPE_F16) return launch_stream_dt<__half>(st, a);
  return launch_stream_dt<__nv_bfloat16>(st, a);
}

// Batches of 17 - 64 rows as passes of 32 rows (16 for a SwiGLU pair) through the streaming kernel.  The tcgen05 pipeline
// gives every CTA one item of 256 weight rows; a projection with few such items (O / down / QKV of
// a 70B-class block, any tensor-parallel shard) leaves most SMs idle there (N = 8192: 32 of 148),
// while the streaming kernel spreads any N over all SMs.  Re-reading the weights once per pass is
// cheaper than that as long as the passes are few (option "stream_passes": 0 never, 2 whenever possible).
// rows per pass: 32 for a single matrix, 16 for a SwiGLU pair (twice the accumulators)
static int stream_pass_rows(const GemvArgs& a) { return a.w1 ? 16 : 32; }

bool stream_passes_ok(const GemvArgs& a) {
  const int mode = options().stream_passes;
  // q6_K has no tcgen05 pipeline form, so it takes passes up to 256 rows.
  if (mode == 0 || a.M <= 16 || a.M > (a.format == F_Q6_K ? 256 : 64)) return false;
  GemvArgs b = a;
  b.M = 16;
  if (!stream_path_ok(b)) return false;
  if (mode == 2 || a.format == F_Q6_K) return true;
  // passes win while the pipeline would leave most SMs without an item
  const long long items = (a.N + 255) / 256;          // work items of the tcgen05 pipeline
  const int per = stream_pass_rows(a);
  const int passes = (int)((a.M + per - 1) / per);
  return (passes <= 2 && items <= 96) || items <= 48;
}

size_t stream_scratch_bytes(const GemvArgs& a) {
  int64_t rows = 0;
  if (stream_path_ok(a)) rows = a.M;
  else if (stream_passes_ok(a)) rows = stream_pass_rows(a);
  if (rows == 0) return 0;
  return (((size_t)rows * a.K * 2 + 255) & ~(size_t)255) + (((size_t)rows * 4 + 255) & ~(size_t)255);
}

bool launch_gemv_stream_passes(cudaStream_t st, const GemvArgs& a) {
  const size_t out_size = a.out_f32 ? 4 : 2;
  const int64_t per = stream_pass_rows(a);
  for (int64_t m0 = 0; m0 < a.M; m0 += per) {
    GemvArgs b = a;
    b.M = a.M - m0 < per ? a.M - m0 : per;
    b.x = (const char*)a.x + (size_t)m0 * a.K * 2;
    b.y = (char*)a.y + (size_t)m0 * a.N * out_size;
    if (a.residual) b.residual = (const char*)a.residual + (size_t)m0 * a.N * 2;
    if (a.q_codes && a.out_quant == OQ_MXFP8) b.q_codes = (char*)a.q_codes + (size_t)m0 * (a.N / 32) * 33;
    if (!launch_gemv_stream(st, b)) return false;
  }
  return true;
}

}  // namespace qx
