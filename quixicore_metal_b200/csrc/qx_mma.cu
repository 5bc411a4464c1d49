// decode_linear_epilogue / decode_swiglu for batch > 16: the tcgen05 tensor-core paths.
//
// 1. Every format but q6_K runs on the shared pipeline of qx_tc_pipeline.cuh (2-D TMA boxes of packed
//    weights -> in-kernel dequant to f16 operand tiles -> tcgen05.mma, block scales applied from
//    tensor memory); this file holds its projection epilogues (bias / activation / residual, the
//    SwiGLU gate, raw fp32 partials) and the launch code.
// 2. q6_K (and anything the pipeline's preconditions exclude) keeps the first kernel of this path,
//    gemm_tc_kernel, below.  Shape of the problem: out[n, m] = sum_k W[n, k] * x[m, k] with W
//    packed.  The weight rows are the M-mode of the MMA (128 rows per CTA tile), the batch is the
//    N-mode (16..128), so small batches waste nothing ("swap-AB").  Per 64-column k-stage:
//   * 256 dequant threads (a weight row and 32 columns each) read their packed bytes from global
//     memory one stage ahead, decode them to fp32, split every weight
//     into NTERMS bf16 terms whose sum is exactly the fp32 weight (1 term for nvfp4 / mxfp4 / mxfp8,
//     whose weights are exact in bf16; 2 for q4_0; 3 for q8_0 / q6_K) and store each term as a
//     K-major 128-byte-swizzled operand tile; they also copy the activation tile (bf16, K-major);
//   * one thread issues tcgen05.mma (kind::f16, bf16 x bf16 -> fp32 in TMEM), one MMA chain per
//     term, all accumulating into the same TMEM columns: the result is the fp32 dequantise-then-dot
//     up to summation order, with no rounding of the weights;
//   * the dequant threads read the accumulator back with tcgen05.ld and apply bias / activation /
//     residual, storing 32 consecutive output channels per warp instruction.
// Every wait on an mbarrier is bounded; on expiry the CTA raises the device error flag, stops
// issuing work, frees its tensor memory and returns.
#include "qx_formats.cuh"
#include "qx_kernels.h"
#include "qx_stream.cuh"
#include "qx_tc.cuh"
#include "qx_tc_pipeline.cuh"

namespace qx {

constexpr int MMA_BM = 128;          // weight rows per CTA tile
constexpr int MMA_BK = 64;           // columns per MMA stage (128 bytes of bf16: one swizzle atom)
constexpr int MMA_GROUP_WARPS = 8;    // one dequant group: thread = (weight row, 32-column half) of a stage
constexpr int MMA_GROUPS = 2;         // groups alternate stages, which doubles the loads in flight
constexpr int MMA_DQ_WARPS = MMA_GROUP_WARPS * MMA_GROUPS;
constexpr int MMA_THREADS = (MMA_DQ_WARPS + 1) * 32;   // + the MMA issuer warp

template <int FMT> struct MmaTerms { static constexpr int N = 1; };
template <> struct MmaTerms<F_Q4_0> { static constexpr int N = 2; };
template <> struct MmaTerms<F_Q8_0> { static constexpr int N = 3; };
template <> struct MmaTerms<F_Q6_K> { static constexpr int N = 3; };


template <int FMT> struct MmaGeom {
  static constexpr int NTERMS = MmaTerms<FMT>::N;
  static constexpr int A_STAGES = NTERMS == 1 ? 6 : (NTERMS == 2 ? 4 : 3);   // operand ring depth
  static constexpr int A_STAGE = NTERMS * MMA_BM * 128;
  static constexpr int B_STAGE = 128 * 128;
  static constexpr int OFF_B = A_STAGES * A_STAGE;
  static constexpr int OFF_BAR = OFF_B + A_STAGES * B_STAGE;
  static constexpr int SMEM = OFF_BAR + 256 + 1024;   // + barriers / tmem slot + alignment slack
};

// Barrier slots: [0,8) a_full, [8,16) a_empty, 16 acc_full, 17 acc_empty.
template <int FMT, typename T>
__global__ void __launch_bounds__(MMA_THREADS, 1)
gemm_tc_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ w,
               const T* __restrict__ bias, const T* __restrict__ residual, T* __restrict__ y, int M,
               int K, int N, int BN, int activation, int use_bias, int use_residual,
               int* __restrict__ err_flag) {
  using G = MmaGeom<FMT>;
  constexpr int NTERMS = G::NTERMS;
  constexpr int STAGES = G::A_STAGES;
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const uint32_t bars = sbase + G::OFF_BAR;
  auto BAR = [&](int i) { return bars + 8u * (uint32_t)i; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + G::OFF_BAR + 192);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + G::OFF_BAR + 196);

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(BAR(s), MMA_GROUP_WARPS); mbar_init(BAR(8 + s), 1); }
    mbar_init(BAR(16), 1);
    mbar_init(BAR(17), MMA_DQ_WARPS);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  int tmem_cols = 32;
  while (tmem_cols < BN) tmem_cols <<= 1;
  if (warp == MMA_DQ_WARPS) tmem_alloc(smem_u32((const void*)tmem_slot), (uint32_t)tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const size_t row_bytes = (size_t)(K / block_k_of(FMT)) * block_bytes_of(FMT);
  const int ntiles = (N + MMA_BM - 1) / MMA_BM;
  const int my_tiles = (int)blockIdx.x < ntiles ? (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int nst = K / MMA_BK;                     // MMA stages per tile

  auto wait_or_abort = [&](uint32_t bar, uint32_t parity) -> bool {
    if (*abort_flag) return false;
    for (int i = 0; i < (1 << 19); ++i)
      if (mbar_try_wait(bar, parity)) return true;
    atomicExch(err_flag, 2);
    *abort_flag = 1;
    return false;
  };

  if (warp == MMA_DQ_WARPS) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(BN);
      int it = 0;
      for (int j = 0; j < my_tiles; ++j) {
        if (j > 0 && !wait_or_abort(BAR(17), (uint32_t)((j - 1) & 1))) break;
        tc_fence_after();
        bool ok = true;
        for (int st = 0; st < nst; ++st, ++it) {
          const int sa = it % STAGES;
          if (!wait_or_abort(BAR(sa), (uint32_t)((it / STAGES) & 1))) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = sbase + (uint32_t)(sa * G::A_STAGE);
          const uint32_t b_base = sbase + (uint32_t)(G::OFF_B + sa * G::B_STAGE);
#pragma unroll
          for (int term = 0; term < NTERMS; ++term) {
#pragma unroll
            for (int kk = 0; kk < MMA_BK / 16; ++kk) {
              const uint64_t ad = umma_desc_sw128(a_base + (uint32_t)(term * MMA_BM * 128 + kk * 32));
              const uint64_t bd = umma_desc_sw128(b_base + (uint32_t)(kk * 32));
              tc_mma_f16(tmem_base, ad, bd, idesc, (st | term | kk) != 0 ? 1u : 0u);
            }
          }
          tc_commit(BAR(8 + sa));            // stage reusable once these MMAs have read it
        }
        if (!ok) break;
        tc_commit(BAR(16));                  // accumulator complete
      }
    }
  } else {
    // ------- dequant + epilogue: thread (r, hsp) owns 32 of the 64 stage columns of weight row r -------
    // Weights come straight from global memory (each thread walks its own row: consecutive stages
    // hit the same or the next 32-byte sector, so L1/L2 turn the strided reads into one pass over
    // DRAM); the raw bytes of the next stage are fetched before the current one is decoded.
    const int r = tid & (MMA_BM - 1);
    const int hsp = (tid >> 7) & 1;
    const int grp = tid >> 8;                  // this group handles the stages st with st % MMA_GROUPS == grp
    const int gtid = tid & (MMA_GROUP_WARPS * 32 - 1);
    int it0 = 0;                               // global stage counter at the start of the tile
    for (int j = 0; j < my_tiles; ++j) {
      const int row0 = ((int)blockIdx.x + j * (int)gridDim.x) * MMA_BM;
      const int nrow = min(row0 + r, N - 1);                      // rows past the end re-read the last row
      const uint8_t* wrow = w + (size_t)nrow * row_bytes;
      const uint8_t* wend = w + (size_t)N * row_bytes;            // K % 256 == 0 makes this 8-byte aligned
      RawSpan<FMT> cur, nxt;
      if (grp < nst) cur.load(wrow, grp * 2 + hsp, wend);
      bool ok = true;
      for (int st = grp; st < nst; st += MMA_GROUPS) {
        const int it = it0 + st;
        const int sa = it % STAGES;
        if (st + MMA_GROUPS < nst) nxt.load(wrow, (st + MMA_GROUPS) * 2 + hsp, wend);
        // activation tile: BN rows x 64 columns (rows beyond the batch are zero); issued early
        const int kcol = st * MMA_BK;
        uint4 bv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = gtid + u * MMA_GROUP_WARPS * 32;
          const int m = idx >> 3, cc = idx & 7;
          bv[u] = make_uint4(0u, 0u, 0u, 0u);
          if (idx < BN * 8 && m < M) bv[u] = __ldg(reinterpret_cast<const uint4*>(x + (size_t)m * K + kcol + cc * 8));
        }
        uint32_t pk[NTERMS][16];
        bool direct = false;
        if constexpr (NTERMS == 1) direct = cur.decode_bf16(pk[0]);
        if (!direct) {
          float wv[32];
          cur.decode(wv);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float v0 = wv[2 * i], v1 = wv[2 * i + 1];
#pragma unroll
            for (int term = 0; term < NTERMS; ++term) {
              const __nv_bfloat16 b0 = __float2bfloat16_rn(v0), b1 = __float2bfloat16_rn(v1);
              pk[term][i] = (uint32_t)__bfloat16_as_ushort(b0) | ((uint32_t)__bfloat16_as_ushort(b1) << 16);
              v0 -= __bfloat162float(b0); v1 -= __bfloat162float(b1);
            }
          }
        }
        if (it >= STAGES && !wait_or_abort(BAR(8 + sa), (uint32_t)((it / STAGES - 1) & 1))) { ok = false; break; }
        uint8_t* a_stage = smem + (size_t)sa * G::A_STAGE;
        uint8_t* b_stage = smem + G::OFF_B + (size_t)sa * G::B_STAGE;
#pragma unroll
        for (int term = 0; term < NTERMS; ++term)
#pragma unroll
          for (int cc = 0; cc < 4; ++cc)
            *reinterpret_cast<uint4*>(a_stage + term * MMA_BM * 128 + sw128_offset(r, hsp * 4 + cc)) =
                make_uint4(pk[term][4 * cc], pk[term][4 * cc + 1], pk[term][4 * cc + 2], pk[term][4 * cc + 3]);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int idx = gtid + u * MMA_GROUP_WARPS * 32;
          if (idx < BN * 8) *reinterpret_cast<uint4*>(b_stage + sw128_offset(idx >> 3, idx & 7)) = bv[u];
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR(sa));
        cur = nxt;
      }
      it0 += nst;
      if (!ok) break;
      // ---- epilogue ----
      if (!wait_or_abort(BAR(16), (uint32_t)(j & 1))) break;
      tc_fence_after();
      const int n = row0 + r;
      const float bvv = (use_bias && n < N) ? to_f32<T>(bias[n]) : 0.f;
      // warp w may touch TMEM lanes 32*(w % 4)..+31: the four warps that share a lane quarter
      // take every fourth 16-column chunk each
      for (int cb = warp >> 2; cb < BN / 16; cb += MMA_DQ_WARPS / 4) {
        float v[16];
        tmem_ld16(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(cb * 16), v);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int m = cb * 16 + i;
          if (m < M && n < N) {
            const size_t o = (size_t)m * N + n;
            float val = apply_act(v[i] + bvv, activation);
            if (use_residual) val += to_f32<T>(residual[o]);
            y[o] = from_f32<T>(val);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR(17));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == MMA_DQ_WARPS) tmem_dealloc(tmem_base, (uint32_t)tmem_cols);
}

template <int FMT, typename T>
static bool launch_tc_t(cudaStream_t st, const GemvArgs& a, int* err) {
  using G = MmaGeom<FMT>;
  static_assert(G::SMEM <= 227 * 1024, "tile configuration exceeds shared memory");
  if (cudaFuncSetAttribute(gemm_tc_kernel<FMT, T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           G::SMEM) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  const int ntiles = (int)((a.N + MMA_BM - 1) / MMA_BM);
  const int blocks = ntiles < sm_count() ? ntiles : sm_count();
  for (int64_t m0 = 0; m0 < a.M; m0 += 128) {
    const int mp = (int)((a.M - m0) < 128 ? (a.M - m0) : 128);
    const int BN = (mp + 15) & ~15;
    gemm_tc_kernel<FMT, T><<<blocks, MMA_THREADS, G::SMEM, st>>>(
        (const __nv_bfloat16*)a.x + m0 * a.K, (const uint8_t*)a.w0, (const T*)a.bias0,
        a.residual ? (const T*)a.residual + m0 * a.N : nullptr, (T*)a.y + m0 * a.N, mp, (int)a.K,
        (int)a.N, BN < 32 ? 32 : BN, a.activation, a.use_bias, a.use_residual, err);
    note_launch();
  }
  return true;
}

// ---- projections on the shared tensor-core pipeline (qx_tc_pipeline.cuh) ---------------------------
// Epilogue: thread = one output channel n of the item, CW activation rows; 32 lanes store 32
// consecutive channels of one row.  Linear: y = act(v * rowscale + bias) (+ residual); an item is
// 256 channels.  SwiGLU: half 0 = gate rows, half 1 = up rows of the same 128 channels,
// y = silu(gate) * up.  Raw fp32 dot products when `raw` is set (row-parallel partials).
template <int BN, typename OT, bool DUAL_>
struct ProjEpi {
  struct Args {
    const OT* bias0; const OT* bias1; const OT* residual;
    void* y;
    int N, activation, use_bias, use_residual, raw;
    uint8_t* mx_blocks;     // fused MXFP8 output rows (N % 32 == 0): a warp holds one 32-channel block per row
  };
  static constexpr bool DUAL = DUAL_;
  __device__ __forceinline__ static void run(const Args& a, const TcItem& it) {
    constexpr int CW = BN / 4;
    if (it.warp >= LTC_DQW) return;
    const uint32_t lane_sel = (uint32_t)((it.warp & 3) * 32) << 16;
    const int RS = (it.warp & 3) * 32 + it.lane;
    const int cg = it.warp >> 2;
    if constexpr (DUAL) {
      uint32_t g[CW], u[CW];
      tmem_ld_nowait<CW>(it.tmem_base + lane_sel + (uint32_t)(cg * CW), g);
      tmem_ld_nowait<CW>(it.tmem_base + lane_sel + (uint32_t)(BN + cg * CW), u);
      tmem_wait_ld();
      const int n = it.tile * 128 + RS;
      if (n < a.N) {
        const float gb = a.use_bias ? to_f32<OT>(a.bias0[n]) : 0.f;
        const float ub = a.use_bias ? to_f32<OT>(a.bias1[n]) : 0.f;
#pragma unroll
        for (int i = 0; i < CW; ++i) {
          const int m = cg * CW + i;
          if (m < it.m_count) {
            const float rs = it.rowscale[it.m_base + m];
            const float gv = __uint_as_float(g[i]) * rs + gb, uv = __uint_as_float(u[i]) * rs + ub;
            const OT out = from_f32<OT>(silu(gv) * uv);
            reinterpret_cast<OT*>(a.y)[(size_t)(it.m_base + m) * a.N + n] = out;
            if (a.mx_blocks)
              mxfp8_block_store(to_f32<OT>(out), it.lane,
                                a.mx_blocks + ((size_t)(it.m_base + m) * (a.N >> 5) + (n >> 5)) * 33);
          }
        }
      }
    } else {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t v[CW];
        tmem_ld_nowait<CW>(it.tmem_base + lane_sel + (uint32_t)(h * BN + cg * CW), v);
        tmem_wait_ld();
        const int n = it.tile * 256 + h * 128 + RS;
        if (n < a.N) {
          const float bv = (a.use_bias && !a.raw) ? to_f32<OT>(a.bias0[n]) : 0.f;
#pragma unroll
          for (int i = 0; i < CW; ++i) {
            const int m = cg * CW + i;
            if (m < it.m_count) {
              const size_t o = (size_t)(it.m_base + m) * a.N + n;
              const float dot = __uint_as_float(v[i]) * it.rowscale[it.m_base + m];
              if (a.raw) {
                reinterpret_cast<float*>(a.y)[o] = dot;
              } else {
                float val = apply_act(dot + bv, a.activation);
                if (a.use_residual) val += to_f32<OT>(a.residual[o]);
                const OT out = from_f32<OT>(val);
                reinterpret_cast<OT*>(a.y)[o] = out;
                if (a.mx_blocks)
                  mxfp8_block_store(to_f32<OT>(out), it.lane,
                                    a.mx_blocks + ((size_t)(it.m_base + m) * (a.N >> 5) + (n >> 5)) * 33);
              }
            }
          }
        }
      }
    }
  }
  __device__ __forceinline__ static void tail(const Args&, const float*, int, int, int) {}
};

template <int FMT, int BN, typename OT, bool DUAL>
static bool launch_pipeline_bn(cudaStream_t st, const GemvArgs& a, int* err) {
  using S = TcSmem<FMT, BN>;
  using C = TcCfg<FMT>;
  using Epi = ProjEpi<BN, OT, DUAL>;
  static_assert(S::TOTAL <= 227 * 1024, "tensor-core pipeline configuration exceeds shared memory");
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
  const size_t row_bytes = (size_t)(a.K / StreamFmt<FMT>::BK) * StreamFmt<FMT>::BB;
  CUtensorMap map0, map1;
  if (!cached_weight_map(&map0, a.w0, a.N, row_bytes, C::BOX)) return false;
  if (DUAL) { if (!cached_weight_map(&map1, a.w1, a.N, row_bytes, C::BOX)) return false; }
  else map1 = map0;
  const int groups = (int)((a.M + BN - 1) / BN);
  const size_t img_bytes = ((size_t)groups * BN * a.K * 2 + 255) & ~(size_t)255;
  if (!a.scratch || a.scratch_bytes < img_bytes + (((size_t)a.M * 4 + 255) & ~(size_t)255)) return false;
  __half* ximg = (__half*)a.scratch;
  float* rowscale = (float*)((char*)a.scratch + img_bytes);
  launch_prep_activations(st, a.x, a.dtype, ximg, rowscale, (int)a.M, (int)a.K, StreamFmt<FMT>::PERM, BN);
  note_launch();
  const int item_rows = DUAL ? 128 : 256;
  const long long items = (long long)((a.N + item_rows - 1) / item_rows) * groups;
  const unsigned grid = (unsigned)(items < sm_count() ? items : sm_count());
  const typename Epi::Args ea{(const OT*)a.bias0, (const OT*)a.bias1, (const OT*)a.residual, a.y, (int)a.N,
                              a.activation, a.use_bias, a.use_residual, a.out_f32,
                              (a.out_quant == OQ_MXFP8 && !a.out_f32 && a.N % 32 == 0) ? (uint8_t*)a.q_codes : nullptr};
  tc_pipeline_kernel<FMT, BN, Epi><<<grid, LTC_WARPS * 32, S::TOTAL, st>>>(
      map0, map1, ximg, rowscale, (int)a.M, (int)a.N, (int)a.K, 1, err, ea);
  note_launch();
  return true;
}

template <int FMT, typename OT>
static bool launch_pipeline_fmt(cudaStream_t st, const GemvArgs& a, int* err) {
  if (a.w1) {
    if (a.M <= 32) return launch_pipeline_bn<FMT, 32, OT, true>(st, a, err);
    return launch_pipeline_bn<FMT, 64, OT, true>(st, a, err);
  }
  if (a.M <= 32) return launch_pipeline_bn<FMT, 32, OT, false>(st, a, err);
  return launch_pipeline_bn<FMT, 64, OT, false>(st, a, err);
}

// bf16 / f16 activations, batch > 16, 128-column multiples, 16-byte aligned rows, at least one
// full 128-row box; q6_K stays on the term-split kernel below.
static bool pipeline_ok(const GemvArgs& a) {
  if (a.dtype != QX_DTYPE_BF16 && a.dtype != QX_DTYPE_F16) return false;
  if (a.M <= 16 || a.format == F_Q6_K || a.K % 128 != 0 || a.N < 128) return false;
  const size_t row_bytes = (size_t)(a.K / block_k_of(a.format)) * block_bytes_of(a.format);
  if (row_bytes % 16 != 0 || ((uintptr_t)a.w0 & 15) != 0 || (a.w1 && ((uintptr_t)a.w1 & 15) != 0)) return false;
  return options().tc_pipeline;
}

// Scratch of the tcgen05 paths: the activation image + row scales of the pipeline, or the two fp32
// projections of a SwiGLU pair on the term-split kernel.
size_t tc_scratch_bytes(const GemvArgs& a) {
  if (!tc_path_ok(a)) return 0;
  size_t need = 0;
  if (pipeline_ok(a)) {
    const int BN = a.M <= 32 ? 32 : 64;
    const size_t groups = (size_t)((a.M + BN - 1) / BN);
    need = ((groups * BN * a.K * 2 + 255) & ~(size_t)255) + (((size_t)a.M * 4 + 255) & ~(size_t)255);
  }
  if (a.w1 && a.dtype == QX_DTYPE_BF16 && a.K % 256 == 0) {
    const size_t legacy = 2 * (size_t)a.M * a.N * sizeof(float);
    if (legacy > need) need = legacy;
  }
  return need;
}

template <typename OT>
static bool launch_pipeline(cudaStream_t st, const GemvArgs& a, int* err) {
  switch (a.format) {
    case F_Q4_0: return launch_pipeline_fmt<F_Q4_0, OT>(st, a, err);
    case F_Q8_0: return launch_pipeline_fmt<F_Q8_0, OT>(st, a, err);
    case F_MXFP8: return launch_pipeline_fmt<F_MXFP8, OT>(st, a, err);
    case F_NVFP4: return launch_pipeline_fmt<F_NVFP4, OT>(st, a, err);
    case F_MXFP4: return launch_pipeline_fmt<F_MXFP4, OT>(st, a, err);
    default: return false;
  }
}

// Preconditions of the tcgen05 paths.
bool tc_path_ok(const GemvArgs& a) {
  if (pipeline_ok(a)) return true;
  if (a.dtype != QX_DTYPE_BF16 || a.M <= 16) return false;
  if (a.w1 && (((uintptr_t)a.w1 & 15) != 0)) return false;
  if (a.K % 256 != 0 || ((uintptr_t)a.x & 15) != 0 || ((uintptr_t)a.w0 & 15) != 0) return false;
  return true;
}

template <typename T>
static bool launch_tc_fmt(cudaStream_t st, const GemvArgs& a, int* err) {
  switch (a.format) {
    case F_Q4_0: return launch_tc_t<F_Q4_0, T>(st, a, err);
    case F_Q8_0: return launch_tc_t<F_Q8_0, T>(st, a, err);
    case F_Q6_K: return launch_tc_t<F_Q6_K, T>(st, a, err);
    case F_MXFP8: return launch_tc_t<F_MXFP8, T>(st, a, err);
    case F_NVFP4: return launch_tc_t<F_NVFP4, T>(st, a, err);
    default: return launch_tc_t<F_MXFP4, T>(st, a, err);
  }
}

template <typename T>
__global__ void swiglu_combine_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                      const T* __restrict__ gb, const T* __restrict__ ub,
                                      T* __restrict__ y, long long total, int N, int use_bias) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    float g = gate[i], u = up[i];
    if (use_bias) { const int n = (int)(i % N); g += to_f32<T>(gb[n]); u += to_f32<T>(ub[n]); }
    y[i] = from_f32<T>(silu(g) * u);
  }
}

void launch_swiglu_combine(cudaStream_t st, const float* gate, const float* up, const void* gb,
                           const void* ub, void* y, int64_t M, int64_t N, qx_dtype dtype, int use_bias) {
  const long long total = (long long)M * N;
  const int blocks = (int)((total + 255) / 256 > 4096 ? 4096 : (total + 255) / 256);
  if (dtype == QX_DTYPE_F16)
    swiglu_combine_kernel<__half><<<blocks, 256, 0, st>>>(gate, up, (const __half*)gb, (const __half*)ub, (__half*)y, total, (int)N, use_bias);
  else if (dtype == QX_DTYPE_F32)
    swiglu_combine_kernel<float><<<blocks, 256, 0, st>>>(gate, up, (const float*)gb, (const float*)ub, (float*)y, total, (int)N, use_bias);
  else
    swiglu_combine_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(gate, up, (const __nv_bfloat16*)gb, (const __nv_bfloat16*)ub, (__nv_bfloat16*)y, total, (int)N, use_bias);
  note_launch();
}

bool launch_gemm_tc(cudaStream_t st, const GemvArgs& a, bool* fused_quant) {
  int* err = device_error_flag();
  if (!err) return false;
  if (fused_quant) *fused_quant = false;
  if (pipeline_ok(a)) {
    const bool ok = a.out_f32 ? launch_pipeline<float>(st, a, err)       // OT only types bias / residual, unused here
                  : a.dtype == QX_DTYPE_F16 ? launch_pipeline<__half>(st, a, err)
                                            : launch_pipeline<__nv_bfloat16>(st, a, err);
    if (ok) {
      if (fused_quant) *fused_quant = true;
      return true;
    }
  }
  if (a.dtype != QX_DTYPE_BF16 || a.K % 256 != 0) return false;
  if (a.w1) {
    // SwiGLU at batch > 16: two fp32 projections into stream-ordered scratch, then the gate
    const size_t bytes = (size_t)a.M * a.N * sizeof(float);
    if (!a.scratch || a.scratch_bytes < 2 * bytes) return false;
    float* tmp = (float*)a.scratch;
    GemvArgs g = a;
    g.w1 = nullptr; g.bias0 = nullptr; g.bias1 = nullptr; g.residual = nullptr;
    g.use_bias = 0; g.use_residual = 0; g.activation = 0; g.out_f32 = 1;
    g.y = tmp;
    bool ok = launch_tc_fmt<float>(st, g, err);
    g.w0 = a.w1; g.y = tmp + (size_t)a.M * a.N;
    ok = ok && launch_tc_fmt<float>(st, g, err);
    if (ok) launch_swiglu_combine(st, tmp, tmp + (size_t)a.M * a.N, a.bias0, a.bias1, a.y, a.M, a.N, a.dtype, a.use_bias);
    return ok;
  }
  if (a.out_f32) return launch_tc_fmt<float>(st, a, err);
  using T = __nv_bfloat16;
  switch (a.format) {
    case F_Q4_0: return launch_tc_t<F_Q4_0, T>(st, a, err);
    case F_Q8_0: return launch_tc_t<F_Q8_0, T>(st, a, err);
    case F_Q6_K: return launch_tc_t<F_Q6_K, T>(st, a, err);
    case F_MXFP8: return launch_tc_t<F_MXFP8, T>(st, a, err);
    case F_NVFP4: return launch_tc_t<F_NVFP4, T>(st, a, err);
    default: return launch_tc_t<F_MXFP4, T>(st, a, err);
  }
}

}  // namespace qx
