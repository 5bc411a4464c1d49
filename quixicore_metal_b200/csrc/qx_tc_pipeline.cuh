// Packed-weight projection for 17..64 activation rows per pass on the 5th-generation tensor cores:
// the pipeline shared by LM-head stage 1 (`lm_head_sample`) and by `decode_linear_epilogue` /
// `decode_swiglu` at batch > 16.  What happens to the finished accumulators is an epilogue policy.
//
// Shape: out[n, m] = sum_k W[n, k] * x[m, k].  The weight rows are the M-mode of the MMA (128 rows
// per instruction), the activation rows its N-mode (BN = 32 or 64), f16 x f16 -> fp32 in tensor
// memory.  A CTA owns one work item at a time: two blocks of 128 weight rows ("halves": the two
// halves of a 256-row tile, or the gate and up rows of a SwiGLU tile) for one group of BN
// activation rows, run one after the other, 128 columns (two 128-byte swizzle atoms) per operand
// stage.  Warp roles:
//   * one loader thread.  Per stage it fetches the packed bytes of 128 rows x 128 columns with ONE
//     2-D TMA box copy (tensor map over the weight matrix as rows of 32-bit words; rows past the
//     end of the matrix arrive as zeros) into a ring of raw stages, and the matching activation
//     tile (prepared once per call as row-scaled f16 in the decoders' column order, already in
//     operand-tile layout) with one bulk copy.  A bulk copy costs its issuing thread 60-120
//     cycles whatever its size, so one box per stage instead of one copy per row matters.
//   * 16 worker warps.  Each decodes 8 rows of every stage with the same exact f16 sequences as
//     the small-batch path and stores them, UNSCALED, as a K-major 128-byte-swizzled operand
//     tile (the block scales go to a small ring); then it turns to the accumulators of the
//     PREVIOUS stage (see below), so that a warp always has work while the tensor core runs the
//     stage it has just produced.
//   * the MMA warp (all lanes poll the barriers - the wake-up is faster - lane 0 issues
//     tcgen05.mma).  For the formats whose scale is applied afterwards (q8_0, q4_0, mxfp4, mxfp8)
//     every 32-column unit accumulates into its own TMEM buffer; the buffers are handed over in
//     pairs (one swizzle atom = two units) through a ring of three pairs.  nvfp4 folds its scale
//     into the f16 weight (exact) and accumulates the whole row in place.
//   * the worker warps again, as scale warps (four per TMEM lane quarter, each taking a quarter
//     of the activation rows; a thread owns one weight row): they read the unit buffers back and
//     add scale * partial into fp32 registers: the result is the fp32 dequantise-then-dot up to
//     summation order.  At the end of a half they park the row's sums in TMEM.
// When both halves are done the results of both sit in tensor memory and the epilogue policy runs
// (LM head: through shared memory - the idle operand ring - into the per-tile selection;
// projections: bias / activation / residual or the SwiGLU gate, straight to global memory).
// Every mbarrier wait is bounded; on expiry the CTA raises the device error flag, stops issuing
// work, runs its loops to the end without waiting, frees its tensor memory and returns.
#pragma once

#include "qx_tc.cuh"
#include "qx_tmap.h"

namespace qx {

// Raw-stage geometry.  A stage holds 128 columns of 128 rows.  Its bytes start at a multiple of 4
// inside the row but not of 16, so the box starts at the 16-byte boundary below and is wide
// enough for the largest misalignment; the box width is an odd multiple of 16 bytes, which puts
// the 8 rows a warp instruction touches in different bank groups.
template <int FMT> struct TcCfg {
  using F = StreamFmt<FMT>;
  static constexpr int CHUNK_BYTES = 128 / F::BK * F::BB;
  static constexpr int G16 = (CHUNK_BYTES % 16 == 0) ? 16 : ((CHUNK_BYTES % 8 == 0) ? 8 : 4);
  static constexpr int NEED = CHUNK_BYTES + 16 - G16;
  static constexpr int N16 = (NEED + 15) / 16;
  static constexpr int BOX = (N16 | 1) * 16;                 // odd multiple of 16 bytes
  static constexpr int RAW_STAGE = 128 * BOX;
  static constexpr int RST = RAW_STAGE > 16 * 1024 ? 5 : 6;  // raw ring depth
  static constexpr bool POST = FMT != F_NVFP4;
};

constexpr int LTC_DQW = 16;                      // worker warps (8 rows each; also the scale warps)
constexpr int LTC_WARPS = LTC_DQW + 2;           // + MMA, loader
constexpr int LTC_AST = 2;                       // operand-stage ring depth (weights)
constexpr int LTC_BST = 3;                       // operand-stage ring depth (activations)
constexpr int LTC_DONE = 6;                      // "stage consumed" barrier ring (multiple of AST and BST)
constexpr int LTC_NACC = 3;                      // TMEM ring of unit-buffer pairs
constexpr int LTC_SCR = 16;                      // scale ring depth in units (4 stages)
constexpr int LTC_KS = 128;                      // columns per operand stage (two swizzle atoms)

template <int FMT, int BN>
struct TcSmem {
  using C = TcCfg<FMT>;
  static constexpr int A_ATOM = 128 * 128;
  static constexpr int B_ATOM = BN * 128;
  static constexpr int A_STAGE = 2 * A_ATOM;
  static constexpr int B_STAGE = 2 * B_ATOM;
  static constexpr int OFF_A = 0;                 // also the logit buffer [BN][256] of the selection
  static constexpr int OFF_B = OFF_A + LTC_AST * A_STAGE;
  static constexpr int OFF_RAW = OFF_B + LTC_BST * B_STAGE;
  static constexpr int OFF_SC = OFF_RAW + C::RST * C::RAW_STAGE;
  static constexpr int OFF_BAR = OFF_SC + LTC_SCR * 128 * 4;
  // barriers (8 bytes each): a_full[AST] b_full[BST] done[DONE] acc_full[NACC] acc_empty[NACC]
  // acc_done raw_full[RST] raw_empty[RST], then the TMEM slot and the abort flag
  static constexpr int NBARS = LTC_AST + LTC_BST + LTC_DONE + 2 * LTC_NACC + 1 + 2 * C::RST;
  static constexpr int TOTAL = OFF_BAR + NBARS * 8 + 16 + 1024;     // + alignment slack
  static_assert(BN * 256 * 4 <= LTC_AST * A_STAGE, "a [BN][256] fp32 buffer must fit the operand ring");
  static_assert(C::RAW_STAGE % 128 == 0, "raw stages must keep the TMA destination aligned");
};

// Position in a ring of n barrier slots: slot index and phase parity, advanced without divisions.
struct RingPos {
  int slot;
  uint32_t par;
  __device__ __forceinline__ void advance(int n) {
    if (++slot == n) { slot = 0; par ^= 1u; }
  }
};
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

// What an epilogue policy sees of the finished item.  TMEM columns [0, BN) hold the fp32
// accumulators of half 0, [BN, 2 BN) of half 1 (lane = weight row inside the half, column =
// activation row of the group), still in units of the row-scaled activations.
struct TcItem {
  uint32_t tmem_base;
  float* smem_f32;          // [BN][256] floats of shared memory, free during the epilogue
  const float* rowscale;    // per activation row of the whole call
  int tile, m_base, m_count;
  int warp, lane;
  int kpart, kparts;        // this CTA computed columns [kpart, kpart + 1) * K / kparts of the item
  int split_index;          // which of the shared items this is (0 .. number of shared items - 1)
};

// Epi: struct Args (by-value kernel argument);
//      static constexpr bool DUAL       half 1 reads the second weight matrix at the same rows
//      static void run(args, item)      all warps call it after a CTA barrier; it may use CTA barriers
//      static void tail(args, ...)      after the last item (LM head: absent partials of padding tiles)
template <int FMT, int BN, class Epi>
__global__ void __launch_bounds__(LTC_WARPS * 32, 1)
tc_pipeline_kernel(const __grid_constant__ CUtensorMap wmap0, const __grid_constant__ CUtensorMap wmap1,
                   const __half* __restrict__ ximg, const float* __restrict__ rowscale, int T_total,
                   int V, int K, int ksplit, int* __restrict__ err_flag, const typename Epi::Args ea) {
  using F = StreamFmt<FMT>;
  using C = TcCfg<FMT>;
  using S = TcSmem<FMT, BN>;
  constexpr bool POST = C::POST;
  constexpr int CW = BN / 4;                      // hidden rows per worker warp in its scale role
  constexpr int RST = C::RST;
  extern __shared__ uint8_t smem_dyn[];
  asm volatile("griddepcontrol.launch_dependents;");   // a programmatic dependent may be scheduled; it waits for this grid's end
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const uint32_t bars = sbase + S::OFF_BAR;
  auto A_FULL = [&](int i) { return bars + 8u * (uint32_t)i; };
  auto B_FULL = [&](int i) { return bars + 8u * (uint32_t)(LTC_AST + i); };
  auto DONE = [&](int i) { return bars + 8u * (uint32_t)(LTC_AST + LTC_BST + i); };
  auto ACC_FULL = [&](int i) { return bars + 8u * (uint32_t)(LTC_AST + LTC_BST + LTC_DONE + i); };
  auto ACC_EMPTY = [&](int i) { return bars + 8u * (uint32_t)(LTC_AST + LTC_BST + LTC_DONE + LTC_NACC + i); };
  const uint32_t ACC_DONE = bars + 8u * (uint32_t)(LTC_AST + LTC_BST + LTC_DONE + 2 * LTC_NACC);
  auto RAW_FULL = [&](int i) { return ACC_DONE + 8u * (uint32_t)(1 + i); };
  auto RAW_EMPTY = [&](int i) { return ACC_DONE + 8u * (uint32_t)(1 + RST + i); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + S::OFF_BAR + S::NBARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + S::OFF_BAR + S::NBARS * 8 + 4);
  float* sc_ring = reinterpret_cast<float*>(smem + S::OFF_SC);
  float* logit = reinterpret_cast<float*>(smem + S::OFF_A);

  if (tid == 0) {
    for (int s = 0; s < LTC_AST; ++s) mbar_init(A_FULL(s), LTC_DQW);
    for (int s = 0; s < LTC_BST; ++s) mbar_init(B_FULL(s), 1);
    for (int s = 0; s < LTC_DONE; ++s) mbar_init(DONE(s), 1);
    for (int s = 0; s < LTC_NACC; ++s) { mbar_init(ACC_FULL(s), 1); mbar_init(ACC_EMPTY(s), LTC_DQW); }
    mbar_init(ACC_DONE, 1);
    for (int s = 0; s < RST; ++s) { mbar_init(RAW_FULL(s), 1); mbar_init(RAW_EMPTY(s), LTC_DQW); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == LTC_DQW) tmem_alloc(smem_u32((const void*)tmem_slot), 512u);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: [0, BN) results of half 0, [BN, 2 BN) of half 1, then NACC pairs of unit buffers
  constexpr uint32_t ACC_COL0 = 2 * BN;

  // Bounded wait.  The CTA-wide abort flag is looked at only while spinning.
  auto wait_or_abort = [&](uint32_t bar, uint32_t parity) -> bool {
    if (mbar_try_wait(bar, parity)) return true;              // the common case: already complete
    for (int i = 0; i < (1 << 21); ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      if ((i & 63) == 63 && *abort_flag) return false;
    }
    atomicExch(err_flag, 3);
    *abort_flag = 1;
    return false;
  };

  const int groups = (T_total + BN - 1) / BN;                 // hidden-row groups (work items)
  constexpr int ITEM_ROWS = Epi::DUAL ? 128 : 256;            // weight rows per work item
  const int real_tiles = (V + ITEM_ROWS - 1) / ITEM_ROWS;
  const int items = real_tiles * groups;
  const int nks = K / LTC_KS;                                 // operand stages per half
  // Items are dealt round-robin.  The items of the last, partial round can be shared: with
  // ksplit > 1 (the host guarantees leftover * ksplit <= grid and ksplit | nks) each of them is
  // given to ksplit CTAs that take K / ksplit columns each, and the epilogue adds the parts.
  const int full_rounds = items / (int)gridDim.x;
  const int leftover = items - full_rounds * (int)gridDim.x;
  const bool has_tail = (int)blockIdx.x < leftover * ksplit;
  const int my_items = full_rounds + (has_tail ? 1 : 0);
  const int tail_nks = nks / ksplit, tail_st0 = ((int)blockIdx.x % ksplit) * tail_nks;
  const int total_stages = 2 * (full_rounds * nks + (has_tail ? tail_nks : 0));   // stage counter range of this CTA
  auto item_of = [&](int j) {
    return j < full_rounds ? (int)blockIdx.x + j * (int)gridDim.x : full_rounds * (int)gridDim.x + (int)blockIdx.x / ksplit;
  };
  // Ring positions of each role, carried across items (a stage's global index only ever grows by one).
  int raw_next = 0, raw_j = 0, raw_h = 0, raw_st = 0;         // loader: next raw stage and where it lies
  int raw_row0 = -1;                                          // loader: first weight row of (raw_j, raw_h); -1 = not computed
  RingPos ld_raw{0, 0}, ld_b{0, 0}, ld_bdone{0, 0};           // loader: raw slot, activation slot, DONE(stage - BST)
  RingPos wk_raw{0, 0}, wk_done{0, 0}, wk_acc{0, 0};          // workers: raw slot, DONE(stage - AST), accumulator pair
  RingPos mm_b{0, 0}, mm_acc{0, 0}, mm_done{0, 0};            // MMA warp: activation slot, accumulator pair, DONE slot
  int g_it = 0;                                               // stages this role has gone through so far
  int g_pairs = 0;                                            // MMA warp: accumulator pairs issued so far

  for (int j = 0; j < my_items; ++j) {
    const int item = item_of(j);
    const int tile = item / groups;
    const int grp = item % groups;
    const int t_base = grp * BN;
    const int T_pass = min(BN, T_total - t_base);
    const int it_base = j * 2 * nks;                          // global operand-stage counter (a shared item is the last)
    const bool shared_item = j >= full_rounds && ksplit > 1;
    const int nks_i = shared_item ? tail_nks : nks;           // stages per half of this item, first column stage
    const int st0 = shared_item ? tail_st0 : 0;

    if (warp < LTC_DQW) {
      // ================= workers: decode stage `it`, then scale the accumulators of stage `it - 1` =================
      const int q = ((lane >> 2) & 1) * 4 + (lane >> 3);      // this thread's row of the warp's 8
      const int t = lane & 3;
      const int R = warp * 8 + q;                             // row inside the 128-row half (decode role)
      constexpr uint32_t ATOM_BYTES = 64 / F::BK * F::BB;     // packed bytes of 64 columns
      const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
      const int RS = (warp & 3) * 32 + lane;                  // row inside the half (scale role)
      const int cg = warp >> 2;                               // which quarter of the hidden rows
      float2 acc2[CW / 2];                                    // sums of (hidden row 2i, 2i + 1) for this thread's weight row
      const uint32_t sc_rd = sbase + (uint32_t)(S::OFF_SC + RS * 4);     // scale ring, this thread's row (scale role)
      auto scale_stage = [&](int it) {                          // both unit pairs of stage `it`, in ring order
        const int buf0 = wk_acc.slot;
        bool ok = wait_or_abort(ACC_FULL(buf0), wk_acc.par);
        wk_acc.advance(LTC_NACC);
        const int buf1 = wk_acc.slot;
        ok = wait_or_abort(ACC_FULL(buf1), wk_acc.par) && ok;
        wk_acc.advance(LTC_NACC);
        tc_fence_after();
        const uint32_t col = tmem_base + lane_sel + ACC_COL0 + (uint32_t)(cg * CW);
        const uint32_t scs = sc_rd + (uint32_t)(((it * 4) & (LTC_SCR - 1)) * 512);
        const float sc0 = lds_f32(scs), sc1 = lds_f32(scs + 512), sc2 = lds_f32(scs + 1024), sc3 = lds_f32(scs + 1536);
        if (ok) {
          uint32_t v0[CW], v1[CW], v2[CW], v3[CW];
          tmem_ld_nowait<CW>(col + (uint32_t)(buf0 * 2 * BN), v0);
          tmem_ld_nowait<CW>(col + (uint32_t)(buf0 * 2 * BN + BN), v1);
          tmem_ld_nowait<CW>(col + (uint32_t)(buf1 * 2 * BN), v2);
          tmem_ld_nowait<CW>(col + (uint32_t)(buf1 * 2 * BN + BN), v3);
          tmem_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) { mbar_arrive(ACC_EMPTY(buf0)); mbar_arrive(ACC_EMPTY(buf1)); }
          // two hidden rows per instruction (packed fp32 fma: each half is an ordinary fmaf)
          const float2 s0 = make_float2(sc0, sc0), s1 = make_float2(sc1, sc1), s2 = make_float2(sc2, sc2),
                       s3 = make_float2(sc3, sc3);
#pragma unroll
          for (int i = 0; i < CW / 2; ++i) {
            float2 a = acc2[i];
            a = __ffma2_rn(s0, make_float2(__uint_as_float(v0[2 * i]), __uint_as_float(v0[2 * i + 1])), a);
            a = __ffma2_rn(s1, make_float2(__uint_as_float(v1[2 * i]), __uint_as_float(v1[2 * i + 1])), a);
            a = __ffma2_rn(s2, make_float2(__uint_as_float(v2[2 * i]), __uint_as_float(v2[2 * i + 1])), a);
            a = __ffma2_rn(s3, make_float2(__uint_as_float(v3[2 * i]), __uint_as_float(v3[2 * i + 1])), a);
            acc2[i] = a;
          }
        } else {
          __syncwarp();
          if (lane == 0) { mbar_arrive(ACC_EMPTY(buf0)); mbar_arrive(ACC_EMPTY(buf1)); }
        }
      };
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int i = 0; i < CW / 2; ++i) acc2[i] = make_float2(0.f, 0.f);
        for (int st = 0; st < nks_i; ++st) {
          const int it = g_it;
          const int sa = it & (LTC_AST - 1), sr = wk_raw.slot;
          const uint32_t off = (uint32_t)((st0 + st) * C::CHUNK_BYTES) & 15u;
          const uint32_t sp0 = sbase + (uint32_t)(S::OFF_RAW + sr * C::RAW_STAGE) + off + (uint32_t)(R * C::BOX);
          wait_or_abort(RAW_FULL(sr), wk_raw.par);
          wk_raw.advance(RST);
          // The operand slot is free once the MMAs of stage it - 2 have completed.  The post-scaled
          // formats have seen that already: scale_stage(it - 2), which precedes this point, waited for
          // the accumulators those MMAs produced.  nvfp4 accumulates in place and asks the barrier.
          if constexpr (!POST) {
            if (it >= LTC_AST) { wait_or_abort(DONE(wk_done.slot), wk_done.par); wk_done.advance(LTC_DONE); }
          }
          const uint32_t a_stage = sbase + (uint32_t)(S::OFF_A + sa * S::A_STAGE);
          if constexpr (FMT == F_NVFP4) {
#pragma unroll
            for (int a = 0; a < 2; ++a) {                     // swizzle atom = 64 columns
              const uint32_t a_atom = a_stage + (uint32_t)(a * S::A_ATOM);
              uint32_t w[4][2];
              GroupProc<F_NVFP4>::block(sp0 + a * ATOM_BYTES, t, w);
              sts128(a_atom + sw128_offset(R, 2 * t), w[0][0], w[0][1], w[1][0], w[1][1]);
              sts128(a_atom + sw128_offset(R, 2 * t + 1), w[2][0], w[2][1], w[3][0], w[3][1]);
            }
          } else {
            // all shared-memory loads of the stage first (four units), then the conversions and stores
            using RD = RowDec<FMT>;
            constexpr bool WIDE = F::GROUP == 128;            // the unit's position inside the decode
            uint32_t raw[4][RD::RAWN], scb[4];                // group fixes its byte alignment
            RD::template load<0>(sp0, t, raw[0], scb[0]);
            RD::template load<1>(sp0 + F::BB, t, raw[1], scb[1]);
            if constexpr (WIDE) {
              RD::template load<2>(sp0 + 2 * F::BB, t, raw[2], scb[2]);
              RD::template load<3>(sp0 + 3 * F::BB, t, raw[3], scb[3]);
            } else {
              RD::template load<0>(sp0 + 2 * F::BB, t, raw[2], scb[2]);
              RD::template load<1>(sp0 + 3 * F::BB, t, raw[3], scb[3]);
            }
            const uint32_t scs = sbase + (uint32_t)(S::OFF_SC + ((it * 4) & (LTC_SCR - 1)) * 512 + R * 4);
#pragma unroll
            for (int u4 = 0; u4 < 4; ++u4) {                  // unit u4: atom u4 / 2, chunk group u4 % 2
              uint32_t w[2][2];
              RD::convert(raw[u4], w);
              sts128(a_stage + (uint32_t)((u4 >> 1) * S::A_ATOM) + sw128_offset(R, 4 * (u4 & 1) + t),
                     w[0][0], w[0][1], w[1][0], w[1][1]);
              if (t == 0) sts_f32(scs + (uint32_t)(u4 * 512), RD::scale(scb[u4]));
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) { mbar_arrive(A_FULL(sa)); mbar_arrive(RAW_EMPTY(sr)); }
          ++g_it;
          if constexpr (POST) { if (st > 0) scale_stage(it - 1); }
        }
        if constexpr (POST) {
          scale_stage(g_it - 1);
          // park the row's sums of this half
          uint32_t v[CW];
#pragma unroll
          for (int i = 0; i < CW / 2; ++i) { v[2 * i] = __float_as_uint(acc2[i].x); v[2 * i + 1] = __float_as_uint(acc2[i].y); }
          tmem_st<CW>(tmem_base + lane_sel + (uint32_t)(h * BN + cg * CW), v);
          tmem_wait_st();
        }
      }
      if constexpr (!POST) {
        wait_or_abort(ACC_DONE, (uint32_t)(j & 1));
        tc_fence_after();
      }
    } else if (warp == LTC_DQW) {
      // ================= MMA issuer (the whole warp polls: the wake-up is faster; lane 0 issues) =================
      const uint32_t idesc = umma_idesc_f16(BN);
      const uint64_t desc0 = umma_desc_sw128(sbase);          // the shared window starts 1024-byte aligned: adding
      for (int h = 0; h < 2; ++h) {                           // offsets below 256 KB never carries out of the field
        for (int st = 0; st < nks_i; ++st) {
          const int it = g_it++;
          const int sa = it & (LTC_AST - 1), sb = mm_b.slot;
          bool ok = wait_or_abort(B_FULL(sb), mm_b.par);
          mm_b.advance(LTC_BST);
          ok = wait_or_abort(A_FULL(sa), (uint32_t)((it >> 1) & 1)) && ok;
          tc_fence_after();
          // descriptors of this stage: only the address field (low word, 16-byte units) varies
          const uint64_t a_desc = desc0 + (uint64_t)((uint32_t)(S::OFF_A + sa * S::A_STAGE) >> 4);
          const uint64_t b_desc = desc0 + (uint64_t)((uint32_t)(S::OFF_B + sb * S::B_STAGE) >> 4);
#pragma unroll
          for (int p = 0; p < 2; ++p) {                       // swizzle atom = pair of units
            if constexpr (POST) {
              const int buf = mm_acc.slot;
              if (g_pairs >= LTC_NACC) {
                ok = wait_or_abort(ACC_EMPTY(buf), mm_acc.par ^ 1u) && ok;
                tc_fence_after();
              }
              mm_acc.advance(LTC_NACC);
              ++g_pairs;
              if (lane == 0) {
                if (ok) {
#pragma unroll
                  for (int kk = 0; kk < 4; ++kk)
                    tc_mma_f16(tmem_base + ACC_COL0 + (uint32_t)(buf * 2 * BN + (kk >> 1) * BN),
                               a_desc + (uint64_t)((p * S::A_ATOM + kk * 32) >> 4),
                               b_desc + (uint64_t)((p * S::B_ATOM + kk * 32) >> 4), idesc, kk & 1);
                }
                tc_commit(ACC_FULL(buf));
              }
            } else {
              if (lane == 0 && ok) {
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                  tc_mma_f16(tmem_base + (uint32_t)(h * BN),
                             a_desc + (uint64_t)((p * S::A_ATOM + kk * 32) >> 4),
                             b_desc + (uint64_t)((p * S::B_ATOM + kk * 32) >> 4), idesc,
                             (st | p | kk) != 0 ? 1u : 0u);
              }
            }
          }
          if (lane == 0) tc_commit(DONE(mm_done.slot));
          mm_done.advance(LTC_DONE);
          __syncwarp();
        }
      }
      if constexpr (!POST) { if (lane == 0) tc_commit(ACC_DONE); }
      __syncwarp();
    } else if (warp == LTC_DQW + 1) {
      // ================= loader: raw weight boxes (may run ahead into the next item) + activation tiles =================
      if (lane == 0) {
        const uint8_t* src = reinterpret_cast<const uint8_t*>(ximg) + (size_t)grp * BN * K * 2;
        int nb = it_base, b_st = 0;                             // next activation stage to request (b_st: inside the half)
        const int nb_end = it_base + 2 * nks_i;
        const int raw_need = min(total_stages, nb_end);          // every raw stage of this item must be requested here
        int idle = 0;
        while ((nb < nb_end || raw_next < raw_need) && idle < (1 << 22)) {
          bool progressed = false;
          if (raw_next < total_stages &&
              (raw_next < RST || mbar_try_wait(RAW_EMPTY(ld_raw.slot), ld_raw.par ^ 1u))) {
            // raw stage raw_next = (item raw_j, half raw_h, stage raw_st)
            const bool raw_shared = raw_j >= full_rounds && ksplit > 1;
            const int raw_nks = raw_shared ? tail_nks : nks, raw_st0 = raw_shared ? tail_st0 : 0;
            if (raw_row0 < 0) raw_row0 = (item_of(raw_j) / groups) * ITEM_ROWS + (Epi::DUAL ? 0 : raw_h * 128);
            const int row0 = raw_row0;
            const int sr = ld_raw.slot;
            mbar_arrive_expect_tx(RAW_FULL(sr), (uint32_t)C::RAW_STAGE);
            tma_box_2d(sbase + (uint32_t)(S::OFF_RAW + sr * C::RAW_STAGE), (Epi::DUAL && raw_h) ? &wmap1 : &wmap0,
                       (int)(((uint32_t)((raw_st0 + raw_st) * C::CHUNK_BYTES) & ~15u) >> 2), row0, RAW_FULL(sr));
            ld_raw.advance(RST);
            ++raw_next;
            if (++raw_st == raw_nks) { raw_st = 0; raw_row0 = -1; if (++raw_h == 2) { raw_h = 0; ++raw_j; } }
            progressed = true;
          }
          if (nb < nb_end && (nb < LTC_BST || mbar_try_wait(DONE(ld_bdone.slot), ld_bdone.par))) {
            if (nb >= LTC_BST) ld_bdone.advance(LTC_DONE);
            const int sb = ld_b.slot;
            mbar_arrive_expect_tx(B_FULL(sb), (uint32_t)S::B_STAGE);
            bulk_g2s(sbase + (uint32_t)(S::OFF_B + sb * S::B_STAGE), src + (size_t)(st0 + b_st) * S::B_STAGE,
                     (uint32_t)S::B_STAGE, B_FULL(sb));
            ld_b.advance(LTC_BST);
            if (++b_st == nks_i) b_st = 0;
            ++nb;
            progressed = true;
          }
          if (progressed) idle = 0;
          else if (((++idle) & 63) == 0 && *abort_flag) break;
        }
        if ((nb < nb_end || raw_next < raw_need) && !*abort_flag) { atomicExch(err_flag, 3); *abort_flag = 1; }
      }
      __syncwarp();
    }

    // ---- the results of both halves are in TMEM columns [0, 2 BN); the operand ring is idle ----
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    {
      TcItem item_ctx{tmem_base, logit, rowscale, tile, t_base, T_pass, warp, lane,
                      shared_item ? (int)blockIdx.x % ksplit : 0, shared_item ? ksplit : 1,
                      shared_item ? (int)blockIdx.x / ksplit : 0};
      Epi::run(ea, item_ctx);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }

  // on an aborted run, raw boxes that were requested but never consumed may still be in flight
  if (warp == LTC_DQW + 1 && lane == 0 && *abort_flag) {
    for (int i = max(0, raw_next - RST); i < raw_next; ++i)
      for (int k = 0; k < (1 << 20); ++k)
        if (mbar_try_wait(RAW_FULL(i % RST), (uint32_t)((i / RST) & 1))) break;   // cold path: divisions are fine
  }

  Epi::tail(ea, logit, real_tiles, warp, lane);

  tc_fence_before();
  __syncthreads();
  if (warp == LTC_DQW) tmem_dealloc(tmem_base, 512u);
}

}  // namespace qx
