// Sorted top-k with log-probabilities over LM-head candidates: the second stage of
// lm_head_masked and lm_head_beam_advance, the whole of lm_head_candidates, and the beam selection.
//
// Reference kernels (kernels/quantization/lm_head/lm_head.metal): lm_head_masked_reduce :1264-1304,
// lm_head_beam_reduce :534-573, lm_head_candidates(_q) :1339-1425; beam_select
// (kernels/sampling/sampling/sampling.metal:432-458).  Ordering everywhere: value descending, ties
// to the smaller id.  The reference finds the k winners by k rounds of masked arg-max; here the
// k-th value is found by a radix select on order-preserving keys and the winners are ranked
// against one another, which gives the same list.
#include "qx_block.cuh"
#include "qx_formats.cuh"
#include "qx_kernels.h"

namespace qx {

constexpr int TOPK_THREADS = 256;
constexpr int TOPK_MAX = 64;

// One CTA per row.  Candidates of row r: entries [begin, end) of (val, id) with
//   begin = offsets ? offsets[r] : r * per_row,  end = offsets ? offsets[r + 1] : begin + per_row;
// an entry counts when 0 <= id < V.  Normaliser: the log-sum-exp of the row's tile values
// lse[r * nlse .. + nlse) (entries at -FLT_MAX are absent tiles), or, when lse is null, of the row's
// valid candidate values themselves.  Output (row, k): ids sorted by (value desc, id asc) and
// score = (cum ? cum[r] : 0) + value - normaliser; missing entries are id -1 / -inf.
__global__ void __launch_bounds__(TOPK_THREADS)
lmh_topk_logprob_kernel(const float* __restrict__ val, const int32_t* __restrict__ id,
                        const int32_t* __restrict__ offsets, long long per_row,
                        const float* __restrict__ lse, long long nlse, const float* __restrict__ cum,
                        int V, int topk, int32_t* __restrict__ out_id, float* __restrict__ out_score) {
  __shared__ BlockScratch S;
  __shared__ float sel_val[TOPK_MAX];
  __shared__ int sel_id[TOPK_MAX];
  const int r = blockIdx.x, tid = threadIdx.x, nth = blockDim.x;
  const long long begin = offsets ? (long long)offsets[r] : (long long)r * per_row;
  const long long end = offsets ? (long long)offsets[r + 1] : begin + per_row;
  const long long n = end > begin ? end - begin : 0;
  const float* v = val + begin;
  const int32_t* ids = id + begin;
  auto valid = [&](long long j) { const int i = ids[j]; return i >= 0 && i < V; };

  // ---- normaliser ----
  float mx = QX_NEG_INF;
  if (lse) {
    const float* l = lse + (long long)r * nlse;
    for (long long j = tid; j < nlse; j += nth) mx = fmaxf(mx, l[j]);
    mx = block_max(mx, S);
    float sum = 0.f;
    for (long long j = tid; j < nlse; j += nth)
      if (l[j] > QX_NEG_INF) sum += expf(l[j] - mx);
    sum = block_sum(sum, S);
    mx = sum > 0.f ? mx + logf(sum) : INFINITY;
  } else {
    for (long long j = tid; j < n; j += nth)
      if (valid(j)) mx = fmaxf(mx, v[j]);
    mx = block_max(mx, S);
    float sum = 0.f;
    for (long long j = tid; j < n; j += nth)
      if (valid(j)) sum += expf(v[j] - mx);
    sum = block_sum(sum, S);
    mx = sum > 0.f ? mx + logf(sum) : INFINITY;
  }
  const float norm = mx;

  // ---- the k-th largest key (radix select), ties at the threshold to the smallest ids ----
  unsigned nvalid_l = 0;
  for (long long j = tid; j < n; j += nth) nvalid_l += valid(j) ? 1u : 0u;
  const unsigned nvalid = block_sum_u(nvalid_l, S);
  uint32_t tau = 0u;
  int id_cut = 0x7fffffff;
  if (nvalid > (unsigned)topk) {
    unsigned remaining = (unsigned)topk, count_eq = 0;
    block_radix_select(n, [&](long long j, uint32_t& kx) {
      if (!valid(j)) return false;
      kx = float_key(v[j]);
      return true;
    }, (unsigned)topk, S, tau, remaining, count_eq);
    if (count_eq > remaining) {
      int cut = -1;
      for (unsigned q = 0; q < remaining; ++q) {
        int mine = 0x7fffffff;
        for (long long j = tid; j < n; j += nth)
          if (valid(j) && ids[j] > cut && float_key(v[j]) == tau) mine = min(mine, ids[j]);
        cut = block_min_int(mine, S);
      }
      id_cut = cut;
    }
  }
  // ---- gather the winners, then rank them against one another ----
  if (tid == 0) S.u[3] = 0u;
  __syncthreads();
  for (long long j = tid; j < n; j += nth) {
    if (!valid(j)) continue;
    const uint32_t key = float_key(v[j]);
    if (key > tau || (key == tau && ids[j] <= id_cut)) {
      const unsigned slot = atomicAdd(&S.u[3], 1u);
      if (slot < (unsigned)topk) { sel_val[slot] = v[j]; sel_id[slot] = ids[j]; }
    }
  }
  __syncthreads();
  const int nsel = min((int)S.u[3], topk);
  const float base = cum ? cum[r] : 0.f;
  if (tid < topk) {
    if (tid < nsel) {
      int rank = 0;
      for (int j = 0; j < nsel; ++j) rank += better(sel_val[j], sel_id[j], sel_val[tid], sel_id[tid]) ? 1 : 0;
      out_id[(size_t)r * topk + rank] = sel_id[tid];
      out_score[(size_t)r * topk + rank] = base + sel_val[tid] - norm;
    }
    if (tid >= nsel) {
      out_id[(size_t)r * topk + tid] = -1;
      out_score[(size_t)r * topk + tid] = -INFINITY;
    }
  }
}

void launch_lm_head_topk_logprob(cudaStream_t st, const float* val, const int32_t* id, const int32_t* offsets,
                                 int64_t per_row, const float* lse, int64_t nlse, const float* cum, int64_t rows,
                                 int64_t V, int topk, int32_t* out_id, float* out_score) {
  lmh_topk_logprob_kernel<<<(unsigned)rows, TOPK_THREADS, 0, st>>>(val, id, offsets, (long long)per_row, lse,
                                                                    (long long)nlse, cum, (int)V, topk, out_id, out_score);
  note_launch();
}

// ---- lm_head_candidates: the logit of every listed (row, token) pair ------------------------------
// One warp per CSR entry: lanes stride over 32-column spans of the token's weight row (packed: exact
// fp32 dequantisation; FMT < 0: a dense row in the dtype of h).  Entries with an id outside [0, V)
// get no logit (the top-k stage skips them).
template <int FMT, typename T>
__global__ void __launch_bounds__(256)
lmh_candidate_logits_kernel(const T* __restrict__ h, const uint8_t* __restrict__ w,
                            const float* __restrict__ bias, const int32_t* __restrict__ cand,
                            const int32_t* __restrict__ offsets, float* __restrict__ logit, int rows,
                            int V, int K) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.y;
  const int begin = offsets[t], end = offsets[t + 1];
  const int wpb = blockDim.x >> 5;
  const T* hr = h + (size_t)t * K;
  for (int e = begin + blockIdx.x * wpb + (threadIdx.x >> 5); e < end; e += gridDim.x * wpb) {
    const int v = cand[e];
    if (v < 0 || v >= V) continue;
    float acc = 0.f;
    if constexpr (FMT < 0) {
      const T* row = reinterpret_cast<const T*>(w) + (size_t)v * K;
      for (int c = lane; c < K; c += 32) acc = fmaf(to_f32<T>(row[c]), to_f32<T>(hr[c]), acc);
    } else {
      constexpr int BK = block_k_of(FMT), BB = block_bytes_of(FMT);
      const uint8_t* row = w + (size_t)v * ((size_t)(K / BK) * BB);
      const int spans = (K + 31) / 32;
      for (int s = lane; s < spans; s += 32) {
        float wv[32];
        int ncol = 32;
        if (FMT == F_NVFP4 && s * 32 + 16 >= K) {          // last 16 columns of a row with K = 16 mod 32
          const uint8_t* b = row + (size_t)s * 18;
          const float sc = e4m3_to_f32(b[0]);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            wv[i] = sc * e2m1_to_f32(b[1 + i] & 15u);
            wv[i + 8] = sc * e2m1_to_f32(b[1 + i] >> 4);
            wv[i + 16] = 0.f; wv[i + 24] = 0.f;
          }
          ncol = 16;
        } else {
          decode_span32<FMT>(row, s, wv);
        }
        float a = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < ncol) a = fmaf(to_f32<T>(hr[(size_t)s * 32 + i]), wv[i], a);
        acc += a;
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) logit[e] = bias ? acc + bias[v] : acc;
  }
}

template <typename T>
static void launch_candidate_logits_t(cudaStream_t st, int format, const void* h, const void* w, const float* bias,
                                      const int32_t* cand, const int32_t* offsets, float* logit, int64_t rows,
                                      int64_t V, int64_t K, int64_t entries) {
  const int per_row = (int)((entries + rows - 1) / (rows > 0 ? rows : 1));
  int bx = (per_row + 7) / 8;
  if (bx < 1) bx = 1;
  if (bx > 64) bx = 64;
  dim3 grid((unsigned)bx, (unsigned)rows);
#define QX_CAND(F) lmh_candidate_logits_kernel<F, T><<<grid, 256, 0, st>>>((const T*)h, (const uint8_t*)w, bias, cand, offsets, logit, (int)rows, (int)V, (int)K)
  switch (format) {
    case F_Q4_0: QX_CAND(F_Q4_0); break;
    case F_Q8_0: QX_CAND(F_Q8_0); break;
    case F_Q6_K: QX_CAND(F_Q6_K); break;
    case F_MXFP8: QX_CAND(F_MXFP8); break;
    case F_NVFP4: QX_CAND(F_NVFP4); break;
    case F_MXFP4: QX_CAND(F_MXFP4); break;
    default: QX_CAND(-1); break;
  }
#undef QX_CAND
  note_launch();
}

void launch_lm_head_candidate_logits(cudaStream_t st, int format, qx_dtype dtype, const void* h, const void* w,
                                     const float* bias, const int32_t* cand, const int32_t* offsets, float* logit,
                                     int64_t rows, int64_t V, int64_t K, int64_t entries) {
  if (dtype == QX_DTYPE_F32) launch_candidate_logits_t<float>(st, format, h, w, bias, cand, offsets, logit, rows, V, K, entries);
  else if (dtype == QX_DTYPE_F16) launch_candidate_logits_t<__half>(st, format, h, w, bias, cand, offsets, logit, rows, V, K, entries);
  else launch_candidate_logits_t<__nv_bfloat16>(st, format, h, w, bias, cand, offsets, logit, rows, V, K, entries);
}

// ---- beam selection: per batch the BM best of its BM x 2BM candidates (score desc, flat index asc) ----
__global__ void __launch_bounds__(32)
beam_select_kernel(const float* __restrict__ cand_score, const int32_t* __restrict__ cand_token,
                   int32_t* __restrict__ next_token, int32_t* __restrict__ parent_beam,
                   float* __restrict__ new_cum, int BM, int two_bm) {
  const int b = blockIdx.x, lane = threadIdx.x;
  const int ncand = BM * two_bm;                        // <= 512: at most 16 per lane
  const float* sc = cand_score + (size_t)b * ncand;
  const int32_t* tk = cand_token + (size_t)b * ncand;
  unsigned taken = 0u;                                  // bit i: this lane's i-th candidate was chosen
  for (int k = 0; k < BM; ++k) {
    float best = QX_NEG_INF;
    int bi = 0x7fffffff;
    for (int i = 0, c = lane; c < ncand; ++i, c += 32)
      if (!((taken >> i) & 1u) && better(sc[c], c, best, bi)) { best = sc[c]; bi = c; }
    warp_argmax(best, bi);
    if (bi != 0x7fffffff && (bi & 31) == lane) taken |= 1u << (bi >> 5);
    if (lane == 0) {
      const int o = b * BM + k;
      if (bi == 0x7fffffff) { next_token[o] = -1; parent_beam[o] = 0; new_cum[o] = QX_NEG_INF; }
      else { next_token[o] = tk[bi]; parent_beam[o] = bi / two_bm; new_cum[o] = best; }
    }
  }
}

void launch_beam_select(cudaStream_t st, const float* cand_score, const int32_t* cand_token, int32_t* next_token,
                        int32_t* parent_beam, float* new_cum, int64_t batches, int BM, int two_bm) {
  beam_select_kernel<<<(unsigned)batches, 32, 0, st>>>(cand_score, cand_token, next_token, parent_beam, new_cum, BM, two_bm);
  note_launch();
}

}  // namespace qx
