// Samplers over materialised logits (rows, V): argmax, categorical, top-k, top-p.
//
// One CTA of 1024 threads per row.  Semantics of the reference's unfused kernels
// (kernels/sampling/sampling/sampling.metal:19-103, :159-217): ordering is value descending with
// ties to the smaller index; the noise is the stateless hash keyed by (seed, row, index);
//   argmax       : largest raw logit
//   categorical  : argmax of logit * invtemp + gumbel
//   top-k        : the k largest logits (exact set, found by a radix select on order-preserving
//                  keys instead of k rounds of masked arg-max), then gumbel-max of logit * invtemp
//   top-p        : mx = max(logit * invtemp), Z = sum exp(. - mx); 32 bisection steps on the
//                  threshold L in [mx - 40, mx] keeping the largest L whose kept mass is >= p;
//                  gumbel-max over { logit * invtemp >= L }.  The bisection stops early once the
//                  half that is kept holds no logit (the selected set can no longer change).
#include "qx_block.cuh"
#include "qx_kernels.h"

namespace qx {

template <typename T>
__global__ void __launch_bounds__(1024)
sample_logits_kernel(const T* __restrict__ logits, int32_t* __restrict__ ids, int V, int kind, int topk,
                     float p, float invtemp, uint32_t seed) {
  __shared__ BlockScratch S;
  const int row = blockIdx.x, tid = threadIdx.x, nth = blockDim.x;
  const T* lr = logits + (size_t)row * V;
  float best = QX_NEG_INF;
  int bid = 0x7fffffff;

  if (kind <= 1) {
    for (int i = tid; i < V; i += nth) {
      float v = to_f32<T>(lr[i]);
      if (kind == 1) v = v * invtemp + rng_gumbel(seed, (uint32_t)row, (uint32_t)i);
      if (better(v, i, best, bid)) { best = v; bid = i; }
    }
  } else if (kind == 2) {
    uint32_t tau = 0u;
    int id_cut = 0x7fffffff;
    if (V > topk) {
      unsigned remaining = (unsigned)topk, count_eq = 0;
      block_radix_select(V, [&](long long i, uint32_t& kx) {
        kx = float_key(to_f32<T>(lr[i]));
        return true;
      }, (unsigned)topk, S, tau, remaining, count_eq);
      if (count_eq > remaining) {            // several logits equal the threshold: the smallest indices win
        int cut = -1;
        for (unsigned r = 0; r < remaining; ++r) {
          int mine = 0x7fffffff;
          for (int i = tid; i < V; i += nth)
            if (i > cut && float_key(to_f32<T>(lr[i])) == tau) mine = min(mine, i);
          cut = block_min_int(mine, S);
        }
        id_cut = cut;
      }
    }
    for (int i = tid; i < V; i += nth) {
      const float v = to_f32<T>(lr[i]);
      const uint32_t key = float_key(v);
      if (key > tau || (key == tau && i <= id_cut)) {
        const float s = v * invtemp + rng_gumbel(seed, (uint32_t)row, (uint32_t)i);
        if (better(s, i, best, bid)) { best = s; bid = i; }
      }
    }
  } else {
    float mx = QX_NEG_INF;
    for (int i = tid; i < V; i += nth) mx = fmaxf(mx, to_f32<T>(lr[i]) * invtemp);
    mx = block_max(mx, S);
    float Z = 0.f;
    for (int i = tid; i < V; i += nth) Z += expf(to_f32<T>(lr[i]) * invtemp - mx);
    Z = block_sum(Z, S);
    float lo = mx - 40.0f, hi = mx;
    for (int it = 0; it < 32; ++it) {
      const float mid = 0.5f * (lo + hi);
      float sm = 0.f;
      unsigned fl = 0u;
      for (int i = tid; i < V; i += nth) {
        const float ls = to_f32<T>(lr[i]) * invtemp;
        if (ls >= mid) { sm += expf(ls - mx); fl |= ls < hi ? 2u : 0u; }
        else fl |= ls >= lo ? 1u : 0u;
      }
      block_sum_or(sm, fl, S);
      if (sm / Z >= p) { lo = mid; if (!(fl & 2u)) break; }
      else { hi = mid; if (!(fl & 1u)) break; }
    }
    for (int i = tid; i < V; i += nth) {
      const float ls = to_f32<T>(lr[i]) * invtemp;
      if (ls < lo) continue;
      const float s = ls + rng_gumbel(seed, (uint32_t)row, (uint32_t)i);
      if (better(s, i, best, bid)) { best = s; bid = i; }
    }
  }
  block_argmax(best, bid, S);
  // an empty nucleus cannot happen (the maximum always passes); rows of NaN fall back to index 0
  if (tid == 0) ids[row] = bid == 0x7fffffff ? 0 : bid;
}

void launch_sample_logits(cudaStream_t st, const void* logits, int32_t* ids, int64_t rows, int64_t V,
                          qx_dtype dtype, int kind, int topk, float p, float invtemp, uint32_t seed) {
  if (dtype == QX_DTYPE_F32)
    sample_logits_kernel<float><<<(unsigned)rows, 1024, 0, st>>>((const float*)logits, ids, (int)V, kind, topk, p, invtemp, seed);
  else if (dtype == QX_DTYPE_F16)
    sample_logits_kernel<__half><<<(unsigned)rows, 1024, 0, st>>>((const __half*)logits, ids, (int)V, kind, topk, p, invtemp, seed);
  else
    sample_logits_kernel<__nv_bfloat16><<<(unsigned)rows, 1024, 0, st>>>((const __nv_bfloat16*)logits, ids, (int)V, kind, topk, p, invtemp, seed);
  note_launch();
}

}  // namespace qx
