// decode_linear_epilogue / decode_swiglu for bf16 / f16 activations, batch <= 16: the streaming
// tensor-core path (see qx_stream.cuh for the design).
//
// Two launches per call: prep_activations_kernel turns the activations into row-scaled f16 in the
// decoder's column order (stream-ordered scratch of M*K*2 + M*4 bytes), then gemv_stream_kernel
// streams the weights.  Work split of the main kernel: an m-tile is 16 weight rows (16 gate + 16 up
// rows for SwiGLU).  A CTA is GROUPS x KS warps; the KS warps of a group share one m-tile and each
// streams its own slice of K through its private ring, then the group adds the KS partial
// accumulators in a fixed order (deterministic) and warp 0 of the group applies the row scale,
// bias / activation / residual and stores.  KS > 1 keeps every SM busy when there are few rows.
#include <cstdlib>
#include <mutex>

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
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
      const uint4 v = __ldg(xv + i);
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float a = fabsf(to_f32<T>(e[j]));
        if (a < 3.0e38f) amax = fmaxf(amax, a);                    // inf / nan do not choose the scale
      }
    }
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
  int slices = (K + 2047) / 2048;
  if (slices > 16) slices = 16;
  const int rows = img_rows > 0 ? (M + img_rows - 1) / img_rows * img_rows : M;
  dim3 grid(slices, rows);
  if (dtype == QX_DTYPE_F16)
    prep_activations_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, x16, rowscale, M, K, perm, img_rows);
  else
    prep_activations_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, x16, rowscale, M, K, perm, img_rows);
}

// ---- scratch for the prepared activations -----------------------------------------------------------
// Calls on one stream are ordered, so a buffer tied to (device, stream) can be reused by every call
// on that stream without synchronisation.  Up to 16 streams get such a buffer (grown on demand,
// kept until process exit); further streams fall back to stream-ordered allocation per call.
struct ScratchSlot { int dev; cudaStream_t st; void* ptr; size_t bytes; };
static ScratchSlot g_scratch[16] = {};
static std::mutex g_scratch_mu;

void* stream_scratch(cudaStream_t st, size_t bytes, bool* must_free) {
  *must_free = false;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  cudaStreamIsCapturing(st, &cap);
  if (cap == cudaStreamCaptureStatusNone) {
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    ScratchSlot* free_slot = nullptr;
    for (auto& s : g_scratch) {
      if (s.ptr && s.dev == dev && s.st == st) {
        if (s.bytes >= bytes) return s.ptr;
        // grow (rare): earlier work of this stream may still read the old buffer
        cudaStreamSynchronize(st);
        cudaFree(s.ptr);
        s.ptr = nullptr;
        free_slot = &s;
        break;
      }
      if (!s.ptr && !free_slot) free_slot = &s;
    }
    if (free_slot) {
      void* p = nullptr;
      const size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
      if (cudaMalloc(&p, want) == cudaSuccess) {
        *free_slot = ScratchSlot{dev, st, p, want};
        return p;
      }
      cudaGetLastError();
    }
  }
  void* p = nullptr;
  if (cudaMallocAsync(&p, bytes, st) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  *must_free = true;
  return p;
}

constexpr int STREAM_STAGES = 2;      // per-warp ring depth; latency is hidden by the number of warps
constexpr int STREAM_MAX_WARPS = 16;

template <int FMT, bool DUAL>
struct StreamCfg {
  static constexpr int KC = StreamFmt<FMT>::KC;
  static constexpr int ROWS = DUAL ? 32 : 16;
  using WS = WarpStream<FMT, KC, ROWS, STREAM_STAGES>;
};

template <int FMT, int NT, bool DUAL, typename T>
__global__ void __launch_bounds__(STREAM_MAX_WARPS * 32, 1)
gemv_stream_kernel(const __grid_constant__ CUtensorMap wmap0, const __grid_constant__ CUtensorMap wmap1,
                   const __half* __restrict__ x16, const float* __restrict__ rowscale,
                   const T* __restrict__ bias0, const T* __restrict__ bias1,
                   const T* __restrict__ residual, T* __restrict__ y, int M, int K, int N,
                   int activation, int use_bias, int use_residual, int ks_log2,
                   int* __restrict__ err_flag) {
  using Cfg = StreamCfg<FMT, DUAL>;
  using WS = typename Cfg::WS;
  using F = StreamFmt<FMT>;
  constexpr int NSETS = DUAL ? 2 : 1;
  constexpr int NACC = NSETS * NT * 4;

  extern __shared__ __align__(128) uint8_t smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int KS = 1 << ks_log2;
  const int groups = nwarps >> ks_log2;                 // host guarantees KS divides nwarps
  const int group = warp >> ks_log2, ks = warp & (KS - 1);

  // shared memory: [per-warp rings][mbarriers][per-group reduction buffers (2 x KS x 32 x NACC f32)]
  uint8_t* ring = smem_raw + (size_t)warp * WS::WARP_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + (size_t)nwarps * WS::WARP_BYTES) + warp * STREAM_STAGES;
  float* red = reinterpret_cast<float*>(smem_raw + (size_t)nwarps * WS::WARP_BYTES + (size_t)nwarps * STREAM_STAGES * 8);
  red += (size_t)group * 2 * KS * 32 * NACC;

  WS ws;
  ws.init(smem_u32(ring), smem_u32(bars), &wmap0, &wmap1, 0, K, lane, err_flag);

  const int ntiles = (N + 15) >> 4;
  const int group_global = blockIdx.x * groups + group;
  const int groups_total = gridDim.x * groups;
  const int my_tiles = group_global < ntiles ? (ntiles - group_global + groups_total - 1) / groups_total : 0;
  const int c_begin = (int)(((long long)ws.nch * ks) >> ks_log2);
  const int c_end = (int)(((long long)ws.nch * (ks + 1)) >> ks_log2);
  const int cper = c_end - c_begin;
  const int steps = my_tiles * cper;

  const __half* xr[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int m = nt * 8 + g;
    xr[nt] = m < M ? x16 + (size_t)m * K : nullptr;
  }

  auto step_tile = [&](int i) { return group_global + (i / cper) * groups_total; };
  auto step_chunk = [&](int i) { return c_begin + (i % cper); };

  if (cper > 0) {
#pragma unroll
    for (int p = 0; p < STREAM_STAGES - 1; ++p)
      if (p < steps) ws.issue(p, step_tile(p) * 16, step_chunk(p));
  }
  // Programmatic dependent launch: this grid may start while the activation-preparation kernel is
  // still running (the weight boxes above do not depend on it); everything below reads its output.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  float acc[NSETS][NT][4];
#pragma unroll
  for (int a = 0; a < NSETS; ++a)
#pragma unroll
    for (int b = 0; b < NT; ++b)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;

  int tile_parity = 0;
  for (int j = 0; j < my_tiles; ++j) {
    const int row0 = (group_global + j * groups_total) * 16;
    for (int cc = 0; cc < cper; ++cc) {
      const int i = j * cper + cc;
      const int stage = i % STREAM_STAGES;
      const int nxt = i + STREAM_STAGES - 1;
      if (nxt < steps) ws.issue(nxt % STREAM_STAGES, step_tile(nxt) * 16, step_chunk(nxt));
      const bool ready = ws.wait(stage, (uint32_t)((i / STREAM_STAGES) & 1));

      const int c = c_begin + cc;
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
      for (int gi = 0; gi < ngroups; ++gi) {
        if (PRE && gi + 1 < ngroups) GP::template load_b<NT>(xr, col_base + (gi + 1) * F::GROUP, t, bnext);
        GP::template run<NSETS, NT, PRE>(s, t, bcur, xr, col_base + gi * F::GROUP, acc);
        if (PRE) bcur = bnext;
#pragma unroll
        for (int r = 0; r < 2 * NSETS; ++r) s[r] += GROUP_BYTES;
      }
      __syncwarp();
    }

    // ---- combine the KS partial sums of this tile (fixed order) ----
    if (KS > 1) {
      float* buf = red + (size_t)tile_parity * KS * 32 * NACC;
      float* flat = &acc[0][0][0];
      if (ks != 0) {
#pragma unroll
        for (int i = 0; i < NACC; ++i) buf[((size_t)ks * NACC + i) * 32 + lane] = flat[i];
      }
      asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(KS * 32) : "memory");
      if (ks == 0) {
        for (int k2 = 1; k2 < KS; ++k2) {
#pragma unroll
          for (int i = 0; i < NACC; ++i) flat[i] += buf[((size_t)k2 * NACC + i) * 32 + lane];
        }
      }
      tile_parity ^= 1;
    }

    // ---- epilogue: row scale back, bias, activation, residual, one rounding ----
    if (ks == 0) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int n = row0 + g + (e >> 1) * 8;
          const int m = nt * 8 + 2 * t + (e & 1);
          if (n < N && m < M) {
            const float rs = rowscale[m];
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
    }
#pragma unroll
    for (int a = 0; a < NSETS; ++a)
#pragma unroll
      for (int b = 0; b < NT; ++b)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;
  }
}

template <int FMT, int NT, bool DUAL>
static size_t stream_smem_bytes(int nwarps, int ks) {
  using WS = typename StreamCfg<FMT, DUAL>::WS;
  const int nacc = NT * 4 * (DUAL ? 2 : 1);
  return (size_t)nwarps * WS::WARP_BYTES + (size_t)nwarps * STREAM_STAGES * 8 +
         (ks > 1 ? (size_t)nwarps * 2 * 32 * nacc * 4 : 0);
}

template <int FMT, int NT, bool DUAL, typename T>
static bool launch_stream_t(cudaStream_t st, const GemvArgs& a) {
  using Cfg = StreamCfg<FMT, DUAL>;
  const int sms = sm_count();
  const int ntiles = (int)((a.N + 15) / 16);
  const int nch = (int)((a.K + Cfg::KC - 1) / Cfg::KC);
  int nwarps = STREAM_MAX_WARPS;
  if (const char* e = getenv("QX_STREAM_WARPS")) nwarps = max(1, min(STREAM_MAX_WARPS, atoi(e)));
  while (nwarps > 1 && stream_smem_bytes<FMT, NT, DUAL>(nwarps, 8) > 220 * 1024) --nwarps;
  if (nwarps > 4) nwarps &= ~3; else if (nwarps == 3) nwarps = 2;
  // split K inside a CTA (KS a power of two that divides nwarps) until there are enough
  // (tile, slice) units for every warp of the GPU
  int ks_log2 = 0;
  while (nwarps % (2 << ks_log2) == 0 && ((long long)ntiles << ks_log2) < (long long)sms * nwarps &&
         (nch >> (ks_log2 + 1)) >= 1)
    ++ks_log2;
  const int groups = nwarps >> ks_log2;
  int blocks = (ntiles + groups - 1) / groups;
  if (blocks > sms) blocks = sms;
  const size_t smem = stream_smem_bytes<FMT, NT, DUAL>(nwarps, 1 << ks_log2);
  static bool attr_set[64] = {};                    // per instantiation and device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return false;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(gemv_stream_kernel<FMT, NT, DUAL, T>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    attr_set[dev] = true;
  }
  int* err = device_error_flag();
  if (!err) return false;

  // stream-ordered scratch for the prepared activations
  const size_t x16_bytes = ((size_t)a.M * a.K * 2 + 255) & ~(size_t)255;
  bool must_free = false;
  void* scratch = stream_scratch(st, x16_bytes + (size_t)a.M * 4, &must_free);
  if (!scratch) return false;
  __half* x16 = (__half*)scratch;
  float* rowscale = (float*)((char*)scratch + x16_bytes);
  launch_prep_activations(st, a.x, a.dtype, x16, rowscale, (int)a.M, (int)a.K, StreamFmt<FMT>::PERM);
  using WSG = typename StreamCfg<FMT, DUAL>::WS::G;
  const size_t row_bytes = (size_t)(a.K / StreamFmt<FMT>::BK) * StreamFmt<FMT>::BB;
  CUtensorMap map0, map1;
  bool maps_ok = make_weight_map(&map0, a.w0, a.N, row_bytes, WSG::PITCH, 16);
  if (maps_ok && DUAL) maps_ok = make_weight_map(&map1, a.w1, a.N, row_bytes, WSG::PITCH, 16);
  if (!DUAL) map1 = map0;
  if (!maps_ok) {
    if (must_free) cudaFreeAsync(scratch, st);
    return false;
  }
  // launched as a programmatic dependent of the preparation kernel (see griddepcontrol.wait)
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
  if (cudaLaunchKernelEx(&cfg, gemv_stream_kernel<FMT, NT, DUAL, T>, map0, map1, (const __half*)x16,
                         (const float*)rowscale, (const T*)a.bias0, (const T*)a.bias1,
                         (const T*)a.residual, (T*)a.y, (int)a.M, (int)a.K, (int)a.N, a.activation,
                         a.use_bias, a.use_residual, ks_log2, err) != cudaSuccess) {
    cudaGetLastError();
    gemv_stream_kernel<FMT, NT, DUAL, T><<<blocks, nwarps * 32, smem, st>>>(
        map0, map1, x16, rowscale, (const T*)a.bias0, (const T*)a.bias1, (const T*)a.residual,
        (T*)a.y, (int)a.M, (int)a.K, (int)a.N, a.activation, a.use_bias, a.use_residual, ks_log2, err);
  }
  if (must_free) cudaFreeAsync(scratch, st);
  note_launch(2);
  return true;
}

template <int FMT, typename T>
static bool launch_stream_f(cudaStream_t st, const GemvArgs& a) {
  const bool dual = a.w1 != nullptr;
  if (a.M <= 8) return dual ? launch_stream_t<FMT, 1, true, T>(st, a) : launch_stream_t<FMT, 1, false, T>(st, a);
  return dual ? launch_stream_t<FMT, 2, true, T>(st, a) : launch_stream_t<FMT, 2, false, T>(st, a);
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

}  // namespace qx
