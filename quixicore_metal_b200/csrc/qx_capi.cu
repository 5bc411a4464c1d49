// C ABI and dispatch: argument validation mirroring the reference host checks, kernel selection
// by (format, dtype, batch, alignment), workspace carving, stream launch.  No CPU fallback.
#include <atomic>
#include <cstring>

#include "qx_common.cuh"
#include <string>

#include "qx_kernels.h"

namespace qx {

static std::atomic<uint64_t> g_launches{0};
void note_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

qx_status ok(const char* op) { return qx_status{(qx_status_code_u8)QX_OK, op, ""}; }
qx_status fail(qx_status_code code, const char* op, const char* detail) {
  return qx_status{(qx_status_code_u8)code, op, detail};
}
qx_status check_launch(const char* op) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(QX_RUNTIME_ERROR, op, cudaGetErrorString(e));
  return ok(op);
}
int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int parse_format(const char* name) {
  if (!name) return -1;
  static const char* names[F_COUNT] = {"q4_0", "q8_0", "q6_K", "mxfp8", "nvfp4", "mxfp4"};
  for (int i = 0; i < F_COUNT; ++i)
    if (std::strcmp(name, names[i]) == 0) return i;
  return -1;
}

static bool float_dtype(qx_dtype d) {
  return d == QX_DTYPE_F32 || d == QX_DTYPE_F16 || d == QX_DTYPE_BF16;
}
static size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

static bool device_ready(const char* op, qx_status* st) {
  int dev = -1;
  const cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    *st = fail(QX_RUNTIME_ERROR, op, "no usable CUDA device (this backend has no CPU fallback)");
    return false;
  }
  return true;
}

// Shared checks of the two projection ops (the reference's check_decode_epilogue_weight).
static qx_status check_projection(const char* op, const void* x, const void* w, void* y, int64_t M,
                                  int64_t K, int64_t N, const char* format, qx_dtype dtype,
                                  int* fmt_out) {
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "x must be non-empty (B,K) fp32/fp16/bf16");
  if (!x || !w || !y) return fail(QX_INVALID_ARGUMENT, op, "x, weight and output pointers must be non-null");
  if (M <= 0 || K <= 0) return fail(QX_INVALID_SHAPE, op, "x must be non-empty (B,K) fp32/fp16/bf16");
  const int f = parse_format(format);
  if (f < 0)
    return fail(QX_UNSUPPORTED_FORMAT, op, "format must be q4_0, q8_0, q6_K, mxfp8, nvfp4, or mxfp4");
  if (N <= 0 || K % block_k_of(f) != 0)
    return fail(QX_INVALID_SHAPE, op, "packed weight must be uint8 (N,K/block_k,block_bytes)");
  if (M > 0x7fffffff || K > 0x7fffffff || N > 0x7fffffff)
    return fail(QX_INVALID_SHAPE, op, "dimensions must fit in 31 bits");
  *fmt_out = f;
  return ok(op);
}

}  // namespace qx

using namespace qx;

extern "C" {

int qx_cuda_format_info(const char* format, int* block_k, int* block_bytes) {
  const int f = parse_format(format);
  if (f < 0) return 0;
  if (block_k) *block_k = block_k_of(f);
  if (block_bytes) *block_bytes = block_bytes_of(f);
  return 1;
}
uint64_t qx_cuda_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
const char* qx_cuda_version(void) { return "quixicore-b200 0.2 (sm_100a)"; }
int qx_cuda_device_error(void) { return read_device_error_flag(); }
int qx_cuda_set_option(const char* name, int value) { return set_option(name, value) ? 1 : 0; }
uint64_t qx_cuda_scratch_alloc_count(void) { return scratch_alloc_count(); }

// Scratch for one projection call: the caller's workspace when it brought one, else the library's
// per-stream buffer.  `held` releases a per-call allocation when it goes out of scope.
struct ScratchHold {
  cudaStream_t st; void* ptr = nullptr; bool must_free = false;
  ~ScratchHold() { if (must_free && ptr) cudaFreeAsync(ptr, st); }
};
static qx_status bind_scratch(const char* op, cudaStream_t st, size_t need, void* workspace,
                              size_t workspace_bytes, ScratchHold* hold, void** out, size_t* out_bytes) {
  *out = nullptr; *out_bytes = 0;
  if (need == 0) return ok(op);
  if (workspace) {
    if (workspace_bytes < need || ((uintptr_t)workspace & 255) != 0)
      return fail(QX_INSUFFICIENT_WORKSPACE, op, "workspace must be 256-byte aligned and at least as large as the op's workspace-bytes query");
    *out = workspace; *out_bytes = workspace_bytes;
    return ok(op);
  }
  hold->st = st;
  hold->ptr = default_scratch(st, need, &hold->must_free);
  if (!hold->ptr) return fail(QX_RUNTIME_ERROR, op, "device scratch allocation failed");
  *out = hold->ptr; *out_bytes = need;
  return ok(op);
}

static qx_status check_out_quant(const char* op, int out_quant, void* out_codes, float* out_scale, int64_t N) {
  if (out_quant < 0 || out_quant > 3) return fail(QX_INVALID_ARGUMENT, op, "output_quant must be None, 'fp8', 'int8', or 'mxfp8'");
  if (out_quant != 0 && !out_codes) return fail(QX_INVALID_ARGUMENT, op, "output_quant needs an out_codes buffer");
  if ((out_quant == 1 || out_quant == 2) && !out_scale) return fail(QX_INVALID_ARGUMENT, op, "per-token output_quant needs an out_scale buffer");
  if (out_quant == 3 && N % 32 != 0) return fail(QX_INVALID_SHAPE, op, "mxfp8 output rows need N to be a multiple of 32");
  return ok(op);
}

// the output quantisation the projection kernel did not fuse
static void finish_out_quant(cudaStream_t st, const GemvArgs& a, bool fused) {
  if (a.out_quant == OQ_NONE || fused) return;
  if (a.out_quant == OQ_MXFP8) launch_quantize_mxfp8_rows(st, a.y, a.q_codes, a.M, a.N, a.dtype);
  else launch_quantize_per_token(st, a.y, a.q_codes, a.q_scale, a.M, a.N, a.dtype, a.out_quant == OQ_INT8 ? 1 : 0);
}

size_t qx_cuda_projection_workspace_bytes(int64_t M, int64_t K, int64_t N, const char* format,
                                          qx_dtype dtype, int swiglu) {
  const int f = parse_format(format);
  if (f < 0 || M <= 0 || K <= 0 || N <= 0 || K % block_k_of(f) != 0 || !float_dtype(dtype)) return 0;
  void* aligned = (void*)(uintptr_t)256;          // alignment stand-in: only the address bits are inspected
  GemvArgs a{aligned, aligned, swiglu ? aligned : nullptr, nullptr, nullptr, nullptr, aligned, M, K, N, f, dtype, 0, 0, 0};
  size_t need = projection_scratch_bytes(a);
  a.out_f32 = 1;                                  // the fp32-partial form of the same shape
  const size_t p = swiglu ? 0 : projection_scratch_bytes(a);
  return need > p ? need : p;
}

qx_status qx_cuda_decode_linear_epilogue(void* stream, const void* x, const void* weight,
                                         const void* bias, const void* residual, void* y,
                                         int64_t M, int64_t K, int64_t N, const char* format,
                                         qx_dtype dtype, int activation, int use_bias,
                                         int use_residual, int out_quant, void* out_codes,
                                         float* out_scale, void* workspace, size_t workspace_bytes) {
  static const char* op = "decode_linear_epilogue";
  if (activation < 0 || activation > 2)
    return fail(QX_INVALID_ARGUMENT, op, "activation must be 0, 1, or 2");
  int f = -1;
  qx_status st = check_projection(op, x, weight, y, M, K, N, format, dtype, &f);
  if (st.code != QX_OK) return st;
  if (use_bias && !bias) return fail(QX_INVALID_ARGUMENT, op, "bias must be (N,) with x dtype");
  if (use_residual && !residual)
    return fail(QX_INVALID_ARGUMENT, op, "residual must be (B,N) with x dtype");
  st = check_out_quant(op, out_quant, out_codes, out_scale, N);
  if (st.code != QX_OK) return st;
  if (!device_ready(op, &st)) return st;
  GemvArgs a{x, weight, nullptr, bias, nullptr, residual, y, M, K, N, f, dtype,
             activation, use_bias ? 1 : 0, use_residual ? 1 : 0};
  a.out_quant = out_quant; a.q_codes = out_codes; a.q_scale = out_scale;
  ScratchHold hold;
  st = bind_scratch(op, (cudaStream_t)stream, projection_scratch_bytes(a), workspace, workspace_bytes, &hold,
                    &a.scratch, &a.scratch_bytes);
  if (st.code != QX_OK) return st;
  const bool fused = launch_projection((cudaStream_t)stream, a);
  finish_out_quant((cudaStream_t)stream, a, fused);
  return check_launch(op);
}

qx_status qx_cuda_decode_linear_partial(void* stream, const void* x, const void* weight, float* y,
                                        int64_t M, int64_t K, int64_t N, const char* format,
                                        qx_dtype dtype, void* workspace, size_t workspace_bytes) {
  static const char* op = "decode_linear_epilogue.partial";
  int f = -1;
  qx_status st = check_projection(op, x, weight, y, M, K, N, format, dtype, &f);
  if (st.code != QX_OK) return st;
  if (!device_ready(op, &st)) return st;
  GemvArgs a{x, weight, nullptr, nullptr, nullptr, nullptr, y, M, K, N, f, dtype, 0, 0, 0};
  a.out_f32 = 1;
  ScratchHold hold;
  st = bind_scratch(op, (cudaStream_t)stream, projection_scratch_bytes(a), workspace, workspace_bytes, &hold,
                    &a.scratch, &a.scratch_bytes);
  if (st.code != QX_OK) return st;
  if (stream_path_ok(a) && launch_gemv_stream((cudaStream_t)stream, a)) return check_launch(op);
  if (stream_passes_ok(a) && launch_gemv_stream_passes((cudaStream_t)stream, a)) return check_launch(op);
  if (tc_path_ok(a) && launch_gemm_tc((cudaStream_t)stream, a)) return check_launch(op);
  return fail(QX_UNSUPPORTED_LAYOUT, op,
              "fp32 partial projections need bf16/f16 activations, 16-byte aligned bases and K a "
              "multiple of 512 columns");
}

qx_status qx_cuda_decode_swiglu(void* stream, const void* x, const void* gate_weight,
                                const void* up_weight, const void* gate_bias, const void* up_bias,
                                void* y, int64_t M, int64_t K, int64_t N, const char* format,
                                qx_dtype dtype, int use_bias, int out_quant, void* out_codes,
                                float* out_scale, void* workspace, size_t workspace_bytes) {
  static const char* op = "decode_swiglu";
  int f = -1;
  qx_status st = check_projection(op, x, gate_weight, y, M, K, N, format, dtype, &f);
  if (st.code != QX_OK) return st;
  if (!up_weight)
    return fail(QX_INVALID_ARGUMENT, op, "gate and up weights must have identical shapes");
  if (use_bias && (!gate_bias || !up_bias))
    return fail(QX_INVALID_ARGUMENT, op, "both biases must be (N,) with x dtype");
  st = check_out_quant(op, out_quant, out_codes, out_scale, N);
  if (st.code != QX_OK) return st;
  if (!device_ready(op, &st)) return st;
  GemvArgs a{x, gate_weight, up_weight, gate_bias, up_bias, nullptr, y, M, K, N, f, dtype,
             0, use_bias ? 1 : 0, 0};
  a.out_quant = out_quant; a.q_codes = out_codes; a.q_scale = out_scale;
  ScratchHold hold;
  st = bind_scratch(op, (cudaStream_t)stream, projection_scratch_bytes(a), workspace, workspace_bytes, &hold,
                    &a.scratch, &a.scratch_bytes);
  if (st.code != QX_OK) return st;
  const bool fused = launch_projection((cudaStream_t)stream, a);
  finish_out_quant((cudaStream_t)stream, a, fused);
  return check_launch(op);
}

qx_status qx_cuda_quantize_per_token(void* stream, const void* x, void* codes, float* scale,
                                     int64_t rows, int64_t D, qx_dtype dtype, int kind) {
  const char* op = kind == 1 ? "quantize_per_token_int8" : "quantize_per_token_fp8";
  if (kind != 0 && kind != 1) return fail(QX_INVALID_ARGUMENT, "quantize_per_token", "kind must be 0 (fp8) or 1 (int8)");
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "x must be fp32/fp16/bf16");
  if (!x || !codes || !scale) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (rows <= 0 || D <= 0 || D > 0x7fffffff || rows > 0x7fffffff)
    return fail(QX_INVALID_SHAPE, op, "x must be a non-empty (rows, D) matrix");
  qx_status st;
  if (!device_ready(op, &st)) return st;
  launch_quantize_per_token((cudaStream_t)stream, x, codes, scale, rows, D, dtype, kind);
  return check_launch(op);
}

qx_status qx_cuda_quantize_mxfp8_rows(void* stream, const void* x, void* blocks, int64_t rows,
                                      int64_t D, qx_dtype dtype) {
  static const char* op = "quantize_mxfp8_rows";
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "x must be fp32/fp16/bf16");
  if (!x || !blocks) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (rows <= 0 || D <= 0 || D % 32 != 0)
    return fail(QX_INVALID_SHAPE, op, "x must be (rows, D) with D a positive multiple of 32");
  qx_status st;
  if (!device_ready(op, &st)) return st;
  launch_quantize_mxfp8_rows((cudaStream_t)stream, x, blocks, rows, D, dtype);
  return check_launch(op);
}

// ---- LM head ---------------------------------------------------------------------------------
static qx_status check_lm_head(const char* op, const void* h, const void* wq, int64_t T, int64_t V,
                               int64_t K, const char* format, qx_dtype dtype, int mode, int topk,
                               double temperature, int* fmt_out) {
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "h must be floating point");
  if (!h || !wq) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (mode < 0 || mode > 3)
    return fail(QX_INVALID_ARGUMENT, op, "mode 0=argmax, 1=categorical, 2=topk, 3=topp");
  if (!(temperature > 0.0)) return fail(QX_INVALID_ARGUMENT, op, "temperature must be positive");
  const int f = parse_format(format);
  if (f < 0)
    return fail(QX_UNSUPPORTED_FORMAT, op, "format must be q8_0, q4_0, q6_K, mxfp8, nvfp4, or mxfp4");
  if (T <= 0 || V <= 0 || K <= 0) return fail(QX_INVALID_SHAPE, op, "T, V, and K must be positive");
  if (K % block_k_of(f) != 0)
    return fail(QX_INVALID_SHAPE, op, "packed weight shape does not match V/K/format");
  if (T > 0x7fffffff || V > 0x7fffffff || K > 0x7fffffff)
    return fail(QX_INVALID_SHAPE, op, "dimensions must fit in 31 bits");
  if (mode >= 2) {
    if (topk < 1 || topk > 64) return fail(QX_INVALID_ARGUMENT, op, "k must be in [1, 64]");
  }
  *fmt_out = f;
  return ok(op);
}

static int64_t tiles_of(int64_t V) { return (V + 255) / 256; }

static size_t partial_bytes(int64_t T, int64_t V, int mode, int topk) {
  const size_t tiles = (size_t)tiles_of(V);
  const size_t kk = mode >= 2 ? (size_t)(topk > 0 ? topk : 1) : 1;
  size_t n = 2 * align256((size_t)T * tiles * kk * 4);
  if (mode == 3) n += align256((size_t)T * tiles * 4);
  return n;
}

size_t qx_cuda_lm_head_workspace_bytes(int64_t T, int64_t V, int64_t K, int mode, int topk) {
  if (T <= 0 || V <= 0 || K <= 0) return 0;
  return partial_bytes(T, V, mode, topk) + lm_head_scratch_full_bytes(T, K);
}

}  // extern "C"

namespace qx {
// The body of qx_cuda_lm_head_sample_q on a given scratch region: [partials | stage-1 scratch].
// min_only: the region only has to hold the partials and the minimum stage-1 scratch (K-split
// items are then shared only as far as the rest reaches).
qx_status lm_head_sample_on(const char* op, void* stream, const void* h, const void* wq, const float* bias,
                            int32_t* ids, void* workspace, size_t workspace_bytes, bool min_only, int64_t T,
                            int64_t V, int64_t K, const char* format, qx_dtype dtype, int mode, int topk,
                            double temperature, uint32_t seed, double top_p) {
  int f = -1;
  qx_status st = check_lm_head(op, h, wq, T, V, K, format, dtype, mode, topk, temperature, &f);
  if (st.code != QX_OK) return st;
  if (!ids) return fail(QX_INVALID_ARGUMENT, op, "null output pointer");
  if (mode >= 2 && topk > V) return fail(QX_INVALID_ARGUMENT, op, "k must be <= vocab size V");
  if (mode == 3 && !(top_p > 0.0 && top_p <= 1.0))
    return fail(QX_INVALID_ARGUMENT, op, "topp requires top_p in (0, 1]");
  const size_t pbytes = partial_bytes(T, V, mode, topk);
  const size_t need = pbytes + (min_only ? lm_head_scratch_min_bytes(T, K) : lm_head_scratch_full_bytes(T, K));
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255) != 0)
    return fail(QX_INSUFFICIENT_WORKSPACE, op, "workspace must be 256-byte aligned and at least qx_cuda_lm_head_workspace_bytes");
  if (!device_ready(op, &st)) return st;
  const int64_t tiles = tiles_of(V);
  const int kk = mode >= 2 ? topk : 1;
  const size_t seg = align256((size_t)T * tiles * kk * 4);
  float* pv = (float*)workspace;
  int32_t* pi = (int32_t*)((char*)workspace + seg);
  float* pl = (float*)((char*)workspace + 2 * seg);
  LmHeadArgs a{h, wq, bias, T, V, K, 0, f, dtype, mode, kk, 1.0f / (float)temperature, seed,
               (float)top_p};
  a.scratch = (char*)workspace + pbytes;
  a.scratch_bytes = workspace_bytes - pbytes;
  launch_lm_head_partials((cudaStream_t)stream, a, pv, pi, pl, tiles);
  launch_lm_head_reduce((cudaStream_t)stream, pv, pi, pl, 1, T, tiles * kk, tiles, 0, mode, kk,
                        a.invtemp, seed, a.top_p, ids, 0, nullptr, nullptr);
  return check_launch(op);
}
}  // namespace qx

extern "C" {

qx_status qx_cuda_lm_head_sample_q(void* stream, const void* h, const void* wq, const float* bias,
                                   int32_t* ids, void* workspace, size_t workspace_bytes, int64_t T,
                                   int64_t V, int64_t K, const char* format, qx_dtype dtype,
                                   int mode, int topk, double temperature, uint32_t seed,
                                   double top_p) {
  return lm_head_sample_on("quantized_lm_head_sample", stream, h, wq, bias, ids, workspace, workspace_bytes,
                           false, T, V, K, format, dtype, mode, topk, temperature, seed, top_p);
}

size_t qx_cuda_lm_head_dense_workspace_bytes(int64_t T, int64_t V, int mode, int topk) {
  if (T <= 0 || V <= 0 || mode < 0 || mode > 2) return 0;
  return partial_bytes(T, V, mode, topk);
}

qx_status qx_cuda_lm_head_sample_dense(void* stream, const void* h, const void* W, const float* bias,
                                       int32_t* ids, void* workspace, size_t workspace_bytes,
                                       int64_t T, int64_t V, int64_t K, qx_dtype dtype, int mode,
                                       int topk, double temperature, uint32_t seed) {
  static const char* op = "lm_head_sample";
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "h/W must be the same float dtype (f32/f16/bf16)");
  if (!h || !W || !ids) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (mode < 0 || mode > 2) return fail(QX_INVALID_ARGUMENT, op, "mode must be 0/1/2");
  if (!(temperature > 0.0)) return fail(QX_INVALID_ARGUMENT, op, "temperature must be positive");
  if (T <= 0 || V <= 0 || K <= 0 || T > 0x7fffffff || V > 0x7fffffff || K > 0x7fffffff)
    return fail(QX_INVALID_SHAPE, op, "h (T,K) and W (V,K) must share K");
  if (mode == 2 && (topk < 1 || topk > 64)) return fail(QX_INVALID_ARGUMENT, op, "topk k must be in [1, 64]");
  if (mode == 2 && topk > V) return fail(QX_INVALID_ARGUMENT, op, "topk k must be <= vocab size V");
  const size_t need = partial_bytes(T, V, mode, topk);
  if (!workspace || workspace_bytes < need)
    return fail(QX_INSUFFICIENT_WORKSPACE, op, "workspace smaller than qx_cuda_lm_head_dense_workspace_bytes");
  qx_status st;
  if (!device_ready(op, &st)) return st;
  const int64_t tiles = tiles_of(V);
  const int kk = mode == 2 ? topk : 1;
  const size_t seg = align256((size_t)T * tiles * kk * 4);
  float* pv = (float*)workspace;
  int32_t* pi = (int32_t*)((char*)workspace + seg);
  const float invtemp = 1.0f / (float)temperature;
  launch_lm_head_dense_partials((cudaStream_t)stream, h, W, bias, pv, pi, T, V, K, dtype, mode, kk, invtemp, seed);
  launch_lm_head_reduce((cudaStream_t)stream, pv, pi, nullptr, 1, T, tiles * kk, 0, 0, mode, kk, invtemp, seed,
                        1.0f, ids, 0, nullptr, nullptr);
  return check_launch(op);
}

qx_status qx_cuda_sample_logits(void* stream, const void* logits, int32_t* ids, int64_t rows, int64_t V,
                                qx_dtype dtype, int kind, int topk, double top_p, double temperature,
                                uint32_t seed) {
  static const char* names[4] = {"argmax_sample", "sample_categorical", "top_k_sample", "top_p_sample"};
  if (kind < 0 || kind > 3) return fail(QX_INVALID_ARGUMENT, "sample_logits", "kind 0=argmax, 1=categorical, 2=top-k, 3=top-p");
  const char* op = names[kind];
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "logits must be fp32/fp16/bf16");
  if (!logits || !ids) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (rows <= 0 || V <= 0 || rows > 0x7fffffff || V > 0x7fffffff)
    return fail(QX_INVALID_SHAPE, op, "logits must be a non-empty (rows, V) matrix");
  if (kind >= 1 && !(temperature > 0.0)) return fail(QX_INVALID_ARGUMENT, op, "temperature must be positive");
  if (kind == 2 && (topk < 1 || topk > 64 || topk > V)) return fail(QX_INVALID_ARGUMENT, op, "k must be in [1, min(64, V)]");
  if (kind == 3 && !(top_p > 0.0 && top_p <= 1.0)) return fail(QX_INVALID_ARGUMENT, op, "p must be in (0, 1]");
  qx_status st;
  if (!device_ready(op, &st)) return st;
  launch_sample_logits((cudaStream_t)stream, logits, ids, rows, V, dtype, kind, topk, (float)top_p,
                       kind == 0 ? 1.0f : 1.0f / (float)temperature, seed);
  return check_launch(op);
}

// ---- the operators either side of the path: qgemv / qgemm, packed embedding lookup ------------------
size_t qx_cuda_qgemm_workspace_bytes(int64_t N, int64_t K, int64_t M, const char* format, qx_dtype dtype) {
  if (N <= 0 || K <= 0 || M <= 0) return 0;
  const size_t es = dtype == QX_DTYPE_F32 ? 4 : 2;
  const size_t proj = qx_cuda_projection_workspace_bytes(M, K, N, format, dtype, 0);
  if (M == 1) return proj;                                  // (K,1) and (N,1) are already the row layout
  return align256((size_t)M * K * es) + align256((size_t)M * N * es) + proj;
}

qx_status qx_cuda_qgemm(void* stream, const void* wq, const void* x, void* out, int64_t N, int64_t K,
                        int64_t M, const char* format, qx_dtype dtype, void* workspace,
                        size_t workspace_bytes) {
  const char* op = M == 1 ? "qgemv" : "qgemm";
  if (dtype != QX_DTYPE_F16 && dtype != QX_DTYPE_F32 && dtype != QX_DTYPE_BF16)
    return fail(QX_UNSUPPORTED_DTYPE, op, "x must be float16 (float32 / bfloat16 are accepted too)");
  int f = -1;
  qx_status st = check_projection(op, x, wq, out, M, K, N, format, dtype, &f);
  if (st.code != QX_OK) return st;
  const size_t need = qx_cuda_qgemm_workspace_bytes(N, K, M, format, dtype);
  if (need && (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255) != 0))
    return fail(QX_INSUFFICIENT_WORKSPACE, op, "workspace must be 256-byte aligned and at least qx_cuda_qgemm_workspace_bytes");
  if (!device_ready(op, &st)) return st;
  const size_t es = dtype == QX_DTYPE_F32 ? 4 : 2;
  const void* xr = x;
  void* yr = out;
  char* ws = (char*)workspace;
  if (M > 1) {
    launch_transpose((cudaStream_t)stream, x, ws, K, M, es);           // (K, M) -> (M, K)
    xr = ws;
    yr = ws + align256((size_t)M * K * es);
    ws = (char*)yr + align256((size_t)M * N * es);
  }
  GemvArgs a{xr, wq, nullptr, nullptr, nullptr, nullptr, yr, M, K, N, f, dtype, 0, 0, 0};
  a.scratch = ws;
  a.scratch_bytes = workspace ? workspace_bytes - (size_t)(ws - (char*)workspace) : 0;
  launch_projection((cudaStream_t)stream, a);
  if (M > 1) launch_transpose((cudaStream_t)stream, yr, out, M, N, es);  // (M, N) -> (N, M)
  return check_launch(op);
}

qx_status qx_cuda_quantized_embedding(void* stream, const void* table, const int32_t* ids, const void* add,
                                      void* out, int64_t rows, int64_t columns, int64_t tokens,
                                      const char* format, double scale, int use_add, qx_dtype out_dtype) {
  static const char* op = "quantized_embedding";
  if (!float_dtype(out_dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "output_dtype must be 'float16', 'bfloat16', or 'float32'");
  const int f = parse_format(format);
  if (f < 0) return fail(QX_UNSUPPORTED_FORMAT, op, "format must be q4_0, q8_0, q6_K, mxfp8, nvfp4, or mxfp4");
  if (!table || !ids || !out || (use_add && !add)) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (rows <= 0 || columns <= 0 || tokens <= 0 || columns % block_k_of(f) != 0 || rows > 0x7fffffff || columns > 0x7fffffff)
    return fail(QX_INVALID_SHAPE, op, "table must be packed uint8 (rows,blocks,block_bytes)");
  qx_status st;
  if (!device_ready(op, &st)) return st;
  launch_quantized_embedding((cudaStream_t)stream, f, out_dtype, table, ids, add, out, rows, columns, tokens,
                             (float)scale, use_add ? 1 : 0);
  return check_launch(op);
}

// ---- norm / activation -> quantiser seams ---------------------------------------------------------
qx_status qx_cuda_rms_norm_add(void* stream, const void* x, const void* residual, const void* weight, void* y,
                               void* codes, void* res_out, float* scale, int64_t rows, int64_t D, qx_dtype dtype,
                               double eps, int quant, double static_scale, int group, int ue8m0) {
  static const char* op = "rms_norm_add";
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "x must be fp32/fp16/bf16");
  if (!x || !residual || !weight || !res_out) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (rows <= 0 || D <= 0 || rows > 0x7fffffff || D > 51200) return fail(QX_INVALID_SHAPE, op, "x must be (rows, D) with 0 < D <= 51200");
  if (quant < 0 || quant > 5) return fail(QX_INVALID_ARGUMENT, op, "quant: 0 none, 1 fp8 static, 2 fp8 per row, 3 int8 per row, 4 fp8 per block, 5 int8 per block");
  if (quant == 0 && !y) return fail(QX_INVALID_ARGUMENT, op, "null output pointer");
  if (quant != 0 && !codes) return fail(QX_INVALID_ARGUMENT, op, "null codes pointer");
  if (quant >= 2 && !scale) return fail(QX_INVALID_ARGUMENT, op, "null scale pointer");
  if (quant == 1 && !(static_scale > 0.0)) return fail(QX_INVALID_ARGUMENT, op, "static scale must be positive");
  if (quant >= 4 && (group <= 0 || D % group != 0)) return fail(QX_INVALID_SHAPE, op, "per-block quant requires D % block == 0");
  qx_status st;
  if (!device_ready(op, &st)) return st;
  if (!launch_rms_norm_add((cudaStream_t)stream, dtype, x, residual, weight, y, codes, res_out, scale, rows, D, (float)eps,
                           quant, quant == 1 ? (float)(1.0 / static_scale) : 0.f, group, ue8m0 ? 1 : 0))
    return fail(QX_RUNTIME_ERROR, op, "kernel configuration failed");
  return check_launch(op);
}

qx_status qx_cuda_silu_mul_quant(void* stream, const void* x, const void* gate, void* codes, float* scale,
                                 int64_t rows, int64_t D, qx_dtype dtype, int act, double alpha, double limit,
                                 int quant, int group, int ue8m0) {
  static const char* op = "silu_mul_quant";
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "x must be fp32/fp16/bf16");
  if (!x || !gate || !codes || !scale) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (rows <= 0 || D <= 0 || rows > 0x7fffffff || D > 51200) return fail(QX_INVALID_SHAPE, op, "x must be (rows, D) with 0 < D <= 51200");
  if (act < 0 || act > 1) return fail(QX_INVALID_ARGUMENT, op, "act: 0 swiglu, 1 swiglu_oai");
  if (quant < 2 || quant > 4) return fail(QX_INVALID_ARGUMENT, op, "quant: 2 fp8 per token, 3 int8 per token, 4 fp8 per group");
  if (quant == 4 && (group <= 0 || group % 4 != 0 || D % group != 0))
    return fail(QX_INVALID_SHAPE, op, "group_size must be a multiple of 4 that divides D");
  qx_status st;
  if (!device_ready(op, &st)) return st;
  if (!launch_silu_mul_quant((cudaStream_t)stream, dtype, x, gate, codes, scale, rows, D, act, (float)alpha, (float)limit,
                             quant, group, ue8m0 ? 1 : 0))
    return fail(QX_RUNTIME_ERROR, op, "kernel configuration failed");
  return check_launch(op);
}

// ---- masked / candidate / beam forms of the LM head ------------------------------------------------
static bool dense_format(const char* format) { return !format || format[0] == '\0'; }

static qx_status check_head_weight(const char* op, const void* h, const void* w, int64_t T, int64_t V, int64_t K,
                                   const char* format, qx_dtype dtype, int* fmt_out) {
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "h must be non-empty (T,K) fp32/fp16/bf16");
  if (!h || !w) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (T <= 0 || K <= 0 || V <= 0 || T > 0x7fffffff || V > 0x7fffffff || K > 0x7fffffff)
    return fail(QX_INVALID_SHAPE, op, "h must be non-empty (T,K) fp32/fp16/bf16");
  *fmt_out = -1;
  if (dense_format(format)) return ok(op);
  const int f = parse_format(format);
  if (f < 0) return fail(QX_UNSUPPORTED_FORMAT, op, "format must be empty/dense, q4_0, q8_0, q6_K, mxfp8, nvfp4, or mxfp4");
  if (K % block_k_of(f) != 0) return fail(QX_INVALID_SHAPE, op, "invalid packed weight shape");
  *fmt_out = f;
  return ok(op);
}

size_t qx_cuda_lm_head_masked_workspace_bytes(int64_t T, int64_t V, int64_t K, int topk) {
  if (T <= 0 || V <= 0 || K <= 0 || topk <= 0) return 0;
  return partial_bytes(T, V, 3, topk) + lm_head_scratch_full_bytes(T, K);
}

qx_status qx_cuda_lm_head_masked(void* stream, const void* h, const void* w, const float* bias,
                                 const uint32_t* allow_mask, int32_t* ids, float* logprobs, void* workspace,
                                 size_t workspace_bytes, int64_t T, int64_t V, int64_t K, const char* format,
                                 qx_dtype dtype, int topk, int normalize_allowed) {
  static const char* op = "lm_head_masked";
  int f = -1;
  qx_status st = check_head_weight(op, h, w, T, V, K, format, dtype, &f);
  if (st.code != QX_OK) return st;
  if (topk < 1 || topk > 8 || topk > V) return fail(QX_INVALID_ARGUMENT, op, "topk must be in [1,min(8,V)]");
  if (!allow_mask) return fail(QX_INVALID_ARGUMENT, op, "allow_mask must be (T,ceil(V/32))");
  if (!ids || !logprobs) return fail(QX_INVALID_ARGUMENT, op, "null output pointer");
  const size_t need = qx_cuda_lm_head_masked_workspace_bytes(T, V, K, topk);
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255) != 0)
    return fail(QX_INSUFFICIENT_WORKSPACE, op, "workspace must be 256-byte aligned and at least qx_cuda_lm_head_masked_workspace_bytes");
  if (!device_ready(op, &st)) return st;
  const int64_t tiles = tiles_of(V);
  const size_t seg = align256((size_t)T * tiles * topk * 4);
  float* pv = (float*)workspace;
  int32_t* pi = (int32_t*)((char*)workspace + seg);
  float* pl = (float*)((char*)workspace + 2 * seg);
  const size_t pbytes = partial_bytes(T, V, 3, topk);
  const LmhMask mask{allow_mask, (V + 31) / 32, normalize_allowed ? 1 : 0};
  if (f < 0) {
    launch_lm_head_dense_partials((cudaStream_t)stream, h, w, bias, pv, pi, T, V, K, dtype, 4, topk, 1.0f, 0u, pl, mask);
  } else {
    LmHeadArgs a{h, w, bias, T, V, K, 0, f, dtype, 4, topk, 1.0f, 0u, 1.0f};
    a.mask = mask;
    a.scratch = (char*)workspace + pbytes;
    a.scratch_bytes = workspace_bytes - pbytes;
    launch_lm_head_partials((cudaStream_t)stream, a, pv, pi, pl, tiles);
  }
  launch_lm_head_topk_logprob((cudaStream_t)stream, pv, pi, nullptr, tiles * topk, pl, tiles, nullptr, T, V, topk, ids, logprobs);
  return check_launch(op);
}

qx_status qx_cuda_lm_head_candidates(void* stream, const void* h, const void* w, const float* bias,
                                     const int32_t* candidate_ids, const int32_t* offsets, int64_t entries,
                                     int32_t* ids, float* logprobs, void* workspace, size_t workspace_bytes,
                                     int64_t T, int64_t V, int64_t K, const char* format, qx_dtype dtype,
                                     int topk) {
  static const char* op = "lm_head_candidates";
  int f = -1;
  qx_status st = check_head_weight(op, h, w, T, V, K, format, dtype, &f);
  if (st.code != QX_OK) return st;
  if (topk < 1 || topk > 8 || topk > V) return fail(QX_INVALID_ARGUMENT, op, "topk must be in [1,min(8,V)]");
  if (!offsets || entries < 0 || (entries > 0 && !candidate_ids) || entries > 0x7fffffff)
    return fail(QX_INVALID_ARGUMENT, op, "flat candidate_ids and T+1 offsets required");
  if (!ids || !logprobs) return fail(QX_INVALID_ARGUMENT, op, "null output pointer");
  const size_t need = align256((size_t)(entries > 0 ? entries : 1) * 4);
  if (!workspace || workspace_bytes < need)
    return fail(QX_INSUFFICIENT_WORKSPACE, op, "workspace must hold one float per candidate entry");
  if (!device_ready(op, &st)) return st;
  float* logit = (float*)workspace;
  launch_lm_head_candidate_logits((cudaStream_t)stream, f, dtype, h, w, bias, candidate_ids, offsets, logit, T, V, K, entries);
  launch_lm_head_topk_logprob((cudaStream_t)stream, logit, candidate_ids, offsets, 0, nullptr, 0, nullptr, T, V, topk, ids, logprobs);
  return check_launch(op);
}

size_t qx_cuda_lm_head_beam_workspace_bytes(int64_t rows, int64_t V, int64_t K, int beam_width) {
  if (rows <= 0 || V <= 0 || K <= 0 || beam_width <= 0) return 0;
  return partial_bytes(rows, V, 3, 2 * beam_width) + 2 * align256((size_t)rows * 2 * beam_width * 4) +
         lm_head_scratch_full_bytes(rows, K);
}

qx_status qx_cuda_lm_head_beam_advance(void* stream, const void* h, const void* wq, const float* bias,
                                       const float* cum_log_probs, int32_t* next_token, int32_t* parent_beam,
                                       float* new_cum, void* workspace, size_t workspace_bytes, int64_t batches,
                                       int beam_width, int64_t V, int64_t K, const char* format, qx_dtype dtype) {
  static const char* op = "lm_head_beam_advance";
  if (beam_width < 1 || beam_width > 16) return fail(QX_INVALID_ARGUMENT, op, "beam_width must be in [1,16]");
  if (batches <= 0) return fail(QX_INVALID_SHAPE, op, "cum_log_probs must be (B,BM), h rows B*BM");
  const int64_t rows = batches * beam_width;
  int f = -1;
  qx_status st = check_head_weight(op, h, wq, rows, V, K, format, dtype, &f);
  if (st.code != QX_OK) return st;
  if (f < 0 || f == F_Q6_K) return fail(QX_UNSUPPORTED_FORMAT, op, "format must be q4_0, q8_0, mxfp8, nvfp4, or mxfp4");
  const int two_bm = 2 * beam_width;
  if (V < two_bm) return fail(QX_INVALID_ARGUMENT, op, "vocab must be >= 2*beam_width");
  if (!cum_log_probs || !next_token || !parent_beam || !new_cum) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  const size_t need = qx_cuda_lm_head_beam_workspace_bytes(rows, V, K, beam_width);
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255) != 0)
    return fail(QX_INSUFFICIENT_WORKSPACE, op, "workspace must be 256-byte aligned and at least qx_cuda_lm_head_beam_workspace_bytes");
  if (!device_ready(op, &st)) return st;
  const int64_t tiles = tiles_of(V);
  const size_t seg = align256((size_t)rows * tiles * two_bm * 4);
  const size_t pbytes = partial_bytes(rows, V, 3, two_bm);
  const size_t cseg = align256((size_t)rows * two_bm * 4);
  float* pv = (float*)workspace;
  int32_t* pi = (int32_t*)((char*)workspace + seg);
  float* pl = (float*)((char*)workspace + 2 * seg);
  float* cand_score = (float*)((char*)workspace + pbytes);
  int32_t* cand_token = (int32_t*)((char*)workspace + pbytes + cseg);
  // per 256-row tile the 2*BM best raw logits and the tile log-sum-exp (the top-p partials at
  // temperature 1), merged per beam row into cum + logit - lse, then BM of BM x 2BM per batch
  LmHeadArgs a{h, wq, bias, rows, V, K, 0, f, dtype, 3, two_bm, 1.0f, 0u, 1.0f};
  a.scratch = (char*)workspace + pbytes + 2 * cseg;
  a.scratch_bytes = workspace_bytes - pbytes - 2 * cseg;
  launch_lm_head_partials((cudaStream_t)stream, a, pv, pi, pl, tiles);
  launch_lm_head_topk_logprob((cudaStream_t)stream, pv, pi, nullptr, tiles * two_bm, pl, tiles, cum_log_probs, rows, V, two_bm,
                              cand_token, cand_score);
  launch_beam_select((cudaStream_t)stream, cand_score, cand_token, next_token, parent_beam, new_cum, batches, beam_width, two_bm);
  return check_launch(op);
}

int64_t qx_cuda_lm_head_shard_candidates(int mode, int topk, int64_t max_tiles) {
  if (mode <= 1) return 1;
  if (mode == 2) return topk;
  return max_tiles * topk;
}

size_t qx_cuda_lm_head_shard_workspace_bytes(int64_t T, int64_t V_local, int64_t K, int mode, int topk) {
  if (T <= 0 || V_local <= 0 || K <= 0) return 0;
  size_t n = lm_head_scratch_full_bytes(T, K);
  if (mode != 3) {
    const size_t kk = mode == 2 ? (size_t)(topk > 0 ? topk : 1) : 1;
    n += 2 * align256((size_t)T * (size_t)tiles_of(V_local) * kk * 4);
  }
  return n;
}

qx_status qx_cuda_lm_head_shard_partials_q(void* stream, const void* h, const void* wq,
                                           const float* bias_local, float* cand_val,
                                           int32_t* cand_id, float* cand_lse, void* workspace,
                                           size_t workspace_bytes, int64_t T, int64_t V_local,
                                           int64_t K, int64_t vocab_offset, int64_t max_tiles,
                                           const char* format, qx_dtype dtype, int mode, int topk,
                                           double temperature, uint32_t seed) {
  static const char* op = "quantized_lm_head_sample.shard_partials";
  int f = -1;
  qx_status st = check_lm_head(op, h, wq, T, V_local, K, format, dtype, mode, topk, temperature, &f);
  if (st.code != QX_OK) return st;
  if (!cand_val || !cand_id || (mode == 3 && !cand_lse))
    return fail(QX_INVALID_ARGUMENT, op, "null candidate buffer");
  if (vocab_offset < 0 || vocab_offset % 256 != 0)
    return fail(QX_INVALID_ARGUMENT, op, "vocab_offset must be a non-negative multiple of 256");
  const int64_t tiles = tiles_of(V_local);
  if (max_tiles < tiles) return fail(QX_INVALID_ARGUMENT, op, "max_tiles smaller than this shard's tile count");
  if (vocab_offset + V_local > 0x7fffffffLL) return fail(QX_INVALID_SHAPE, op, "global vocab ids must fit in 31 bits");
  const size_t need = qx_cuda_lm_head_shard_workspace_bytes(T, V_local, K, mode, topk);
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255) != 0)
    return fail(QX_INSUFFICIENT_WORKSPACE, op, "workspace must be 256-byte aligned and at least qx_cuda_lm_head_shard_workspace_bytes");
  if (!device_ready(op, &st)) return st;
  const int kk = mode >= 2 ? topk : 1;
  LmHeadArgs a{h, wq, bias_local, T, V_local, K, vocab_offset, f, dtype, mode, kk,
               1.0f / (float)temperature, seed, 1.0f};
  if (mode == 3) {
    a.scratch = workspace; a.scratch_bytes = workspace_bytes;
    launch_lm_head_partials((cudaStream_t)stream, a, cand_val, cand_id, cand_lse, max_tiles);
    return check_launch(op);
  }
  const size_t seg = align256((size_t)T * tiles * kk * 4);
  float* pv = (float*)workspace;
  int32_t* pi = (int32_t*)((char*)workspace + seg);
  a.scratch = (char*)workspace + 2 * seg; a.scratch_bytes = workspace_bytes - 2 * seg;
  launch_lm_head_partials((cudaStream_t)stream, a, pv, pi, nullptr, tiles);
  launch_lm_head_reduce((cudaStream_t)stream, pv, pi, nullptr, 1, T, tiles * kk, 0, 0, mode, kk,
                        a.invtemp, seed, 1.0f, nullptr, 1, cand_val, cand_id);
  return check_launch(op);
}

qx_status qx_cuda_lm_head_shard_reduce(void* stream, const float* cand_val, const int32_t* cand_id,
                                       const float* cand_lse, int32_t* ids, int64_t shards,
                                       int64_t T, int64_t max_tiles, int64_t shard_stride,
                                       int mode, int topk, double temperature, uint32_t seed,
                                       double top_p) {
  static const char* op = "quantized_lm_head_sample.shard_reduce";
  if (!cand_val || !cand_id || !ids || (mode == 3 && !cand_lse))
    return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (mode < 0 || mode > 3) return fail(QX_INVALID_ARGUMENT, op, "mode 0=argmax, 1=categorical, 2=topk, 3=topp");
  if (shards <= 0 || shards > 1024 || T <= 0 || max_tiles <= 0) return fail(QX_INVALID_SHAPE, op, "shards, T and max_tiles must be positive");
  if (shard_stride < 0) return fail(QX_INVALID_ARGUMENT, op, "shard_stride must be >= 0");
  if (!(temperature > 0.0)) return fail(QX_INVALID_ARGUMENT, op, "temperature must be positive");
  if (mode >= 2 && (topk < 1 || topk > 64)) return fail(QX_INVALID_ARGUMENT, op, "k must be in [1, 64]");
  if (mode == 3 && !(top_p > 0.0 && top_p <= 1.0)) return fail(QX_INVALID_ARGUMENT, op, "topp requires top_p in (0, 1]");
  qx_status st;
  if (!device_ready(op, &st)) return st;
  const int kk = mode >= 2 ? topk : 1;
  const int64_t C = qx_cuda_lm_head_shard_candidates(mode, kk, max_tiles);
  // stage-1 scores of modes 0/1 already carry temperature, bias and noise: the merge is a plain max
  launch_lm_head_reduce((cudaStream_t)stream, cand_val, cand_id, cand_lse, (int)shards, T, C,
                        mode == 3 ? max_tiles : 0, shard_stride, mode, kk, 1.0f / (float)temperature, seed,
                        (float)top_p, ids, 0, nullptr, nullptr);
  return check_launch(op);
}

// ---- generic dispatcher ----------------------------------------------------------------------
static const qx_attribute* find_attr(const qx_kernel_call* c, const char* name) {
  for (size_t i = 0; i < c->attribute_count; ++i)
    if (c->attributes[i].name && std::strcmp(c->attributes[i].name, name) == 0) return &c->attributes[i];
  return nullptr;
}
static int64_t attr_i64(const qx_kernel_call* c, const char* name, int64_t dflt) {
  const qx_attribute* a = find_attr(c, name);
  if (!a) return dflt;
  if (a->kind == QX_ATTR_F64) return (int64_t)a->f64;
  return a->i64;
}
static double attr_f64(const qx_kernel_call* c, const char* name, double dflt) {
  const qx_attribute* a = find_attr(c, name);
  if (!a) return dflt;
  if (a->kind == QX_ATTR_F64) return a->f64;
  return (double)a->i64;
}
static const char* attr_str(const qx_kernel_call* c, const char* name) {
  const qx_attribute* a = find_attr(c, name);
  if (!a || a->kind != QX_ATTR_STRING) return nullptr;
  return (const char*)a->data;
}
static bool contiguous(const qx_tensor_view& t) {
  if (!t.strides) return true;
  int64_t expect = 1;
  for (size_t i = t.rank; i-- > 0;) {
    if (t.shape[i] != 1 && t.strides[i] != expect) return false;
    expect *= t.shape[i];
  }
  return true;
}
static bool present(const qx_kernel_call* c, size_t i) {
  return i < c->input_count && c->inputs[i].data != nullptr;
}

static qx_status lm_head_dims(const qx_kernel_call* call, int64_t* T, int64_t* V, int64_t* K,
                              const char** fmt) {
  static const char* op = "quantized_lm_head_sample";
  if (!call || call->input_count < 2) return fail(QX_INVALID_ARGUMENT, op, "expects inputs h, Wq[, bias]");
  const qx_tensor_view& h = call->inputs[0];
  const qx_tensor_view& w = call->inputs[1];
  if (h.rank != 2 || w.rank != 3) return fail(QX_INVALID_SHAPE, op, "h must be (T, K)");
  *fmt = attr_str(call, "format");
  int bk = 0, bb = 0;
  if (!qx_cuda_format_info(*fmt, &bk, &bb))
    return fail(QX_UNSUPPORTED_FORMAT, op, "format must be q8_0, q4_0, q6_K, mxfp8, nvfp4, or mxfp4");
  *T = h.shape[0]; *K = h.shape[1]; *V = w.shape[0];
  if (w.shape[1] * bk != *K || w.shape[2] != bb)
    return fail(QX_INVALID_SHAPE, op, "packed weight shape does not match V/K/format");
  return ok(op);
}

size_t qx_cuda_workspace_bytes(const char* op_name, const qx_kernel_call* call) {
  if (!op_name || !call) return 0;
  if (std::strcmp(op_name, "quantized_lm_head_sample") == 0) {
    int64_t T, V, K; const char* fmt;
    if (lm_head_dims(call, &T, &V, &K, &fmt).code != QX_OK) return 0;
    const int mode = (int)attr_i64(call, "mode", 0);
    int topk = (int)attr_i64(call, "topk", 0);
    if (mode >= 2 && topk <= 0) topk = 32;
    return qx_cuda_lm_head_workspace_bytes(T, V, K, mode, topk);
  }
  const bool lin = std::strcmp(op_name, "decode_linear_epilogue") == 0;
  const bool glu = std::strcmp(op_name, "decode_swiglu") == 0;
  if ((lin || glu) && call->input_count >= 2 && call->inputs[0].rank == 2 && call->inputs[1].rank == 3)
    return qx_cuda_projection_workspace_bytes(call->inputs[0].shape[0], call->inputs[0].shape[1],
                                              call->inputs[1].shape[0], attr_str(call, "format"),
                                              (qx_dtype)call->inputs[0].dtype, glu ? 1 : 0);
  return 0;
}

qx_status qx_cuda_dispatch(const char* op_name, const qx_kernel_call* call) {
  if (!op_name) return fail(QX_INVALID_ARGUMENT, "dispatch", "null operation name");
  if (!call) return fail(QX_INVALID_ARGUMENT, op_name, "null call");
  for (size_t i = 0; i < call->input_count; ++i) {
    const qx_tensor_view& t = call->inputs[i];
    if (!t.data) continue;
    if (t.memory_space != QX_MEMORY_DEVICE) return fail(QX_UNSUPPORTED_LAYOUT, op_name, "tensors must be in device memory");
    if (!contiguous(t)) return fail(QX_UNSUPPORTED_LAYOUT, op_name, "tensors must be contiguous");
  }
  for (size_t i = 0; i < call->output_count; ++i) {
    const qx_tensor_view& t = call->outputs[i];
    if (!t.data || t.memory_space != QX_MEMORY_DEVICE || !contiguous(t))
      return fail(QX_UNSUPPORTED_LAYOUT, op_name, "outputs must be contiguous device tensors");
  }
  const bool lin = std::strcmp(op_name, "decode_linear_epilogue") == 0;
  const bool glu = std::strcmp(op_name, "decode_swiglu") == 0;
  if (lin || glu) {
    const size_t wcount = glu ? 3 : 2;
    if (call->input_count < wcount || call->output_count < 1)
      return fail(QX_INVALID_ARGUMENT, op_name, "missing inputs or outputs");
    const qx_tensor_view& x = call->inputs[0];
    const qx_tensor_view& w = call->inputs[1];
    if (x.rank != 2) return fail(QX_INVALID_SHAPE, op_name, "x must be non-empty (B,K) fp32/fp16/bf16");
    const char* fmt = attr_str(call, "format");
    int bk = 0, bb = 0;
    if (!qx_cuda_format_info(fmt, &bk, &bb))
      return fail(QX_UNSUPPORTED_FORMAT, op_name, "format must be q4_0, q8_0, q6_K, mxfp8, nvfp4, or mxfp4");
    const int64_t M = x.shape[0], K = x.shape[1];
    if (w.rank != 3 || w.dtype != QX_DTYPE_U8 || K % bk != 0 || w.shape[1] != K / bk || w.shape[2] != bb)
      return fail(QX_INVALID_SHAPE, op_name, "packed weight must be uint8 (N,K/block_k,block_bytes)");
    const int64_t N = w.shape[0];
    const qx_tensor_view& y = call->outputs[0];
    if (y.rank != 2 || y.shape[0] != M || y.shape[1] != N || y.dtype != x.dtype)
      return fail(QX_INVALID_SHAPE, op_name, "output must be (B,N) with x dtype");
    // output_quant attribute ("fp8" / "int8" / "mxfp8"): codes in outputs[1], per-row scales in outputs[2]
    int oq = 0; void* oq_codes = nullptr; float* oq_scale = nullptr;
    if (const char* q = attr_str(call, "output_quant")) {
      oq = std::strcmp(q, "fp8") == 0 ? 1 : std::strcmp(q, "int8") == 0 ? 2 : std::strcmp(q, "mxfp8") == 0 ? 3 : -1;
      if (oq < 0) return fail(QX_INVALID_ARGUMENT, op_name, "output_quant must be None, 'fp8', 'int8', or 'mxfp8'");
      if (call->output_count < (oq == 3 ? 2u : 3u)) return fail(QX_INVALID_ARGUMENT, op_name, "output_quant needs codes (and scale) outputs");
      oq_codes = call->outputs[1].data;
      if (oq != 3) oq_scale = (float*)call->outputs[2].data;
    }
    if (lin) {
      const bool ub = attr_i64(call, "use_bias", present(call, 2)) != 0;
      const bool ur = attr_i64(call, "use_residual", present(call, 3)) != 0;
      if (ub && !(present(call, 2) && call->inputs[2].rank == 1 && call->inputs[2].shape[0] == N && call->inputs[2].dtype == x.dtype))
        return fail(QX_INVALID_SHAPE, op_name, "bias must be (N,) with x dtype");
      if (ur && !(present(call, 3) && call->inputs[3].rank == 2 && call->inputs[3].shape[0] == M && call->inputs[3].shape[1] == N && call->inputs[3].dtype == x.dtype))
        return fail(QX_INVALID_SHAPE, op_name, "residual must be (B,N) with x dtype");
      return qx_cuda_decode_linear_epilogue(call->stream, x.data, w.data, ub ? call->inputs[2].data : nullptr,
                                            ur ? call->inputs[3].data : nullptr, y.data, M, K, N, fmt, (qx_dtype)x.dtype,
                                            (int)attr_i64(call, "activation", 0), ub, ur, oq, oq_codes, oq_scale,
                                            call->workspace, call->workspace_size);
    }
    const qx_tensor_view& u = call->inputs[2];
    if (u.rank != 3 || u.dtype != QX_DTYPE_U8 || u.shape[0] != N || u.shape[1] != w.shape[1] || u.shape[2] != bb)
      return fail(QX_INVALID_SHAPE, op_name, "gate and up weights must have identical shapes");
    const bool ub = attr_i64(call, "use_bias", present(call, 3) && present(call, 4)) != 0;
    if (ub) {
      for (size_t i = 3; i <= 4; ++i)
        if (!(present(call, i) && call->inputs[i].rank == 1 && call->inputs[i].shape[0] == N && call->inputs[i].dtype == x.dtype))
          return fail(QX_INVALID_SHAPE, op_name, "both biases must be (N,) with x dtype");
    }
    return qx_cuda_decode_swiglu(call->stream, x.data, w.data, u.data, ub ? call->inputs[3].data : nullptr,
                                 ub ? call->inputs[4].data : nullptr, y.data, M, K, N, fmt, (qx_dtype)x.dtype, ub,
                                 oq, oq_codes, oq_scale, call->workspace, call->workspace_size);
  }
  if (std::strcmp(op_name, "quantized_lm_head_sample") == 0) {
    int64_t T, V, K; const char* fmt;
    qx_status st = lm_head_dims(call, &T, &V, &K, &fmt);
    if (st.code != QX_OK) return st;
    if (call->output_count < 1 || call->outputs[0].dtype != QX_DTYPE_I32 || call->outputs[0].rank != 1 || call->outputs[0].shape[0] != T)
      return fail(QX_INVALID_SHAPE, op_name, "output must be int32 (T,)");
    const int mode = (int)attr_i64(call, "mode", 0);
    int topk = (int)attr_i64(call, "topk", 0);
    if (mode >= 2 && topk <= 0) topk = 32;
    const float* bias = nullptr;
    if (present(call, 2)) {
      const qx_tensor_view& b = call->inputs[2];
      int64_t n = 1;
      for (size_t i = 0; i < b.rank; ++i) n *= b.shape[i];
      if (n > 1) {   // a 1-element bias is the reference's "no bias" placeholder
        if (b.dtype != QX_DTYPE_F32 || n != V) return fail(QX_INVALID_SHAPE, op_name, "bias must be fp32 (V,)");
        bias = (const float*)b.data;
      }
    }
    return qx_cuda_lm_head_sample_q(call->stream, call->inputs[0].data, call->inputs[1].data, bias,
                                    (int32_t*)call->outputs[0].data, call->workspace, call->workspace_size,
                                    T, V, K, fmt, (qx_dtype)call->inputs[0].dtype, mode, topk,
                                    attr_f64(call, "temperature", 1.0), (uint32_t)attr_i64(call, "seed", 0),
                                    attr_f64(call, "top_p", 0.9));
  }
  const bool q8 = std::strcmp(op_name, "quantize_per_token_fp8") == 0;
  const bool qi = std::strcmp(op_name, "quantize_per_token_int8") == 0;
  if (q8 || qi) {
    if (call->input_count < 1 || call->output_count < 2) return fail(QX_INVALID_ARGUMENT, op_name, "expects x -> (codes, scale)");
    const qx_tensor_view& x = call->inputs[0];
    if (x.rank < 1) return fail(QX_INVALID_SHAPE, op_name, "x must have at least one dimension");
    int64_t rows = 1;
    for (size_t i = 0; i + 1 < x.rank; ++i) rows *= x.shape[i];
    return qx_cuda_quantize_per_token(call->stream, x.data, call->outputs[0].data, (float*)call->outputs[1].data,
                                      rows, x.shape[x.rank - 1], (qx_dtype)x.dtype, qi ? 1 : 0);
  }
  return fail(QX_NOT_IMPLEMENTED, op_name, "operation is not part of the B200 decode-projection backend");
}

// ---- BaseQN separate-plane consumers -----------------------------------------------------------------
// The descriptor checks of the reference (kernels/common/base_q_descriptor.h:34-68), same messages.
static qx_status base_q_desc_of(const char* op, const qx_base_q_desc* d, BaseQDesc* out) {
  if (!d) return fail(QX_INVALID_ARGUMENT, op, "null descriptor");
  const int b = d->bits, g = d->group_size;
  if (b != 2 && b != 3 && b != 4 && b != 5 && b != 6 && b != 8)
    return fail(QX_INVALID_ARGUMENT, op, "BaseQN: bits must be one of 2, 3, 4, 5, 6, or 8");
  if (g != 32 && g != 64 && g != 128) return fail(QX_INVALID_ARGUMENT, op, "BaseQN: group_size must be 32, 64, or 128");
  const std::string sd = d->scale_dtype ? d->scale_dtype : "";
  int stype = -1;
  if (sd == "bf16" || sd == "bfloat16") stype = 0;
  else if (sd == "f16" || sd == "float16") stype = 1;
  else if (sd == "e8m0") stype = 2;
  else if (sd == "e4m3") stype = 3;
  if (stype < 0) return fail(QX_INVALID_ARGUMENT, op, "BaseQN: scale_dtype must be bf16, f16, e8m0, or e4m3");
  if (stype == 3 && b != 8) return fail(QX_INVALID_ARGUMENT, op, "BaseQN: e4m3 scale storage is valid only for q8");
  const std::string lay = d->layout ? d->layout : "";
  if (lay != "metal" && lay != "metal_lane_strided" && lay != "metal_lane_strided_q" + std::to_string(b))
    return fail(QX_INVALID_ARGUMENT, op, "BaseQN: layout must be metal or metal_lane_strided_q<bits>");
  *out = BaseQDesc{b, g, stype, d->symmetric ? 1 : 0};
  return ok(op);
}
static qx_status base_q_planes_ok(const char* op, const qx_base_q_planes* w, const BaseQDesc& d, int64_t rows, int64_t K) {
  if (!w || !w->codes || !w->scales) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (!d.symmetric && !w->biases) return fail(QX_INVALID_ARGUMENT, op, "biases are required for asymmetric BaseQN");
  if (rows <= 0 || K <= 0 || K % d.group != 0 || rows > 0x7fffffff || K > 0x7fffffff)
    return fail(QX_INVALID_SHAPE, op, "codes/scales rows and group count must be positive and match");
  return ok(op);
}

size_t qx_cuda_base_q_workspace_bytes(int64_t K, int64_t M, int64_t V, qx_dtype dtype) {
  if (K <= 0 || M <= 0) return 0;
  size_t n = base_q_scratch_bytes(K, M, dtype, true);
  if (V > 0) n += align256((size_t)M * V * (dtype == QX_DTYPE_F32 ? 4 : 2));
  return n;
}

qx_status qx_cuda_base_qdequant(void* stream, const qx_base_q_planes* w, const qx_base_q_desc* desc, void* out,
                                int64_t rows, int64_t K, qx_dtype out_dtype) {
  static const char* op = "base_qdequant";
  BaseQDesc d;
  qx_status st = base_q_desc_of(op, desc, &d);
  if (st.code != QX_OK) return st;
  if (!float_dtype(out_dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "BaseQN: output_dtype must be float16, bfloat16, or float32");
  st = base_q_planes_ok(op, w, d, rows, K);
  if (st.code != QX_OK) return st;
  if (!out) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (!device_ready(op, &st)) return st;
  launch_base_q_rows((cudaStream_t)stream, d, w->codes, w->scales, w->biases, nullptr, out, rows, rows, K, out_dtype);
  return check_launch(op);
}

qx_status qx_cuda_base_qembedding(void* stream, const qx_base_q_planes* w, const qx_base_q_desc* desc,
                                  const int32_t* ids, void* out, int64_t rows, int64_t K, int64_t tokens,
                                  qx_dtype out_dtype) {
  static const char* op = "base_qembedding";
  BaseQDesc d;
  qx_status st = base_q_desc_of(op, desc, &d);
  if (st.code != QX_OK) return st;
  if (!float_dtype(out_dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "BaseQN: output_dtype must be float16, bfloat16, or float32");
  st = base_q_planes_ok(op, w, d, rows, K);
  if (st.code != QX_OK) return st;
  if (tokens <= 0) return fail(QX_INVALID_SHAPE, op, "ids must be non-empty");
  if (!out || !ids) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (!device_ready(op, &st)) return st;
  launch_base_q_rows((cudaStream_t)stream, d, w->codes, w->scales, w->biases, ids, out, tokens, rows, K, out_dtype);
  return check_launch(op);
}

// shared tail of the multiplying entry points
static qx_status base_q_run(const char* op, void* stream, const BaseQDesc& d, const BaseQMat* mats, int nmat, int mode,
                     const void* x, bool x_is_km, int64_t K, int64_t M, qx_dtype dtype, int64_t orow, int64_t ocol,
                     void* workspace, size_t workspace_bytes, size_t ws_skip, const BaseQExperts* ex) {
  qx_status st;
  if (!device_ready(op, &st)) return st;
  ScratchHold hold;
  void* scratch = nullptr; size_t sbytes = 0;
  const size_t need = ws_skip + base_q_scratch_bytes(K, M, dtype, x_is_km);
  st = bind_scratch(op, (cudaStream_t)stream, need, workspace, workspace_bytes, &hold, &scratch, &sbytes);
  if (st.code != QX_OK) return st;
  if (!launch_base_q_matmul((cudaStream_t)stream, d, mats, nmat, mode, x, x_is_km, K, M, dtype, orow, ocol,
                            scratch ? (char*)scratch + ws_skip : nullptr, scratch ? sbytes - ws_skip : 0, ex))
    return fail(QX_INVALID_SHAPE, op, "no device path for this shape (expert stacks: 16-bit input, K % 128 == 0, K >= 512, 16-byte aligned planes)");
  return check_launch(op);
}

qx_status qx_cuda_base_qgemm(void* stream, const qx_base_q_planes* w, const qx_base_q_desc* desc, const void* x,
                             void* out, int64_t rows, int64_t K, int64_t M, qx_dtype dtype, void* workspace,
                             size_t workspace_bytes) {
  const char* op = M == 1 ? "base_qgemv" : "base_qgemm";
  BaseQDesc d;
  qx_status st = base_q_desc_of(op, desc, &d);
  if (st.code != QX_OK) return st;
  st = base_q_planes_ok(op, w, d, rows, K);
  if (st.code != QX_OK) return st;
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "BaseQN matmul: x must be float16, bfloat16, or float32");
  if (M <= 0 || M > 0x7fffffff) return fail(QX_INVALID_SHAPE, op, "BaseQN matmul: M must be positive");
  if (!x || !out) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  BaseQMat m{w->codes, w->scales, w->biases, rows, out};
  return base_q_run(op, stream, d, &m, 1, 0, x, true, K, M, dtype, M, 1, workspace, workspace_bytes, 0, nullptr);
}

qx_status qx_cuda_base_qgemv_qkv(void* stream, const qx_base_q_planes* q, const qx_base_q_planes* k,
                                 const qx_base_q_planes* v, const qx_base_q_desc* desc, const void* x, void* q_out,
                                 void* k_out, void* v_out, int64_t q_rows, int64_t k_rows, int64_t v_rows,
                                 int64_t K, qx_dtype dtype, void* workspace, size_t workspace_bytes) {
  static const char* op = "base_qgemv_qkv";
  BaseQDesc d;
  qx_status st = base_q_desc_of(op, desc, &d);
  if (st.code != QX_OK) return st;
  const qx_base_q_planes* w[3] = {q, k, v};
  const int64_t rows[3] = {q_rows, k_rows, v_rows};
  void* outs[3] = {q_out, k_out, v_out};
  BaseQMat m[3];
  for (int i = 0; i < 3; ++i) {
    st = base_q_planes_ok(op, w[i], d, rows[i], K);
    if (st.code != QX_OK) return st;
    if (!outs[i]) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
    m[i] = BaseQMat{w[i]->codes, w[i]->scales, w[i]->biases, rows[i], outs[i]};
  }
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "BaseQN matmul: x must be float16, bfloat16, or float32");
  if (!x) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  return base_q_run(op, stream, d, m, 3, 0, x, true, K, 1, dtype, 1, 1, workspace, workspace_bytes, 0, nullptr);
}

qx_status qx_cuda_base_qgemv_swiglu(void* stream, const qx_base_q_planes* gate, const qx_base_q_planes* up,
                                    const qx_base_q_desc* desc, const void* x, void* out, int64_t rows, int64_t K,
                                    qx_dtype dtype, void* workspace, size_t workspace_bytes) {
  static const char* op = "base_qgemv_swiglu";
  BaseQDesc d;
  qx_status st = base_q_desc_of(op, desc, &d);
  if (st.code != QX_OK) return st;
  st = base_q_planes_ok(op, gate, d, rows, K);
  if (st.code != QX_OK) return st;
  st = base_q_planes_ok(op, up, d, rows, K);
  if (st.code != QX_OK) return st;
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "BaseQN matmul: x must be float16, bfloat16, or float32");
  if (!x || !out) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  BaseQMat m[2] = {{gate->codes, gate->scales, gate->biases, rows, out}, {up->codes, up->scales, up->biases, rows, out}};
  return base_q_run(op, stream, d, m, 2, 1, x, true, K, 1, dtype, 1, 1, workspace, workspace_bytes, 0, nullptr);
}

qx_status qx_cuda_base_qlm_head_argmax(void* stream, const qx_base_q_planes* w, const qx_base_q_desc* desc,
                                       const void* x, int32_t* ids, int64_t V, int64_t K, int64_t batch,
                                       qx_dtype dtype, void* workspace, size_t workspace_bytes) {
  static const char* op = "base_qlm_head_argmax";
  BaseQDesc d;
  qx_status st = base_q_desc_of(op, desc, &d);
  if (st.code != QX_OK) return st;
  st = base_q_planes_ok(op, w, d, V, K);
  if (st.code != QX_OK) return st;
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "BaseQN matmul: x must be float16, bfloat16, or float32");
  if (batch <= 0 || batch > 0x7fffffff) return fail(QX_INVALID_SHAPE, op, "base_qlm_head_argmax: x must be non-empty (K, batch)");
  if (!x || !ids) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (!device_ready(op, &st)) return st;
  // logits (batch, V) in the dtype of x at the head of the workspace, then the row-wise argmax
  const size_t logit_bytes = align256((size_t)batch * V * (dtype == QX_DTYPE_F32 ? 4 : 2));
  ScratchHold hold;
  void* scratch = nullptr; size_t sbytes = 0;
  st = bind_scratch(op, (cudaStream_t)stream, logit_bytes + base_q_scratch_bytes(K, batch, dtype, true), workspace,
                    workspace_bytes, &hold, &scratch, &sbytes);
  if (st.code != QX_OK) return st;
  BaseQMat m{w->codes, w->scales, w->biases, V, scratch};
  if (!launch_base_q_matmul((cudaStream_t)stream, d, &m, 1, 0, x, true, K, batch, dtype, 1, V,
                            (char*)scratch + logit_bytes, sbytes - logit_bytes, nullptr))
    return fail(QX_RUNTIME_ERROR, op, "kernel configuration failed");
  launch_sample_logits((cudaStream_t)stream, scratch, ids, batch, V, dtype, 0, 0, 1.f, 1.f, 0u);
  return check_launch(op);
}

qx_status qx_cuda_base_qmoe(void* stream, const qx_base_q_planes* w, const qx_base_q_desc* desc, const void* input,
                            const int32_t* expert_of_tile, void* out, int64_t experts, int64_t expert_rows,
                            int64_t K, int64_t total_rows, int swiglu, qx_dtype dtype, void* workspace,
                            size_t workspace_bytes) {
  const char* op = swiglu ? "base_qmoe_swiglu" : "base_qmoe_gemm";
  BaseQDesc d;
  qx_status st = base_q_desc_of(op, desc, &d);
  if (st.code != QX_OK) return st;
  if (experts <= 0 || experts * expert_rows > 0x7fffffff)
    return fail(QX_INVALID_SHAPE, op, "codes/scales expert, row, and group dimensions must be positive and match");
  st = base_q_planes_ok(op, w, d, expert_rows, K);
  if (st.code != QX_OK) return st;
  if (dtype != QX_DTYPE_F16 && dtype != QX_DTYPE_BF16) return fail(QX_UNSUPPORTED_DTYPE, op, "input must be float16 or bfloat16");
  if (total_rows <= 0 || total_rows % 32 != 0 || total_rows > 0x7fffffff)
    return fail(QX_INVALID_SHAPE, op, "input rows must be a positive multiple of 32");
  if (swiglu && expert_rows % 2 != 0) return fail(QX_INVALID_SHAPE, op, "the gate/up row axis must be even");
  if (!input || !expert_of_tile || !out) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  const int64_t I = swiglu ? expert_rows / 2 : expert_rows;
  BaseQExperts ex{expert_of_tile, experts, expert_rows, swiglu ? I : 0};
  BaseQMat m[2] = {{w->codes, w->scales, w->biases, I, out}, {w->codes, w->scales, w->biases, I, out}};
  return base_q_run(op, stream, d, m, swiglu ? 2 : 1, swiglu ? 1 : 0, input, false, K, total_rows, dtype, 1, I,
                    workspace, workspace_bytes, 0, &ex);
}

// ---- peer exchange ---------------------------------------------------------------------------------------
qx_status qx_cuda_peer_push(void* stream, const void* src, size_t bytes, void* const* peer_dst,
                            void* const* peer_flags, int world, int self, int step, void* tickets) {
  static const char* op = "peer_push";
  if (!src || !peer_dst || !peer_flags || !tickets) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (world < 1 || world > 16 || self < 0 || self >= world) return fail(QX_INVALID_ARGUMENT, op, "world must be 1..16 and self a rank of it");
  if (bytes == 0 || bytes % 16 != 0) return fail(QX_INVALID_SHAPE, op, "bytes must be a positive multiple of 16");
  qx_status st;
  if (!device_ready(op, &st)) return st;
  if (!launch_peer_push((cudaStream_t)stream, src, bytes, peer_dst, peer_flags, world, self, step, (unsigned*)tickets))
    return fail(QX_INVALID_ARGUMENT, op, "source and peer destinations must be 16-byte aligned, flags non-null");
  return check_launch(op);
}

qx_status qx_cuda_peer_wait(void* stream, const void* flags, int world, int self, int step, int timeout_ms,
                            int32_t* status) {
  static const char* op = "peer_wait";
  if (!flags || !status) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (world < 1 || world > 16 || self < 0 || self >= world) return fail(QX_INVALID_ARGUMENT, op, "world must be 1..16 and self a rank of it");
  if (timeout_ms < 1 || timeout_ms > 10000) return fail(QX_INVALID_ARGUMENT, op, "timeout_ms must be 1..10000");
  qx_status st;
  if (!device_ready(op, &st)) return st;
  // one poll = a volatile load + nanosleep(200): about 0.3 us
  launch_peer_wait((cudaStream_t)stream, (const int*)flags, world, self, step, timeout_ms * 3000, status);
  return check_launch(op);
}

qx_status qx_cuda_peer_gather(void* stream, float* gather, int64_t slot_floats, void* const* peer_words, int world,
                              int self, int step, int timeout_ms, int32_t* status) {
  static const char* op = "peer_gather";
  if (!gather || !peer_words || !status) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (world < 1 || world > 16 || self < 0 || self >= world) return fail(QX_INVALID_ARGUMENT, op, "world must be 1..16, self in [0, world)");
  if (slot_floats <= 0 || slot_floats % 2 != 0) return fail(QX_INVALID_SHAPE, op, "slot_floats must be a positive even number");
  if (timeout_ms < 1 || timeout_ms > 10000) return fail(QX_INVALID_ARGUMENT, op, "timeout_ms must be 1..10000");
  qx_status st;
  if (!device_ready(op, &st)) return st;
  int* sp = status;
  if (!launch_peer_gather((cudaStream_t)stream, &gather, (size_t)slot_floats, peer_words, world, self, 1, step, &sp, timeout_ms * 1000))
    return fail(QX_INVALID_ARGUMENT, op, "gather must be 8-byte aligned, every word buffer 16-byte aligned");
  return check_launch(op);
}

qx_status qx_cuda_peer_gather_local(void* stream, float* const* gather, int64_t slot_floats, void* const* peer_words,
                                    int world, int step, int timeout_ms, int32_t* const* status) {
  static const char* op = "peer_gather_local";
  if (!gather || !peer_words || !status) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (world < 1 || world > 16) return fail(QX_INVALID_ARGUMENT, op, "world must be 1..16");
  if (slot_floats <= 0 || slot_floats % 2 != 0) return fail(QX_INVALID_SHAPE, op, "slot_floats must be a positive even number");
  if (timeout_ms < 1 || timeout_ms > 10000) return fail(QX_INVALID_ARGUMENT, op, "timeout_ms must be 1..10000");
  qx_status st;
  if (!device_ready(op, &st)) return st;
  if (!launch_peer_gather((cudaStream_t)stream, gather, (size_t)slot_floats, peer_words, world, 0, world, step,
                          (int* const*)status, timeout_ms * 1000))
    return fail(QX_INVALID_ARGUMENT, op, "null / misaligned buffers, or the cooperative launch was refused");
  return check_launch(op);
}

qx_status qx_cuda_lm_head_sample_sharded(void* stream, const void* h, const void* wq, const float* bias_local,
                                         int32_t* ids, float* gather, int64_t slot_stride, void* const* peer_gather,
                                         void* const* peer_flags, const void* flags, void* tickets,
                                         void* const* peer_words, int32_t* status,
                                         int world, int self, int step, int timeout_ms, void* workspace,
                                         size_t workspace_bytes, int64_t T, int64_t V_local, int64_t K,
                                         int64_t vocab_offset, int64_t max_tiles, const char* format, qx_dtype dtype,
                                         int mode, int topk, double temperature, uint32_t seed, double top_p) {
  static const char* op = "quantized_lm_head_sample.sharded";
  if (!gather || !ids) return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (world < 1 || world > 16 || self < 0 || self >= world) return fail(QX_INVALID_ARGUMENT, op, "world must be 1..16 and self a rank of it");
  const int kk = mode >= 2 ? topk : 1;
  const int64_t C = qx_cuda_lm_head_shard_candidates(mode, kk, max_tiles);
  const int64_t Ls = mode == 3 ? max_tiles : 0;
  const int64_t per = T * (2 * C + Ls);
  if (slot_stride < per || slot_stride % 4 != 0) return fail(QX_INVALID_SHAPE, op, "slot_stride must be a multiple of 4 floats and hold T * (2C + L)");
  float* mine = gather + (size_t)self * slot_stride;
  qx_status st = qx_cuda_lm_head_shard_partials_q(stream, h, wq, bias_local, mine, (int32_t*)(mine + T * C),
                                                  Ls ? mine + 2 * T * C : nullptr, workspace, workspace_bytes, T, V_local,
                                                  K, vocab_offset, max_tiles, format, dtype, mode, topk, temperature, seed);
  if (st.code != QX_OK) return st;
  if (world > 1 && peer_words) {
    st = qx_cuda_peer_gather(stream, gather, slot_stride, peer_words, world, self, step, timeout_ms, status);
    if (st.code != QX_OK) return st;
  } else if (world > 1) {
    st = qx_cuda_peer_push(stream, mine, (size_t)slot_stride * 4, peer_gather, peer_flags, world, self, step, tickets);
    if (st.code != QX_OK) return st;
    st = qx_cuda_peer_wait(stream, flags, world, self, step, timeout_ms, status);
    if (st.code != QX_OK) return st;
  }
  return qx_cuda_lm_head_shard_reduce(stream, gather, (const int32_t*)(gather + T * C), Ls ? gather + 2 * T * C : nullptr, ids,
                                      world, T, max_tiles, world > 1 ? slot_stride : 0, mode, topk, temperature, seed, top_p);
}

qx_status qx_cuda_peer_allreduce(void* stream, const float* src, const void* residual, void* out, int64_t n,
                                 void* const* peer_bufs, int world, int self, void* counter, void* tickets,
                                 int32_t* status, qx_dtype dtype, int timeout_ms) {
  static const char* op = "peer_allreduce";
  if (!src || !residual || !out || !peer_bufs || !counter || !tickets || !status)
    return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (world < 1 || world > 16 || self < 0 || self >= world) return fail(QX_INVALID_ARGUMENT, op, "world must be 1..16, self in [0, world)");
  if (n <= 0 || n % 2 != 0) return fail(QX_INVALID_SHAPE, op, "n must be a positive even number");
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "residual / out must be fp32, fp16 or bf16");
  if (timeout_ms < 1 || timeout_ms > 10000) return fail(QX_INVALID_ARGUMENT, op, "timeout_ms must be 1..10000");
  qx_status st;
  if (!device_ready(op, &st)) return st;
  int* c = (int*)counter; unsigned* t = (unsigned*)tickets; int* sp = status;
  if (!launch_peer_allreduce((cudaStream_t)stream, &src, &residual, &out, (size_t)n, peer_bufs, world, self, 1,
                             &c, &t, &sp, dtype, timeout_ms * 1000))
    return fail(QX_INVALID_ARGUMENT, op, "src must be 8-byte aligned, every buffer 16-byte aligned");
  return check_launch(op);
}

qx_status qx_cuda_peer_allreduce_local(void* stream, const float* const* src, const void* const* residual, void* const* out,
                                       int64_t n, void* const* peer_bufs, int world, void* const* counter,
                                       void* const* tickets, int32_t* const* status, qx_dtype dtype, int timeout_ms) {
  static const char* op = "peer_allreduce_local";
  if (!src || !residual || !out || !peer_bufs || !counter || !tickets || !status)
    return fail(QX_INVALID_ARGUMENT, op, "null pointer");
  if (world < 1 || world > 16) return fail(QX_INVALID_ARGUMENT, op, "world must be 1..16");
  if (n <= 0 || n % 2 != 0) return fail(QX_INVALID_SHAPE, op, "n must be a positive even number");
  if (!float_dtype(dtype)) return fail(QX_UNSUPPORTED_DTYPE, op, "residual / out must be fp32, fp16 or bf16");
  if (timeout_ms < 1 || timeout_ms > 10000) return fail(QX_INVALID_ARGUMENT, op, "timeout_ms must be 1..10000");
  qx_status st;
  if (!device_ready(op, &st)) return st;
  if (!launch_peer_allreduce((cudaStream_t)stream, src, residual, out, (size_t)n, peer_bufs, world, 0, world,
                             (int* const*)counter, (unsigned* const*)tickets, (int* const*)status, dtype, timeout_ms * 1000))
    return fail(QX_INVALID_ARGUMENT, op, "null / misaligned buffers, or the cooperative launch was refused");
  return check_launch(op);
}

}  // extern "C"
