// Internal launch interface between the C ABI / dispatch layer and the kernel translation units.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/quixicore_cuda.h"

namespace qx {

// One decode projection (w1 == nullptr) or a gate/up SwiGLU pair (w1 != nullptr).
struct GemvArgs {
  const void* x; const void* w0; const void* w1;
  const void* bias0; const void* bias1; const void* residual;
  void* y;
  int64_t M, K, N;
  int format;          // qx::Format
  qx_dtype dtype;      // F32 / F16 / BF16
  int activation, use_bias, use_residual;
  int out_f32 = 0;     // 1: y is fp32 (M,N) raw dot products, no bias / activation / residual
};

void launch_gemv_generic(cudaStream_t st, const GemvArgs& a);
// Streaming tensor-core path (bf16 activations, batch <= 16, 16-byte aligned bases).
bool stream_path_ok(const GemvArgs& a);
bool launch_gemv_stream(cudaStream_t st, const GemvArgs& a);
// The same kernel in passes of 16 rows for batches of 17 - 64 rows, when that beats the tcgen05 path.
bool stream_passes_ok(const GemvArgs& a);
bool launch_gemv_stream_passes(cudaStream_t st, const GemvArgs& a);
// tcgen05 path (bf16 activations, batch > 16, K % 256 == 0, single weight matrix).
bool tc_path_ok(const GemvArgs& a);
bool launch_gemm_tc(cudaStream_t st, const GemvArgs& a);
// Value of the device-side error flag that bounded waits raise (synchronises the device).
int read_device_error_flag();
// Device address of that flag on the current device (nullptr if it cannot be resolved).
int* device_error_flag();
// Device scratch of at least `bytes` for work enqueued on `st` (see qx_gemv_stream.cu); when
// *must_free is set the caller releases it with cudaFreeAsync on the same stream.
void* stream_scratch(cudaStream_t st, size_t bytes, bool* must_free);
// Row-scaled f16 copy of (M,K) bf16 / f16 activations in the column order `perm` of the decoders.
// silu(gate + gb) * (up + ub) over fp32 (M,N) projections -> T (M,N)
void launch_swiglu_combine(cudaStream_t st, const float* gate, const float* up, const void* gb,
                           const void* ub, void* y, int64_t M, int64_t N, qx_dtype dtype, int use_bias);
void launch_prep_activations(cudaStream_t st, const void* x, qx_dtype dtype, __half* x16,
                             float* rowscale, int M, int K, int perm, int img_rows = 0);
// Picks the kernel family for one projection call (format, dtype, batch, alignment).
void launch_projection(cudaStream_t st, const GemvArgs& a);

// Fused LM head.  Stage 1 writes per-256-row-tile partials, stage 2 merges them.
struct LmHeadArgs {
  const void* h; const void* wq; const float* bias;   // bias: fp32 (V_local,) or nullptr
  int64_t T, V, K;                                    // V = rows held by this call
  int64_t vocab_offset;                               // global id of local row 0
  int format; qx_dtype dtype;
  int mode, topk;
  float invtemp; uint32_t seed; float top_p;
};
// part_val/part_id: (T, tiles_stride, kk) with kk = 1 (modes 0/1) or topk; part_lse: (T, tiles_stride)
void launch_lm_head_partials(cudaStream_t st, const LmHeadArgs& a, float* part_val,
                             int32_t* part_id, float* part_lse, int64_t tiles_stride);
// ncand candidates per row and shard at cand_val/cand_id (+ nlse tile lses, mode 3).
// emit_set = 0: write the sampled id per row to ids.  emit_set = 1: write the selected candidate
// set ((val,id) x set_size per row, absent = id -1) to out_val/out_id instead (modes 0..2).
// Candidates are laid out (shards, T, ncand) and lses (shards, T, nlse); with shard_stride > 0 the
// three arrays instead advance by shard_stride elements from one shard to the next.
void launch_lm_head_reduce(cudaStream_t st, const float* cand_val, const int32_t* cand_id,
                           const float* cand_lse, int shards, int64_t T, int64_t ncand,
                           int64_t nlse, int64_t shard_stride, int mode, int topk, float invtemp,
                           uint32_t seed, float top_p, int32_t* ids, int emit_set, float* out_val,
                           int32_t* out_id);

void launch_quantize_per_token(cudaStream_t st, const void* x, void* codes, float* scale,
                               int64_t rows, int64_t D, qx_dtype dtype, int kind);
void launch_quantize_mxfp8_rows(cudaStream_t st, const void* x, void* blocks, int64_t rows,
                                int64_t D, qx_dtype dtype);

}  // namespace qx
