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
  // Output requantisation fused behind the epilogue: 0 none, 1 per-token fp8, 2 per-token int8,
  // 3 MXFP8 rows (N % 32 == 0).  q_codes receives the codes / packed blocks, q_scale the per-row
  // scales (kinds 1 and 2).  y is written in every case (the codes are defined on its rounded values).
  int out_quant = 0;
  void* q_codes = nullptr;
  float* q_scale = nullptr;
  // Device scratch of at least projection_scratch_bytes(*this) bytes, 256-byte aligned.
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
};

enum OutQuant : int { OQ_NONE = 0, OQ_FP8 = 1, OQ_INT8 = 2, OQ_MXFP8 = 3 };

// Switches between device paths that compute the same result (identical up to fp32 summation
// order).  Defaults are the measured-fastest choices; qx_cuda_set_option changes them.
struct Options {
  int stream_passes = 1;        // 17 - 64 rows as passes of the streaming kernel: 0 never, 1 when faster, 2 whenever possible
  bool force_generic = false;   // keep every call on the shape-generic kernels
  bool tc_pipeline = true;      // batch > 16 on the tcgen05 pipeline
  bool lm_head_ksplit = true;   // share the items of a partial round over K between CTAs
};
const Options& options();
bool set_option(const char* name, int value);

// Scratch for a call that brought no workspace (see qx_scratch.cu); *must_free: cudaFreeAsync on st.
void* default_scratch(cudaStream_t st, size_t bytes, bool* must_free);
uint64_t scratch_alloc_count();

void launch_gemv_generic(cudaStream_t st, const GemvArgs& a);
// Streaming tensor-core path (bf16 activations, batch <= 16, 16-byte aligned bases).
bool stream_path_ok(const GemvArgs& a);
bool launch_gemv_stream(cudaStream_t st, const GemvArgs& a);
// The same kernel in passes of 32 / 16 rows for batches of 17 - 64 rows, when that beats the tcgen05 path.
bool stream_passes_ok(const GemvArgs& a);
bool launch_gemv_stream_passes(cudaStream_t st, const GemvArgs& a);
// tcgen05 path (bf16 activations, batch > 16, K % 256 == 0, single weight matrix).
bool tc_path_ok(const GemvArgs& a);
// *fused_quant (optional): set when the kernel that ran packed the requested MXFP8 output rows itself
bool launch_gemm_tc(cudaStream_t st, const GemvArgs& a, bool* fused_quant = nullptr);
// Value of the device-side error flag that bounded waits raise (synchronises the device).
int read_device_error_flag();
// Device address of that flag on the current device (nullptr if it cannot be resolved).
int* device_error_flag();
// Scratch bytes each path family needs for this call (0 when the family cannot take it).
size_t stream_scratch_bytes(const GemvArgs& a);
size_t tc_scratch_bytes(const GemvArgs& a);
size_t projection_scratch_bytes(const GemvArgs& a);
// Row-scaled f16 copy of (M,K) bf16 / f16 activations in the column order `perm` of the decoders.
// silu(gate + gb) * (up + ub) over fp32 (M,N) projections -> T (M,N)
void launch_swiglu_combine(cudaStream_t st, const float* gate, const float* up, const void* gb,
                           const void* ub, void* y, int64_t M, int64_t N, qx_dtype dtype, int use_bias);
void launch_prep_activations(cudaStream_t st, const void* x, qx_dtype dtype, __half* x16,
                             float* rowscale, int M, int K, int perm, int img_rows = 0);
// Picks the kernel family for one projection call (format, dtype, batch, alignment); true when the
// kernel that ran also wrote the requested MXFP8 output rows.
bool launch_projection(cudaStream_t st, const GemvArgs& a);

// Per-row allow mask of lm_head_masked: bit (v & 31) of word bits[t * words + (v >> 5)] admits global
// vocabulary id v for hidden row t; norm_allowed: the log-sum-exp runs over admitted ids only.
struct LmhMask { const uint32_t* bits; long long words; int norm_allowed; };

// Fused LM head.  Stage 1 writes per-256-row-tile partials, stage 2 merges them.
struct LmHeadArgs {
  const void* h; const void* wq; const float* bias;   // bias: fp32 (V_local,) or nullptr
  int64_t T, V, K;                                    // V = rows held by this call
  int64_t vocab_offset;                               // global id of local row 0
  int format; qx_dtype dtype;
  int mode, topk;                                     // mode 4: masked top-k (mask below), raw logits
  float invtemp; uint32_t seed; float top_p;
  LmhMask mask = LmhMask{nullptr, 0, 1};
  // Device scratch of at least lm_head_scratch_bytes(T, K) bytes (prepared activations, row scales,
  // the release flags and - as far as it reaches - the exchange slots of K-split items).
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
};
// Minimum scratch of stage 1 (without exchange slots: items are then not shared) and the size
// with which every sharing choice fits.
size_t lm_head_scratch_min_bytes(int64_t T, int64_t K);
size_t lm_head_scratch_full_bytes(int64_t T, int64_t K);
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

// qx_cuda_lm_head_sample_q on a caller-chosen region [partials | stage-1 scratch] (see qx_capi.cu).
qx_status lm_head_sample_on(const char* op, void* stream, const void* h, const void* wq, const float* bias,
                            int32_t* ids, void* workspace, size_t workspace_bytes, bool min_only, int64_t T,
                            int64_t V, int64_t K, const char* format, qx_dtype dtype, int mode, int topk,
                            double temperature, uint32_t seed, double top_p);

// Stage 1 over a dense (V, K) head in h's dtype (modes 0..2); partials as in the packed form.
void launch_lm_head_dense_partials(cudaStream_t st, const void* h, const void* W, const float* bias,
                                   float* part_val, int32_t* part_id, int64_t T, int64_t V, int64_t K,
                                   qx_dtype dtype, int mode, int topk, float invtemp, uint32_t seed,
                                   float* part_lse = nullptr, const LmhMask mask = LmhMask{nullptr, 0, 1});
// Samplers over materialised logits (rows, V): kind 0 argmax, 1 categorical, 2 top-k, 3 top-p.
void launch_sample_logits(cudaStream_t st, const void* logits, int32_t* ids, int64_t rows, int64_t V,
                          qx_dtype dtype, int kind, int topk, float p, float invtemp, uint32_t seed);

// Sorted top-k ids with scores (cum + value - log-sum-exp) per row: see qx_lm_head_topk.cu.
void launch_lm_head_topk_logprob(cudaStream_t st, const float* val, const int32_t* id, const int32_t* offsets,
                                 int64_t per_row, const float* lse, int64_t nlse, const float* cum, int64_t rows,
                                 int64_t V, int topk, int32_t* out_id, float* out_score);
// logit[e] = dot(h[row of e], W[cand[e]]) (+ bias) for every CSR entry e with 0 <= cand[e] < V; format < 0: dense W.
void launch_lm_head_candidate_logits(cudaStream_t st, int format, qx_dtype dtype, const void* h, const void* w,
                                     const float* bias, const int32_t* cand, const int32_t* offsets, float* logit,
                                     int64_t rows, int64_t V, int64_t K, int64_t entries);
void launch_beam_select(cudaStream_t st, const float* cand_score, const int32_t* cand_token, int32_t* next_token,
                        int32_t* parent_beam, float* new_cum, int64_t batches, int BM, int two_bm);

// Packed embedding lookup: out (tokens, columns) = T(dequant(table[ids]) * scale (+ add)); see qx_gather.cu.
void launch_quantized_embedding(cudaStream_t st, int format, qx_dtype out_dtype, const void* table, const int32_t* ids,
                                const void* add, void* out, int64_t rows, int64_t columns, int64_t tokens, float scale,
                                int use_add);
// out (C, R) = in (R, C)^T for 2- or 4-byte elements.
void launch_transpose(cudaStream_t st, const void* in, void* out, int64_t R, int64_t C, size_t elem_bytes);

// Residual add + RMSNorm with optional quantising tail, gated activation to codes: see qx_seams.cu.
// qmode: 0 none, 1 fp8 static, 2 fp8 per row, 3 int8 per row, 4 fp8 per group, 5 int8 per group.
bool launch_rms_norm_add(cudaStream_t st, qx_dtype dtype, const void* x, const void* residual, const void* weight,
                         void* y, void* codes, void* res_out, float* scale, int64_t rows, int64_t D, float eps,
                         int qmode, float inv_static, int G, int pow2);
bool launch_silu_mul_quant(cudaStream_t st, qx_dtype dtype, const void* x, const void* gate, void* codes, float* scale,
                           int64_t rows, int64_t D, int act, float alpha, float limit, int qmode, int G, int pow2);

// BaseQN separate-plane weights (see qx_base_q.cu).  stype: 0 bf16, 1 f16, 2 e8m0, 3 e4m3.
struct BaseQDesc { int bits, group, stype, symmetric; };
struct BaseQMat { const void* codes; const void* scales; const void* biases; int64_t rows; void* out; };
// Expert stack: activation row m belongs to expert expert_of_tile[m / 32]; an expert holds expert_rows
// plane rows, the second matrix of a gate / up pair starts up_offset rows into them.
struct BaseQExperts { const int32_t* expert_of_tile; int64_t experts, expert_rows, up_offset; };
size_t base_q_scratch_bytes(int64_t K, int64_t M, qx_dtype dtype, bool x_is_km);
bool launch_base_q_matmul(cudaStream_t st, const BaseQDesc& d, const BaseQMat* mats, int nmat, int mode,
                          const void* x, bool x_is_km, int64_t K, int64_t M, qx_dtype dtype, int64_t orow,
                          int64_t ocol, void* scratch, size_t scratch_bytes, const BaseQExperts* ex = nullptr);
void launch_base_q_rows(cudaStream_t st, const BaseQDesc& d, const void* codes, const void* scales,
                        const void* biases, const int32_t* ids, void* out, int64_t out_rows, int64_t rows,
                        int64_t K, qx_dtype out_dtype);

// Peer exchange of a gather-buffer slot by plain peer stores, and the bounded wait for the peers' flags
// (see qx_peer.cu).
bool launch_peer_push(cudaStream_t st, const void* src, size_t bytes, void* const* peer_dst, void* const* peer_flags,
                      int world, int self, int step, unsigned* tickets);
void launch_peer_wait(cudaStream_t st, const int* flags, int world, int self, int step, int max_polls, int* status);
// All-reduce of fp32 partials over peer stores with the residual add and the cast fused into the consumer.
bool launch_peer_gather(cudaStream_t st, float* const* gather, size_t slot_floats, void* const* peer_words, int world,
                        int self, int local_ranks, int step, int* const* status, int max_polls);
bool launch_peer_allreduce(cudaStream_t st, const float* const* src, const void* const* residual, void* const* out,
                           size_t n, void* const* peer_bufs, int world, int self, int local_ranks,
                           int* const* counter, unsigned* const* tickets, int* const* status, qx_dtype dtype,
                           int max_polls);

void launch_quantize_per_token(cudaStream_t st, const void* x, void* codes, float* scale,
                               int64_t rows, int64_t D, qx_dtype dtype, int kind);
void launch_quantize_mxfp8_rows(cudaStream_t st, const void* x, void* blocks, int64_t rows,
                                int64_t D, qx_dtype dtype);

}  // namespace qx
