/*
 * quixicore_cuda.h - C ABI of the B200 (sm_100a) backend for the QuixiCore quantized
 * decode-projection path: decode_linear_epilogue, decode_swiglu, fused lm_head_sample and the
 * runtime output quantizers.
 *
 * Plain C: pointers, sizes and PODs only.  No exception crosses this boundary; every entry point
 * returns a qx_status whose `operation` / `detail` strings are static (never freed by the caller).
 * All device pointers must belong to the CUDA device that is current on the calling thread.
 * Work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = the legacy default
 * stream) and no entry point synchronises the host, so results are valid after the caller
 * synchronises that stream.  There is no CPU fallback: without a usable CUDA device the calls
 * return QX_RUNTIME_ERROR.
 *
 * Each declaration cites the reference interface it stands in for (path:line inside the
 * QuixiCore-Metal project).  The reference has no C binding of its own (bindings/c is empty);
 * the generic call structs have the memory layout of its cross-backend contract header
 * include/quixicore/contract/kernel_abi.hpp:10-107: the same fields in the same order, and the
 * enumerations stored in one byte as there (`enum class ... : std::uint8_t`), so that
 * sizeof / offsetof agree (qx_tensor_view 40 bytes, dtype at 32, memory_space at 33, flags at 36;
 * qx_attribute 48 bytes; qx_kernel_call 80 bytes; qx_status 24 bytes) and a
 * quixicore::contract::KernelCall can be handed over by pointer.  The enum TYPES below are what
 * the typed entry points take as parameters; the structs store the same constants in the
 * one-byte typedefs qx_status_code_u8 / qx_dtype_u8 / qx_memory_space_u8 / qx_attribute_kind_u8.
 */
#ifndef QUIXICORE_CUDA_H
#define QUIXICORE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status (kernel_abi.hpp:10-31) ---------------------------------------------------------- */
typedef enum qx_status_code {
  QX_OK = 0,
  QX_INVALID_ARGUMENT,
  QX_INVALID_SHAPE,
  QX_UNSUPPORTED_DTYPE,
  QX_UNSUPPORTED_FORMAT,
  QX_UNSUPPORTED_LAYOUT,
  QX_INSUFFICIENT_WORKSPACE,
  QX_ADAPTER_NOT_WIRED,
  QX_NOT_IMPLEMENTED,
  QX_RUNTIME_ERROR
} qx_status_code;

typedef uint8_t qx_status_code_u8; /* a qx_status_code constant in the contract's 1-byte storage */

typedef struct qx_status {
  qx_status_code_u8 code;
  const char* operation;
  const char* detail;
} qx_status;

/* ---- element types (kernel_abi.hpp:33-51) ---------------------------------------------------- */
typedef enum qx_dtype {
  QX_DTYPE_UNKNOWN = 0, QX_DTYPE_BOOL, QX_DTYPE_I8, QX_DTYPE_U8, QX_DTYPE_I16, QX_DTYPE_U16,
  QX_DTYPE_I32, QX_DTYPE_U32, QX_DTYPE_I64, QX_DTYPE_U64, QX_DTYPE_F16, QX_DTYPE_BF16,
  QX_DTYPE_F32, QX_DTYPE_F64, QX_DTYPE_E4M3, QX_DTYPE_E5M2, QX_DTYPE_PACKED
} qx_dtype;

typedef enum qx_memory_space {
  QX_MEMORY_UNKNOWN = 0, QX_MEMORY_HOST, QX_MEMORY_DEVICE, QX_MEMORY_SHARED
} qx_memory_space;

typedef uint8_t qx_dtype_u8;
typedef uint8_t qx_memory_space_u8;

enum { QX_TENSOR_NONE = 0, QX_TENSOR_READ_ONLY = 1, QX_TENSOR_CONTIGUOUS = 2, QX_TENSOR_OPTIONAL = 4 };

/* ---- generic call (kernel_abi.hpp:66-107) ---------------------------------------------------- */
typedef struct qx_tensor_view {
  void* data;
  const int64_t* shape;
  const int64_t* strides; /* in elements; NULL = contiguous row-major */
  size_t rank;
  qx_dtype_u8 dtype;
  qx_memory_space_u8 memory_space;
  uint32_t flags;
} qx_tensor_view;

typedef enum qx_attribute_kind {
  QX_ATTR_BOOL = 0, QX_ATTR_I64, QX_ATTR_F64, QX_ATTR_STRING, QX_ATTR_BYTES
} qx_attribute_kind;

typedef uint8_t qx_attribute_kind_u8;

typedef struct qx_attribute {
  const char* name;
  qx_attribute_kind_u8 kind;
  const void* data; /* string / bytes payload */
  size_t size;
  int64_t i64;      /* bool / i64 payload */
  double f64;
} qx_attribute;

typedef struct qx_kernel_call {
  const qx_tensor_view* inputs;
  size_t input_count;
  qx_tensor_view* outputs;
  size_t output_count;
  const qx_attribute* attributes;
  size_t attribute_count;
  void* backend_context; /* unused, must be NULL */
  void* stream;          /* cudaStream_t */
  void* workspace;       /* device scratch, see qx_cuda_workspace_bytes */
  size_t workspace_size;
} qx_kernel_call;

/*
 * Generic dispatcher: the slot the reference's
 * quixicore::metal::contract_api::dispatch(OperationId, const KernelCall&)
 * (include/quixicore/metal/contract.hpp:12-16) leaves as `not_implemented`.
 * op_name is the contract's operation name (include/quixicore/contract/operations.hpp:72-75,232):
 *   "decode_linear_epilogue"   inputs x, weight, bias, residual      outputs y
 *   "decode_swiglu"            inputs x, gate_w, up_w, gate_b, up_b  outputs y
 *   "quantized_lm_head_sample" inputs h, Wq, bias                    outputs ids(i32)
 *   "quantize_per_token_fp8" / "quantize_per_token_int8"  inputs x   outputs codes, scale
 * Attribute names equal the Python keyword names of the reference API: format, activation,
 * use_bias, use_residual, mode, topk, temperature, seed, top_p.  Unknown op -> QX_NOT_IMPLEMENTED.
 */
qx_status qx_cuda_dispatch(const char* op_name, const qx_kernel_call* call);

/* Scratch bytes `call->workspace` should provide for op_name with these shapes (0 for ops without
 * scratch).  Counterpart of the partial buffers the reference host code allocates itself
 * (bindings/pytorch_mps/tk_torch/torch_kernels.mm:5071-5073, :5093-5094).  The LM head requires
 * that workspace; the projection ops fall back to the library's own scratch (see "Workspace"
 * below) when call->workspace is NULL. */
size_t qx_cuda_workspace_bytes(const char* op_name, const qx_kernel_call* call);

/* ---- typed entry points ----------------------------------------------------------------------
 * dtype: QX_DTYPE_F32 / QX_DTYPE_F16 / QX_DTYPE_BF16 = element type of x, bias, residual, y.
 * format: "q4_0" "q8_0" "q6_K" "mxfp8" "nvfp4" "mxfp4"; weight = uint8 (N, K/block_k, block_bytes)
 * contiguous, K % block_k == 0.  activation: 0 none, 1 erf-GELU (Abramowitz-Stegun), 2 SiLU.
 *
 * Output quantisation (`output_quant` of tk.decode_linear_epilogue / decode_swiglu,
 * bindings/python/tk/__init__.py:3684-3691): out_quant selects what is written besides y, on the
 * values of y as rounded to dtype:
 *   QX_OUT_QUANT_NONE   nothing
 *   QX_OUT_QUANT_FP8    out_codes uint8 (M,N) e4m3, out_scale f32 (M,) = amax/448   (quant_rt.metal:21-53)
 *   QX_OUT_QUANT_INT8   out_codes int8 (M,N),       out_scale f32 (M,) = amax/127   (quant_rt.metal:55-87)
 *   QX_OUT_QUANT_MXFP8  out_codes uint8 (M, N/32, 33) packed MXFP8 rows, N % 32 == 0; out_scale unused.
 *                       An extension: the reference router only knows the first two.  For bf16 /
 *                       f16 calls that take the streaming or tcgen05 kernels the blocks are packed
 *                       by the projection kernel itself; every other case is a second launch inside
 *                       the call.
 *
 * Workspace.  The bf16 / f16 kernels keep a row-scaled f16 copy of the activations in device
 * scratch.  Pass `workspace` (256-byte aligned, at least qx_cuda_projection_workspace_bytes) and the
 * call allocates nothing, frees nothing and never synchronises: it may then be captured in a CUDA
 * graph and replayed on any stream.  With workspace == NULL the library uses a buffer of its own per
 * (device, stream): the first call on a stream, and a call that needs more than any before it,
 * run cudaMalloc (which synchronises the device and is not allowed while another thread captures
 * in global mode); smaller buffers are kept until exit, nothing is freed or waited for.  Calls on
 * cudaStreamPerThread, on a stream that is being captured, or on more than 16 distinct streams
 * use cudaMallocAsync / cudaFreeAsync per call instead.  Too small a non-NULL workspace fails with
 * QX_INSUFFICIENT_WORKSPACE.
 */
enum { QX_OUT_QUANT_NONE = 0, QX_OUT_QUANT_FP8 = 1, QX_OUT_QUANT_INT8 = 2, QX_OUT_QUANT_MXFP8 = 3 };

/* Upper bound of the scratch one projection call uses (swiglu != 0: the gate/up pair); 0 when the
 * shape takes a kernel without scratch (fp32 activations). */
size_t qx_cuda_projection_workspace_bytes(int64_t M, int64_t K, int64_t N, const char* format,
                                          qx_dtype dtype, int swiglu);

/* y[m,n] = T( act( dot(x[m,:], deq(W[n,:])) + bias[n] ) + residual[m,n] ), fp32 math, one rounding.
 * Replaces decode_linear_epilogue_mps (torch_kernels.mm:6407-6435) and
 * tk::launch_decode_linear_epilogue (kernels/common/tk_launch.h:444-456). bias / residual are
 * ignored (may be NULL) when their flag is 0. */
qx_status qx_cuda_decode_linear_epilogue(void* stream, const void* x, const void* weight,
                                         const void* bias, const void* residual, void* y,
                                         int64_t M, int64_t K, int64_t N, const char* format,
                                         qx_dtype dtype, int activation, int use_bias,
                                         int use_residual, int out_quant, void* out_codes,
                                         float* out_scale, void* workspace, size_t workspace_bytes);

/* y[m,n] = dot(x[m,:], deq(W[n,:])) as fp32, no epilogue: the per-rank piece of a row-parallel
 * (K-split) projection, to be summed over ranks before bias / activation / residual are applied
 * once.  No counterpart in the reference (single device).  Needs bf16 / f16 activations, 16-byte
 * aligned bases and K a multiple of 512; otherwise QX_UNSUPPORTED_LAYOUT. */
qx_status qx_cuda_decode_linear_partial(void* stream, const void* x, const void* weight, float* y,
                                        int64_t M, int64_t K, int64_t N, const char* format,
                                        qx_dtype dtype, void* workspace, size_t workspace_bytes);

/* y[m,n] = T( silu(gate.x + gb) * (up.x + ub) ).  Replaces decode_swiglu_mps
 * (torch_kernels.mm:6437-6466) and tk::launch_decode_swiglu (tk_launch.h:458-470). */
qx_status qx_cuda_decode_swiglu(void* stream, const void* x, const void* gate_weight,
                                const void* up_weight, const void* gate_bias, const void* up_bias,
                                void* y, int64_t M, int64_t K, int64_t N, const char* format,
                                qx_dtype dtype, int use_bias, int out_quant, void* out_codes,
                                float* out_scale, void* workspace, size_t workspace_bytes);

/* Per-row dynamic quantisation of x (rows, D): scale[row] = amax/448 (fp8, e4m3 codes, halves
 * round away from zero, saturating at 448) or amax/127 (int8).  Replaces
 * quantize_per_token_fp8 / _int8 (kernels/quantization/quant_rt/quant_rt.metal:21-87,
 * tk_launch.h:1449-1468, tk_torch/__init__.py:1738-1745). kind: 0 = fp8, 1 = int8. */
qx_status qx_cuda_quantize_per_token(void* stream, const void* x, void* codes, float* scale,
                                     int64_t rows, int64_t D, qx_dtype dtype, int kind);

/* x (rows, D), D % 32 == 0 -> MXFP8 blocks (rows, D/32, 33) = {e8m0 exponent; 32 e4m3 codes},
 * scale = 2^ceil(log2(amax/448)).  The rule of quantize_per_group_fp8 with G = 32, ue8m0 = 1
 * (quant_rt.metal:266-306) emitted in the packed mxfp8 block layout
 * (include/metal/ops/warp/register/tile/dequant.metal:422-429). */
qx_status qx_cuda_quantize_mxfp8_rows(void* stream, const void* x, void* blocks, int64_t rows,
                                      int64_t D, qx_dtype dtype);

/* ---- fused LM head ---------------------------------------------------------------------------
 * mode: 0 argmax, 1 categorical, 2 top-k, 3 top-p.  topk in [1,64] for modes 2/3.  bias is fp32
 * (V,) or NULL.  seed is the 32-bit RNG key; the noise stream is the reference's stateless hash
 * keyed by (seed, row, global vocab id) (include/metal/common/rng.metal:18-30).
 */

/* Scratch bytes for qx_cuda_lm_head_sample_q: the per-tile partials of stage 1, the prepared
 * hidden rows and the exchange slots of vocabulary tiles that several thread blocks share.  The
 * workspace must be 256-byte aligned.  With it the call allocates nothing and never synchronises. */
size_t qx_cuda_lm_head_workspace_bytes(int64_t T, int64_t V, int64_t K, int mode, int topk);

/* ids[t] = sampled token for row t of h (T,K); logits are never written to memory.  Replaces
 * lm_head_sample_q_mps (torch_kernels.mm:5019-5101) = partial + reduce launches
 * (tk_launch.h:2836-2871, :2952-3013). */
qx_status qx_cuda_lm_head_sample_q(void* stream, const void* h, const void* wq, const float* bias,
                                   int32_t* ids, void* workspace, size_t workspace_bytes, int64_t T,
                                   int64_t V, int64_t K, const char* format, qx_dtype dtype,
                                   int mode, int topk, double temperature, uint32_t seed,
                                   double top_p);

/* No counterpart in the reference (whose host code always allocates its partial buffers): the
 * same operation as qx_cuda_lm_head_sample_q for callers that cannot allocate device memory at
 * call time - code running inside a latency-critical serving loop that has handed all of its
 * memory to a pool, a plugin host that forbids cudaMalloc after start-up, or a region that is
 * being stream-ordered without an allocator.  All global scratch of the two stages (per-tile
 * partials, the prepared hidden rows and their row scales, the flags and exchange slots of shared
 * tiles) is carved out of a fixed array of QX_CUDA_LM_HEAD_STATIC_SCRATCH_BYTES bytes that is part
 * of the library image (every GPU that loads the library keeps that much memory until the process
 * exits).  A call needs  2 * align256(4 * T * tiles * kk)  [+ align256(4 * T * tiles) for top-p]
 * + 1024 + align256(2 * roundup(T, 64) * K) + align256(4 * T)  bytes of it, tiles = ceil(V / 256),
 * kk = topk for modes 2 / 3 and 1 otherwise; a call that needs more fails with
 * QX_INSUFFICIENT_WORKSPACE.  Nothing in this call allocates or frees, for any dtype of h.  The
 * first call on each device looks the array's device address up once; make that first call before
 * starting any stream capture.  All calls on one device share the array: two calls that overlap
 * on the GPU (different streams) race on it, so keep them on one stream or order them with
 * events.  Stage 1 overwrites every slot that stage 2 reads and the flags are cleared by the call
 * itself, so nothing has to be cleared between calls. */
#define QX_CUDA_LM_HEAD_STATIC_SCRATCH_BYTES (4u << 20)
qx_status qx_cuda_lm_head_sample_q_noalloc(void* stream, const void* h, const void* wq,
                                           const float* bias, int32_t* ids, int64_t T, int64_t V,
                                           int64_t K, const char* format, qx_dtype dtype, int mode,
                                           int topk, double temperature, uint32_t seed,
                                           double top_p);

/* The same over a dense head W (V,K) in the dtype of h, modes 0..2; logits are never written.
 * Replaces lm_head_sample_mps (torch_kernels.mm:4966-5016; kernels lm_head.metal:175-235,
 * :400-470).  bias fp32 (V,) or NULL. */
size_t qx_cuda_lm_head_dense_workspace_bytes(int64_t T, int64_t V, int mode, int topk);
qx_status qx_cuda_lm_head_sample_dense(void* stream, const void* h, const void* W, const float* bias,
                                       int32_t* ids, void* workspace, size_t workspace_bytes,
                                       int64_t T, int64_t V, int64_t K, qx_dtype dtype, int mode,
                                       int topk, double temperature, uint32_t seed);

/* Samplers over materialised logits (rows, V): kind 0 argmax (raw logits), 1 categorical, 2 top-k
 * (k <= 64), 3 top-p; ids int32 (rows,).  The noise row index is the row of the call.  Replaces
 * argmax_sample / sample_categorical / top_k_sample / top_p_sample
 * (kernels/sampling/sampling/sampling.metal:19-103, :159-217; tk_torch/__init__.py:1620-1637). */
qx_status qx_cuda_sample_logits(void* stream, const void* logits, int32_t* ids, int64_t rows, int64_t V,
                                qx_dtype dtype, int kind, int topk, double top_p, double temperature,
                                uint32_t seed);

/* ---- the operators either side of the path ----------------------------------------------------- */

/* out (N, M) = dequantise(wq) (N, K) @ x (K, M), x / out in `dtype` (float16 in the reference; M == 1
 * is qgemv, where float32 is accepted as well).  The activation matrix is column-major per token as
 * in the reference; the call transposes it into the row layout of the projection kernels and the
 * result back, inside the workspace.  Exact fp32 dequantisation and accumulation, one rounding.
 * Replaces qgemv_mps / qgemm_mps (torch_kernels.mm:5616-5640, :5682-5712; qgemv.metal:13-45,
 * qgemm.metal:11-50), without their N % 32 / M % 32 restrictions. */
size_t qx_cuda_qgemm_workspace_bytes(int64_t N, int64_t K, int64_t M, const char* format, qx_dtype dtype);
qx_status qx_cuda_qgemm(void* stream, const void* wq, const void* x, void* out, int64_t N, int64_t K,
                        int64_t M, const char* format, qx_dtype dtype, void* workspace,
                        size_t workspace_bytes);

/* Packed embedding lookup: out (tokens, columns) = T(dequantise(table[ids[t]]) * scale (+ add[t])),
 * fp32 arithmetic, one rounding; ids outside [0, rows) give all-zero rows and ignore `add`.
 * table uint8 (rows, columns/block_k, block_bytes), ids int32 (tokens,), add / out in out_dtype.
 * Replaces dequant_gather_mps / quantized_embedding_mps (torch_kernels.mm:6468-6546;
 * dequant_gather.metal:10-105) for the six formats of this backend. */
qx_status qx_cuda_quantized_embedding(void* stream, const void* table, const int32_t* ids, const void* add,
                                      void* out, int64_t rows, int64_t columns, int64_t tokens,
                                      const char* format, double scale, int use_add, qx_dtype out_dtype);

/* ---- norm / activation -> quantiser seams ------------------------------------------------------
 * What feeds quantised activations into a projection.  fp32 arithmetic on the I/O-dtype inputs.
 * quant: 0 none, 1 fp8 static per tensor, 2 fp8 dynamic per row (scale = amax/448), 3 int8 dynamic
 * per row (amax/127), 4 fp8 per block of `group` columns, 5 int8 per block; ue8m0 != 0 rounds the
 * fp8 block scales up to powers of two.  e4m3 codes round halves away from zero and saturate at 448.
 */

/* res_out = T(x + residual); n = rms_norm(x + residual) * weight on the unrounded fp32 sum;
 * quant 0: y = T(n); otherwise codes (rows, D) of n and, for quant >= 2, scale (rows,) or
 * (rows, D / group).  Replaces rms_norm_add / rms_norm_add_fp8 / _fp8_dyn / _int8_dyn /
 * rms_norm_add_per_block (kernels/norms/add_norm/add_norm.metal:26-65, :181-392), for any D up to
 * 51200 and f32 / f16 / bf16 (the Metal kernels: bf16, D in a fixed list). */
qx_status qx_cuda_rms_norm_add(void* stream, const void* x, const void* residual, const void* weight, void* y,
                               void* codes, void* res_out, float* scale, int64_t rows, int64_t D, qx_dtype dtype,
                               double eps, int quant, double static_scale, int group, int ue8m0);

/* codes = quantise(act(x, gate)) without the (rows, D) intermediate: act 0 = silu(x) * gate, 1 = the
 * clamped variant x' = min(x, limit), g' = clamp(gate, +-limit), x' * sigmoid(alpha x') * (1 + g').
 * quant 2 / 3 / 4 as above (group % 4 == 0).  Replaces silu_mul_quant_fp8 / _int8 / _fp8_group
 * (kernels/quantization/act_quant/act_quant.metal:26-160). */
qx_status qx_cuda_silu_mul_quant(void* stream, const void* x, const void* gate, void* codes, float* scale,
                                 int64_t rows, int64_t D, qx_dtype dtype, int act, double alpha, double limit,
                                 int quant, int group, int ue8m0);

/* ---- LM-head forms that return log-probabilities ------------------------------------------------
 * format NULL or "" = dense W (V,K) in the dtype of h; otherwise a packed head.  Raw logits (no
 * temperature); ordering: logit descending, ties to the smaller token id; bias fp32 (V,) or NULL.
 */

/* Top-k (k <= 8) of the tokens admitted by a per-row bit mask, with log-probabilities.
 * allow_mask: uint32 (T, ceil(V/32)), bit (v & 31) of word v >> 5 admits token v.  ids / logprobs
 * (T, topk): ids sorted best first, logprob = logit - log-sum-exp over the admitted tokens
 * (normalize_allowed != 0) or over the whole vocabulary; missing entries id -1 / -inf.
 * Replaces lm_head_masked_mps (torch_kernels.mm:6655-6698; lm_head.metal:1152-1304). */
size_t qx_cuda_lm_head_masked_workspace_bytes(int64_t T, int64_t V, int64_t K, int topk);
qx_status qx_cuda_lm_head_masked(void* stream, const void* h, const void* w, const float* bias,
                                 const uint32_t* allow_mask, int32_t* ids, float* logprobs, void* workspace,
                                 size_t workspace_bytes, int64_t T, int64_t V, int64_t K, const char* format,
                                 qx_dtype dtype, int topk, int normalize_allowed);

/* Projects only the tokens listed per row in CSR form (candidate_ids flat int32, offsets int32
 * (T+1,), `entries` = offsets[T]; ids outside [0, V) are skipped; ids within a row must be unique)
 * and returns their top-k (k <= 8) with log-probabilities normalised over the listed tokens.
 * workspace: one float per entry.  Replaces lm_head_candidates_mps (torch_kernels.mm:6700-6731;
 * lm_head.metal:1339-1425). */
qx_status qx_cuda_lm_head_candidates(void* stream, const void* h, const void* w, const float* bias,
                                     const int32_t* candidate_ids, const int32_t* offsets, int64_t entries,
                                     int32_t* ids, float* logprobs, void* workspace, size_t workspace_bytes,
                                     int64_t T, int64_t V, int64_t K, const char* format, qx_dtype dtype,
                                     int topk);

/* One beam-search step over a packed head without logits in memory: h (B*BM, K), cum_log_probs
 * fp32 (B, BM) -> next_token, parent_beam int32 (B, BM), new_cum fp32 (B, BM): per batch the BM best
 * of (cum[beam] + log_softmax(logits[beam])[token]), ties to the lower (beam, rank) index.
 * BM <= 16, V >= 2 BM; q4_0 / q8_0 / mxfp8 / nvfp4 / mxfp4.  Replaces lm_head_beam_advance_mps
 * (torch_kernels.mm:5105-5172; lm_head.metal:534-573, sampling.metal:432-458). */
size_t qx_cuda_lm_head_beam_workspace_bytes(int64_t rows, int64_t V, int64_t K, int beam_width);
qx_status qx_cuda_lm_head_beam_advance(void* stream, const void* h, const void* wq, const float* bias,
                                       const float* cum_log_probs, int32_t* next_token, int32_t* parent_beam,
                                       float* new_cum, void* workspace, size_t workspace_bytes, int64_t batches,
                                       int beam_width, int64_t V, int64_t K, const char* format, qx_dtype dtype);

/* Vocabulary-sharded form.  A shard holds rows [vocab_offset, vocab_offset + V_local) of the full
 * matrix, vocab_offset a multiple of 256 so every 256-row tile of the reference lies in one shard.
 * Stage 1 writes this shard's candidates for every row t:
 *   cand_val / cand_id  (T, C) with C = qx_cuda_lm_head_shard_candidates(...); absent slots carry
 *                       id -1; ids are GLOBAL vocab ids
 *   cand_lse            (T, L) per-tile log-sum-exp (mode 3 only, L = tiles of the largest shard;
 *                       absent tiles carry -FLT_MAX)
 * After an all-gather over shards into (S, T, C) / (S, T, L) buffers (shard_stride = 0), or into
 * one buffer per shard laid end to end in which the three arrays sit at fixed offsets and the
 * shards are shard_stride elements apart (the all-gather output as it is), stage 2 picks the tokens.
 * The merges (max with lowest id, top-k of top-k, sum of exp) are associative, so the result
 * equals the single-device call on the same logits.  The reference has no multi-device code; the
 * split follows its own two-stage tile -> reduce structure (lm_head.metal:219-235, :444-529).
 */
int64_t qx_cuda_lm_head_shard_candidates(int mode, int topk, int64_t max_tiles);
size_t qx_cuda_lm_head_shard_workspace_bytes(int64_t T, int64_t V_local, int64_t K, int mode, int topk);

qx_status qx_cuda_lm_head_shard_partials_q(void* stream, const void* h, const void* wq,
                                           const float* bias_local, float* cand_val,
                                           int32_t* cand_id, float* cand_lse, void* workspace,
                                           size_t workspace_bytes, int64_t T, int64_t V_local,
                                           int64_t K, int64_t vocab_offset, int64_t max_tiles,
                                           const char* format, qx_dtype dtype, int mode, int topk,
                                           double temperature, uint32_t seed);

qx_status qx_cuda_lm_head_shard_reduce(void* stream, const float* cand_val, const int32_t* cand_id,
                                       const float* cand_lse, int32_t* ids, int64_t shards,
                                       int64_t T, int64_t max_tiles, int64_t shard_stride,
                                       int mode, int topk, double temperature, uint32_t seed,
                                       double top_p);

/* ---- BaseQN: weights as separate code / scale / bias planes -----------------------------------------
 * codes uint8 (rows, K * bits / 8), lane c of a row in bits [c * bits, (c + 1) * bits) of the row's
 * little-endian bit string; scales and (asymmetric tensors) biases (rows, K / group) stored as
 * scale_dtype "bf16" / "f16" (2 bytes) or "e8m0" / "e4m3" (1 byte; e4m3 only with bits == 8).
 * w = fl(fl(code * scale) + bias); symmetric != 0: w = (code - 2^(bits - 1)) * scale, biases ignored
 * (may be NULL).  bits in {2,3,4,5,6,8}, group in {32,64,128}, layout "metal", "metal_lane_strided"
 * or "metal_lane_strided_q<bits>" (one layout, three spellings).  Contract:
 * kernels/quantization/base_q/README.md:8-27, descriptor checks kernels/common/base_q_descriptor.h:34-68,
 * storage checks kernels/quantization/base_q/base_q.cpp:57-90.  Activations / outputs f32, f16 or
 * bf16; 16-bit activations with K % 128 == 0, K >= 512 run on the streaming tensor-core kernel and
 * need the workspace below, everything else on a shape-generic kernel.  workspace NULL = library
 * scratch. */
typedef struct qx_base_q_planes {
  const void* codes;
  const void* scales;
  const void* biases;
} qx_base_q_planes;
typedef struct qx_base_q_desc {
  int32_t bits;
  int32_t group_size;
  const char* scale_dtype;
  int32_t symmetric;
  const char* layout;
} qx_base_q_desc;

/* Workspace of the BaseQN calls that multiply: K inner dimension, M activation columns (batch;
 * total_rows for the expert forms), V = vocabulary rows for base_qlm_head_argmax (its logits live
 * in the workspace), else 0. */
size_t qx_cuda_base_q_workspace_bytes(int64_t K, int64_t M, int64_t V, qx_dtype dtype);

/* out (rows, K) = dequantised weights.  Replaces base_qdequant (base_q.cpp:170-187, base_q.metal:71-91). */
qx_status qx_cuda_base_qdequant(void* stream, const qx_base_q_planes* w, const qx_base_q_desc* desc, void* out,
                                int64_t rows, int64_t K, qx_dtype out_dtype);
/* out (tokens, K) = rows ids[i] of the dequantised table; an id outside [0, rows) gives a zero row.
 * Replaces base_qembedding (base_q.cpp:279-300, base_q.metal:251-280). */
qx_status qx_cuda_base_qembedding(void* stream, const qx_base_q_planes* w, const qx_base_q_desc* desc,
                                  const int32_t* ids, void* out, int64_t rows, int64_t K, int64_t tokens,
                                  qx_dtype out_dtype);
/* out (rows, M) = dequant(W) (rows, K) @ x (K, M), in the dtype of x.  M == 1 is base_qgemv.
 * Replaces base_qgemv / base_qgemm (base_q.cpp:134-212, base_q.metal:93-115,222-249). */
qx_status qx_cuda_base_qgemm(void* stream, const qx_base_q_planes* w, const qx_base_q_desc* desc, const void* x,
                             void* out, int64_t rows, int64_t K, int64_t M, qx_dtype dtype, void* workspace,
                             size_t workspace_bytes);
/* q / k / v (rows_i, 1) = dequant(W_i) @ x (K, 1) for three matrices that share desc and K, one launch.
 * Replaces base_qgemv_qkv (base_q.cpp:214-251, base_q.metal:117-163). */
qx_status qx_cuda_base_qgemv_qkv(void* stream, const qx_base_q_planes* q, const qx_base_q_planes* k,
                                 const qx_base_q_planes* v, const qx_base_q_desc* desc, const void* x, void* q_out,
                                 void* k_out, void* v_out, int64_t q_rows, int64_t k_rows, int64_t v_rows,
                                 int64_t K, qx_dtype dtype, void* workspace, size_t workspace_bytes);
/* out (rows, 1) = silu(W_gate @ x) * (W_up @ x), rounded once.  Replaces base_qgemv_swiglu
 * (base_q.cpp:253-277, base_q.metal:165-220). */
qx_status qx_cuda_base_qgemv_swiglu(void* stream, const qx_base_q_planes* gate, const qx_base_q_planes* up,
                                    const qx_base_q_desc* desc, const void* x, void* out, int64_t rows, int64_t K,
                                    qx_dtype dtype, void* workspace, size_t workspace_bytes);
/* ids (batch,) = argmax over the V logits of every column of x (K, batch); logits are rounded to the
 * dtype of x first, the smaller id wins an exact tie.  Replaces base_qlm_head_argmax
 * (bindings/python/tk/__init__.py:4033-4059, README.md:43-47). */
qx_status qx_cuda_base_qlm_head_argmax(void* stream, const qx_base_q_planes* w, const qx_base_q_desc* desc,
                                       const void* x, int32_t* ids, int64_t V, int64_t K, int64_t batch,
                                       qx_dtype dtype, void* workspace, size_t workspace_bytes);
/* Expert stack: codes (experts, expert_rows, K * bits / 8), scales / biases (experts, expert_rows,
 * K / group); input (total_rows, K); expert_of_tile (total_rows / 32,) names the expert of every 32
 * input rows, a negative entry leaves those output rows untouched.  swiglu == 0: out (total_rows,
 * expert_rows) = input @ dequant(W[e])^T.  swiglu != 0: expert_rows = 2 * I laid out [gate(I), up(I)],
 * out (total_rows, I) = silu(gate) * up.  Replaces base_qmoe_gemm / base_qmoe_swiglu
 * (base_q.cpp:302-375, base_q.metal:313-430).  16-bit input, K % 128 == 0, K >= 512. */
qx_status qx_cuda_base_qmoe(void* stream, const qx_base_q_planes* w, const qx_base_q_desc* desc, const void* input,
                            const int32_t* expert_of_tile, void* out, int64_t experts, int64_t expert_rows,
                            int64_t K, int64_t total_rows, int swiglu, qx_dtype dtype, void* workspace,
                            size_t workspace_bytes);

/* ---- exchange of per-shard candidates by peer stores (no reference counterpart) -----------------------
 * For hosts whose ranks share a symmetric allocation (the same buffer layout on every GPU, each rank
 * holding device pointers to every peer's copy): qx_cuda_peer_push copies `bytes` (a multiple of 16)
 * from src (this rank's slot of its own buffer) to peer_dst[r] for every r != self with plain peer
 * stores, then writes `step` to ((int*)peer_flags[r])[self] on every peer, data before flag
 * (system-scope fences).  tickets: one zero-initialised device word owned by the caller.
 * qx_cuda_peer_wait enqueues a one-warp kernel that waits until flags[r] - step >= 0 for every
 * r != self; the wait is bounded (timeout_ms): when it runs out the kernel writes 1 to *status (a device
 * int the caller zeroed) and returns, so a missing peer never hangs the GPU.  world <= 16.
 * Buffers must alternate between two halves by step parity (a peer may be one step ahead, never two
 * while every rank enqueues push(n), wait(n), consumer(n) in that order on one stream). */
qx_status qx_cuda_peer_push(void* stream, const void* src, size_t bytes, void* const* peer_dst,
                            void* const* peer_flags, int world, int self, int step, void* tickets);
qx_status qx_cuda_peer_wait(void* stream, const void* flags, int world, int self, int step, int timeout_ms,
                            int32_t* status);

/* All-reduce of fp32 partial sums (row-parallel projections) over peer stores with the residual add and
 * the cast fused, as ONE launch, flag-in-data (what the tensor-parallel projection stack uses for
 * decode-sized partials).  Every rank owns a zero-initialised symmetric buffer of 2 * world * (n / 2)
 * 16-byte words = 16 * world * n bytes (two halves by step parity, one slot per rank); a word is
 * {x, step, y, step}: two floats, each beside the step number, so that the receiver polls the data itself
 * and nothing else (no flag array, no fence) crosses NVLink.  The step is *counter + 1 (device int,
 * zero-initialised, local; stored back by the last CTA: replayable from a CUDA graph).  A thread stores
 * its elements of src (n floats, n even) into slot [step & 1][self] of every rank's buffer (peer_bufs[r] =
 * rank r's buffer base, this rank's included), reads slot [step & 1][r] of its own buffer for r = 0 ..
 * world - 1 in that order - bounded polls, about timeout_ms; on expiry *status = 1, the call carries on
 * with invalid sums and later calls on that status word do not wait - and writes
 * out[i] = T(sum over r + residual[i]): the same order on every rank, so all ranks hold identical
 * results.  n must be the same on every rank.  Replaces (Python) `dist.all_reduce(partial); out = (partial +
 * residual).to(dtype)` after the row-parallel projections of a decoder block.
 * qx_cuda_peer_allreduce_local runs all `world` ranks, whose buffers all live on the current device, as
 * one cooperative launch (arrays of `world` pointers per argument): ranks that wait for one another
 * cannot be separate launches on one GPU. */
qx_status qx_cuda_peer_allreduce(void* stream, const float* src, const void* residual, void* out, int64_t n,
                                 void* const* peer_bufs, int world, int self, void* counter, void* tickets,
                                 int32_t* status, qx_dtype dtype, int timeout_ms);
qx_status qx_cuda_peer_allreduce_local(void* stream, const float* const* src, const void* const* residual,
                                       void* const* out, int64_t n, void* const* peer_bufs, int world,
                                       void* const* counter, void* const* tickets, int32_t* const* status,
                                       qx_dtype dtype, int timeout_ms);

/* All-gather of small slots as ONE launch, flag-in-data: the latency form of qx_cuda_peer_push +
 * qx_cuda_peer_wait for slots of a few KB.  `gather` is LOCAL memory of world slots of slot_floats floats
 * (slot_floats even) whose slot [self] is filled; peer_words[r] = base of rank r's zero-initialised
 * symmetric word buffer of 2 * world * (slot_floats / 2) 16-byte words {x, step, y, step} (two halves by
 * step parity, one slot per sending rank).  A thread sends its pair of floats to every peer's word buffer,
 * then polls its own word buffer for the same pair of every peer (bounded, about timeout_ms; on expiry
 * *status = 1, the call carries on and later calls on that status word do not wait) and writes it into
 * slot [r] of `gather`.  `step` must grow by one per exchange on every rank.  Replaces (Python)
 * `dist.all_gather_into_tensor`.  qx_cuda_peer_gather_local: all `world` ranks on the current device as one
 * cooperative launch (gather / status: arrays of `world` pointers). */
qx_status qx_cuda_peer_gather(void* stream, float* gather, int64_t slot_floats, void* const* peer_words, int world,
                              int self, int step, int timeout_ms, int32_t* status);
qx_status qx_cuda_peer_gather_local(void* stream, float* const* gather, int64_t slot_floats, void* const* peer_words,
                                    int world, int step, int timeout_ms, int32_t* const* status);

/* One call for a rank's whole step of the vocabulary-parallel LM head over the peer exchange:
 * qx_cuda_lm_head_shard_partials_q into this rank's slot of `gather` (slots are slot_stride floats
 * apart, slot_stride a multiple of 4 and at least T * (2C + L)), then the exchange, then
 * qx_cuda_lm_head_shard_reduce over the world slots.  Exchange with peer_words == NULL:
 * qx_cuda_peer_push of the slot to peer_gather[r] (each peer's address of the SAME slot) and
 * qx_cuda_peer_wait; `gather` is then the half of the symmetric buffer that belongs to this step's
 * parity.  With peer_words: qx_cuda_peer_gather (small slots; peer_gather / peer_flags / flags /
 * tickets are not used). */
qx_status qx_cuda_lm_head_sample_sharded(void* stream, const void* h, const void* wq, const float* bias_local,
                                         int32_t* ids, float* gather, int64_t slot_stride, void* const* peer_gather,
                                         void* const* peer_flags, const void* flags, void* tickets,
                                         void* const* peer_words, int32_t* status,
                                         int world, int self, int step, int timeout_ms, void* workspace,
                                         size_t workspace_bytes, int64_t T, int64_t V_local, int64_t K,
                                         int64_t vocab_offset, int64_t max_tiles, const char* format, qx_dtype dtype,
                                         int mode, int topk, double temperature, uint32_t seed, double top_p);

/* ---- introspection --------------------------------------------------------------------------- */
/* block_k / block_bytes of a format name; returns 0 and leaves the outputs alone if unknown
 * (the table of kernels/matmul/decode_linear/decode_linear.cpp:25-34). */
int qx_cuda_format_info(const char* format, int* block_k, int* block_bytes);
/* Number of kernel launches this library has enqueued since it was loaded. */
uint64_t qx_cuda_launch_count(void);
/* 0 while every bounded device-side wait of this library has completed; non-zero once a kernel
 * gave up waiting for one of its own asynchronous copies (its results are then invalid).
 * Synchronises the device.  -1 if the flag cannot be read.  No counterpart in the reference. */
int qx_cuda_device_error(void);
/* Chooses between device paths that compute the same result (identical up to fp32 summation
 * order); meant for tests and A/B timing.  Names: "stream_passes" (0 never / 1 when faster / 2
 * whenever possible: 17 - 64 rows as passes (32 rows; 16 for a SwiGLU pair) of the streaming kernel instead of the tcgen05
 * pipeline), "force_generic", "tc_pipeline", "lm_head_ksplit" (0 / 1).  Returns
 * 1 if the option exists and took the value.  Process-wide, not synchronised with running calls. */
int qx_cuda_set_option(const char* name, int value);
/* Number of device allocations the library has made for scratch of its own (calls that passed
 * no workspace).  Stays unchanged across calls that bring a workspace and across
 * qx_cuda_lm_head_sample_q_noalloc. */
uint64_t qx_cuda_scratch_alloc_count(void);
/* Library version string, e.g. "quixicore-b200 0.2 (sm_100a)". */
const char* qx_cuda_version(void);

#ifdef __cplusplus
}
#endif
#endif /* QUIXICORE_CUDA_H */
