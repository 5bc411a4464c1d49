// lm_head_sample for callers that must not allocate: every byte of global scratch the two stages
// use (partials, prepared hidden rows, row scales, flags, exchange slots) lives in a fixed device
// array that is part of this library's image instead of a caller-provided workspace.
#include <mutex>

#include "qx_common.cuh"
#include "qx_kernels.h"

namespace qx {

constexpr size_t kStaticScratchBytes = (size_t)QX_CUDA_LM_HEAD_STATIC_SCRATCH_BYTES;

// Lives in every device that loads this library, from module load until the process exits.
static __device__ __align__(256) unsigned char g_lm_head_scratch[kStaticScratchBytes];

// In host code `g_lm_head_scratch` is only a handle for the symbol; the address kernels can use
// has to be asked from the runtime, once per device, while that device is current.
static void* g_scratch_ptr[64] = {nullptr};
static std::mutex g_scratch_mutex;

static qx_status scratch_for_current_device(const char* op, void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess)
    return fail(QX_RUNTIME_ERROR, op, "no usable CUDA device (this backend has no CPU fallback)");
  if (dev < 0 || dev >= 64) return fail(QX_RUNTIME_ERROR, op, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_lm_head_scratch);
    if (e != cudaSuccess || !p) return fail(QX_RUNTIME_ERROR, op, cudaGetErrorString(e));
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return ok(op);
}

}  // namespace qx

using namespace qx;

extern "C" qx_status qx_cuda_lm_head_sample_q_noalloc(void* stream, const void* h, const void* wq,
                                                      const float* bias, int32_t* ids, int64_t T,
                                                      int64_t V, int64_t K, const char* format,
                                                      qx_dtype dtype, int mode, int topk,
                                                      double temperature, uint32_t seed,
                                                      double top_p) {
  static const char* op = "quantized_lm_head_sample.noalloc";
  // Everything the two stages keep in global memory besides inputs and outputs comes out of the
  // built-in array: the stage-1 partials, then the prepared hidden rows, their row scales and the
  // release flags; what is left serves as exchange slots for tiles shared between thread blocks
  // (with none left, tiles are simply not shared).  The K-dependent part makes the limit depend
  // on T * K as well as on T * tiles * k.
  if (T > 0 && V > 0 && K > 0) {
    const size_t need = qx_cuda_lm_head_workspace_bytes(T, V, K, mode, topk) - lm_head_scratch_full_bytes(T, K) +
                        lm_head_scratch_min_bytes(T, K);
    if (need > kStaticScratchBytes)
      return fail(QX_INSUFFICIENT_WORKSPACE, op,
                  "partials + prepared hidden rows exceed the built-in scratch "
                  "(QX_CUDA_LM_HEAD_STATIC_SCRATCH_BYTES); use qx_cuda_lm_head_sample_q with a "
                  "caller workspace");
  }
  void* scratch = nullptr;
  // Argument errors are reported before the device is touched; the shared body validates again.
  if (T > 0 && V > 0 && K > 0 && h && wq && ids) {
    const qx_status st = scratch_for_current_device(op, &scratch);
    if (st.code != QX_OK) return st;
  }
  return lm_head_sample_on(op, stream, h, wq, bias, ids, scratch, scratch ? kStaticScratchBytes : 0,
                           true, T, V, K, format, dtype, mode, topk, temperature, seed, top_p);
}
